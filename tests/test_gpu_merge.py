"""QFunctional merges and table-driven quantized activations on the GPU, against the oracle
and the fixtures made by executing the reference's functional_module.py."""

import numpy as np
import pytest
import torch

import lucid_b200 as L
import lucid_b200.nn.quantized as nnq
import lucid_b200.quantization as Q
from gpu_util import dev, host
from lucid_b200 import _lib
from lucid_b200.nn.quantized._utils import QCodes, codes_of, tag
from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu
F32 = np.float32


def _coded(codes, scale, zp):
    """A fake-quantized float tensor carrying its codes, as a quantized layer hands it over."""
    c = dev(codes)
    s, z = torch.tensor(scale, device="cuda"), torch.tensor(zp, device="cuda")
    return tag(Q.dequantize(c, s, z), QCodes(c, s, z))


@pytest.mark.parametrize("grid", ["u8", "s8"])
def test_qfunctional_golden(golden, grid):
    sc, zp, qmin, qmax = golden[f"qf_{grid}_grid"].tolist()
    qd = Q.quint8 if grid == "u8" else Q.qint8
    qf = nnq.QFunctional(sc, zp, qd).cuda()
    x = _coded(golden["qf_xq"].astype(np.uint8), 0.04, 120.0)  # quint8 codes arrive as int16 in the fixture
    y = _coded(golden["qf_yq"], 0.025, 0.0)
    for name, got in (("add", qf.add(x, y)), ("mul", qf.mul(x, y)), ("add_relu", qf.add_relu(x, y)),
                      ("add_scalar", qf.add_scalar(x, 0.75)), ("mul_scalar", qf.mul_scalar(x, -1.5)),
                      ("cat", qf.cat([x, y], dim=1))):
        want = golden[f"qf_{grid}_{name}"]
        assert np.array_equal(host(got), want), name
        qc = codes_of(got)
        assert qc is not None and qc.codes.dtype == (torch.uint8 if grid == "u8" else torch.int8)
        assert np.array_equal(host(Q.dequantize(qc.codes, qc.scale, qc.zero_point)), want), name
    # the same merges on untagged float operands (values instead of codes)
    xf, yf = x.detach().clone(), y.detach().clone()
    assert np.array_equal(host(qf.add(xf, yf)), golden[f"qf_{grid}_add"])
    assert np.array_equal(host(qf.add(dev(golden["qf_xraw"]), dev(golden["qf_yraw"]))),
                          golden[f"qf_{grid}_add_raw"])
    # mixed: one operand as codes, the other as values
    assert np.array_equal(host(qf.add_relu(x, yf)), golden[f"qf_{grid}_add_relu"])


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 65536 + 5])
@pytest.mark.parametrize("op", ["add", "mul", "add_relu"])
def test_qmerge_sizes_and_dtypes(n, op):
    g = np.random.default_rng(n)
    xq = g.integers(0, 256, n).astype(np.uint8)
    yq = g.integers(-128, 128, n).astype(np.int8)
    x, y = _coded(xq, 0.031, 97.0), _coded(yq, 0.017, 3.0)
    qf = nnq.QFunctional(0.045, 128.0, Q.quint8).cuda()
    want = O.qfunctional(op, O.dequantize(xq, 0.031, 97.0), O.dequantize(yq, 0.017, 3.0), 0.045, 128.0, 0, 255)
    assert np.array_equal(host(getattr(qf, op)(x, y)), want)
    # bfloat16 values as operands
    xb = dev((g.standard_normal(n)).astype(F32), torch.bfloat16)
    yb = dev((g.standard_normal(n)).astype(F32), torch.bfloat16)
    want = O.qfunctional(op, host(xb), host(yb), 0.045, 128.0, 0, 255)
    assert np.array_equal(host(getattr(qf, op)(xb, yb)), want)
    # an operand that starts off a 4-element boundary takes the scalar path
    if n > 8:
        got = getattr(qf, op)(xb.float()[1:], yb.float()[1:])
        assert np.array_equal(host(got), want[1:])


def test_qmerge_large_properties():
    """64 Mi elements: adding zero requantizes, requantizing to the operand's own grid is the
    identity on codes, and add commutes bit for bit."""
    g = torch.Generator(device="cuda").manual_seed(3)
    xq = torch.randint(0, 256, (1 << 26,), device="cuda", generator=g, dtype=torch.int32).to(torch.uint8)
    yq = torch.randint(0, 256, (1 << 26,), device="cuda", generator=g, dtype=torch.int32).to(torch.uint8)
    s, z = torch.tensor(0.02, device="cuda"), torch.tensor(128.0, device="cuda")
    x = tag(torch.empty(0), QCodes(xq, s, z))
    y = tag(torch.empty(0), QCodes(yq, s, z))
    same = nnq.QFunctional(0.02, 128.0, Q.quint8).cuda()
    out = same._merge(_lib.MERGE_COPY, x, None)
    assert torch.equal(codes_of(out).codes, xq)
    assert torch.equal(codes_of(same.add_scalar(x, 0.0)).codes, xq)
    a, b = same.add(x, y), same.add(y, x)
    assert torch.equal(codes_of(a).codes, codes_of(b).codes) and torch.equal(a, b)
    part = slice(0, 1 << 20)
    want = O.qfunctional("add", O.dequantize(host(xq[part]), 0.02, 128.0), O.dequantize(host(yq[part]), 0.02, 128.0),
                         0.02, 128.0, 0, 255)
    assert np.array_equal(host(a[part]), want)


def test_qmerge_rejects():
    qf = nnq.QFunctional(0.1, 0.0).cuda()
    with pytest.raises(L.DeviceMismatch):
        qf.add(torch.zeros(4), torch.zeros(4))
    with pytest.raises(L.ShapeMismatch):
        qf.add(torch.zeros(4, device="cuda"), torch.zeros(5, device="cuda"))
    lib = _lib.load()
    one = torch.zeros(4, device="cuda")
    assert lib.lq_qmerge(9, _lib.ptr(one), 0, None, None, None, 0, None, None, 0.0, 4, _lib.ptr(one), _lib.ptr(one),
                         0, 255, None, 3, _lib.ptr(one), None) == 5
    assert lib.lq_qmerge(0, _lib.ptr(one), 0, None, None, None, 0, None, None, 0.0, 4, _lib.ptr(one), _lib.ptr(one),
                         0, 255, None, 3, None, None) == 3


ACTS = [(nnq.Sigmoid, torch.nn.Sigmoid(), {}), (nnq.Tanh, torch.nn.Tanh(), {}),
        (nnq.Hardswish, torch.nn.Hardswish(), {}), (nnq.Hardsigmoid, torch.nn.Hardsigmoid(), {}),
        (nnq.ELU, torch.nn.ELU(alpha=0.7), {"alpha": 0.7}),
        (nnq.LeakyReLU, torch.nn.LeakyReLU(0.2), {"negative_slope": 0.2})]


@pytest.mark.parametrize("cls,float_mod,attrs", ACTS)
@pytest.mark.parametrize("signed_in", [False, True])
def test_quantized_activation_table_equals_float_route(cls, float_mod, attrs, signed_in):
    """Codes in -> table lookup must equal the module's own float route (activation, then
    fake-quantize) on the decoded input, bit for bit, for every input code."""
    g = np.random.default_rng(5)
    n = 100_003
    codes = g.integers(-128, 128, n).astype(np.int8) if signed_in else g.integers(0, 256, n).astype(np.uint8)
    x = _coded(codes, 0.05, -3.0 if signed_in else 131.0)
    act = cls(1.0 / 128.0, 128.0, Q.quint8).cuda()
    for k, v in attrs.items():
        setattr(act, k, v)
    got = act(x)
    want = act(x.detach().clone())  # untagged: the float route
    assert torch.equal(got, want)
    qc = codes_of(got)
    assert qc is not None and torch.equal(Q.dequantize(qc.codes, qc.scale, qc.zero_point), got)
    # and that float route is the reference's composition: fake_quantize(act(x))
    ref = O.fake_quantize(host(float_mod(x.detach().clone())), 1.0 / 128.0, 128.0, 0, 255)
    assert np.array_equal(host(want), ref)


def test_residual_block_workflow():
    """prepare -> calibrate -> convert on a residual block: FloatFunctional becomes QFunctional,
    the standalone activation becomes its quantized form, codes flow from layer to layer."""
    torch.manual_seed(0)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.quant = Q.QuantStub()
            self.fc1 = torch.nn.Linear(64, 64)
            self.act = torch.nn.Hardswish()
            self.fc2 = torch.nn.Linear(64, 64)
            self.skip = nnq.FloatFunctional()
            self.dequant = Q.DeQuantStub()

        def forward(self, x):
            x = self.quant(x)
            y = self.fc2(self.act(self.fc1(x)))
            return self.dequant(self.skip.add_relu(y, x))

    model = Block().cuda()
    x = torch.randn(256, 64, device="cuda")
    y_float = model(x)
    prepared = Q.prepare(model)
    assert isinstance(prepared.skip.activation_post_process, Q.HistogramObserver)
    for _ in range(3):
        prepared(torch.randn(256, 64, device="cuda"))
    prepared(x)
    qmodel = Q.convert(prepared)
    assert type(qmodel.skip) is nnq.QFunctional and type(qmodel.act) is nnq.Hardswish
    y_q = qmodel(x)
    err = float((y_q - y_float).abs().mean() / y_float.abs().mean())
    assert err < 0.08, err
    # every hop inside the quantized region handed codes over
    seen = []
    qmodel.skip.add_relu = (lambda f: lambda a, b: (seen.append((codes_of(a) is not None, codes_of(b) is not None)),
                                                    f(a, b))[1])(qmodel.skip.add_relu)
    qmodel(x)
    assert seen == [(True, True)]
