"""Group-wise weight-only codes and the decode matmul against the CPU oracle, with the gates the
reference's own tests hold for this route (lucid/test/unit/quantization/test_real_gemm.py:28-92:
int8 within 2 % and int4 within 15 % of the float layer, the fused kernel within 1e-3 of the
dequantize-then-matmul path, the packed weight under half the float bytes, a state-dict round
trip)."""

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

import lucid_b200.nn.quantized as nnq  # noqa: E402
from gpu_util import dev, host  # noqa: E402
from lucid_b200 import _lib  # noqa: E402
from lucid_b200.quantization import _qgemm  # noqa: E402


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("group", [32, 64, 128])
def test_pack_and_unpack_equal_the_oracle(bits, group):
    rng = np.random.default_rng(bits + group)
    w = (rng.standard_normal((96, 512)) * 0.05).astype(np.float32)
    w[5, :group] = 0.125          # a constant group
    w[7, group:2 * group] = 0.0   # an all-zero group
    packed, scales, biases = _qgemm.quantize(dev(w), group_size=group, bits=bits)
    p_ref, s_ref, b_ref = O.groupwise_quantize(w, group, bits)
    assert packed.dtype == torch.int32 and tuple(packed.shape) == (96, 512 * bits // 32)
    assert np.array_equal(host(packed).view(np.uint32), p_ref)
    assert np.array_equal(host(scales), s_ref) and np.array_equal(host(biases), b_ref)
    w_hat = _qgemm.dequantize(packed, scales, biases, group_size=group, bits=bits)
    assert np.array_equal(host(w_hat), O.groupwise_dequantize(p_ref, s_ref, b_ref, group, bits))
    assert np.all(np.abs(host(w_hat) - w) <= np.repeat(s_ref, group, axis=1) * 0.5000001 + 1e-7)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 3, 8, 21])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_matmul_against_the_oracle(bits, m, dtype):
    rng = np.random.default_rng(10 * bits + m)
    n, k, group = 320, 1024, 64
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    packed, scales, biases = _qgemm.quantize(dev(w), group_size=group, bits=bits)
    xd = dev(x).to(dtype)
    y = _qgemm.quantized_matmul(xd, packed, scales, biases, group_size=group, bits=bits)
    assert y.dtype == dtype and tuple(y.shape) == (m, n)
    ref = O.groupwise_matmul_f64(host(xd.float()), host(packed).view(np.uint32), host(scales), host(biases), group, bits)
    tol = 1e-3 if dtype == torch.float32 else 2e-2 * float(np.abs(ref).max())
    assert float(np.abs(host(y.float()) - ref).max()) < tol
    # the reference's gate: the fused kernel agrees with dequantize -> float matmul
    if dtype == torch.float32:
        with _lib.ieee_float32():
            y_deq = xd @ _qgemm.dequantize(packed, scales, biases, group_size=group, bits=bits).T
        assert torch.allclose(y, y_deq, atol=1e-3)


@pytest.mark.parametrize("bits,gate", [(8, 0.02), (4, 0.15)])
def test_module_tracks_the_float_layer_and_round_trips(bits, gate):
    torch.manual_seed(bits)
    lin = torch.nn.Linear(256, 256).cuda().eval()
    x = torch.randn(16, 256, device="cuda")
    with torch.no_grad(), _lib.ieee_float32():
        yf = lin(x)
    q = nnq.QuantizedLinearMLX.from_float(lin, bits=bits)
    yq = q(x)
    assert float((yf - yq).abs().max() / (yf.abs().max() + 1e-9)) < gate
    packed_bytes = q.packed_weight.numel() * 4 + q.scales.numel() * 4 + q.biases.numel() * 4
    assert packed_bytes < 256 * 256 * 4 / 2
    q2 = nnq.QuantizedLinearMLX(256, 256, bits=bits).cuda()
    q2.load_state_dict(q.state_dict())
    assert torch.allclose(q2(x), yq, atol=1e-4)
    relu = nnq.QuantizedLinearMLX.from_float(lin, bits=bits, relu=True)
    assert torch.equal(relu(x), torch.relu(yq))


def test_the_route_reports_itself_available():
    assert _qgemm.is_available() is True


def test_bad_arguments_raise():
    w = torch.randn(8, 96, device="cuda")
    with pytest.raises(_lib.ShapeMismatch):
        _qgemm.quantize(w, group_size=64, bits=8)
    with pytest.raises(NotImplementedError):
        _qgemm.quantize(torch.randn(8, 128, device="cuda"), group_size=48, bits=8)
    with pytest.raises(NotImplementedError):
        _qgemm.quantize(torch.randn(8, 128, device="cuda"), group_size=64, bits=2)
    with pytest.raises(_lib.DeviceMismatch):
        _qgemm.quantize(torch.randn(8, 128), group_size=64, bits=8)


def test_convert_routes_linear_layers_under_the_group_wise_engine():
    """`backends.quantized.engine = "mlx_group"`: `convert` and `quantize_dynamic` turn Linear
    layers into the weight-only group-wise layer (test_real_gemm.py:95-140), a layer whose width
    no group size divides keeps its calibrated / dynamic form."""
    import lucid_b200.backends as backends
    import lucid_b200.quantization as Q

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.ReLU(), torch.nn.Linear(256, 80),
                                torch.nn.ReLU(), torch.nn.Linear(80, 16)).cuda().eval()
    x = torch.randn(8, 128, device="cuda")
    with torch.no_grad(), _lib.ieee_float32():
        y_float = model(x)
    old = backends.quantized.engine
    backends.quantized.engine = "mlx_group"
    try:
        prepared = Q.prepare(model)
        prepared(x)
        qmodel = Q.convert(prepared)
        dmodel = Q.quantize_dynamic(model)
    finally:
        backends.quantized.engine = old
    assert isinstance(qmodel[0], nnq.QuantizedLinearMLX) and isinstance(qmodel[2], nnq.QuantizedLinearMLX)
    assert isinstance(qmodel[4], nnq.Linear) and qmodel[0].group_size == 64 and qmodel[2].group_size == 64
    assert isinstance(dmodel[0], nnq.QuantizedLinearMLX) and isinstance(dmodel[4], nnq.dynamic.Linear)
    for m in (qmodel, dmodel):
        y = m(x)
        assert float((y - y_float).abs().max() / y_float.abs().max()) < 0.05
