"""Host logic of the quantization workflows on the CPU: what ``prepare`` / ``prepare_qat`` swap,
what ``convert`` builds from calibrated and trained modules, where each grid ends up.

The C ABI is replaced for the duration of each test by the NumPy stand-in of
``tests/abi_standin.py`` and the engine is ``"reference"`` (layers run the reference's float
sequence), so these tests say nothing about the kernels -- the GPU tests do that through the
real library -- and everything about the Python that surrounds them.  Gates follow the
reference's own tests: lucid/test/unit/quantization/test_qat.py, test_qat_fused.py,
test_qat_convbn_ranks.py, test_static_ptq.py, test_graph_mode.py."""

import pytest
import torch

import abi_standin
import lucid_b200.nn.qat as nnqat
import lucid_b200.nn.quantized as nnq
import lucid_b200.quantization as Q
from lucid_b200.nn.intrinsic import qat as nniqat


@pytest.fixture(autouse=True)
def standin(monkeypatch):
    return abi_standin.install(monkeypatch)


def _rel(a, b):
    a, b = a.detach(), b.detach()
    return float((a - b).abs().mean() / b.abs().mean().clamp_min(1e-6))


def _minmax_qconfig():
    return Q.QConfig(activation=Q.MinMaxObserver, weight=Q.get_default_qconfig().weight)


def test_qat_trains_through_the_grids_and_converts():
    torch.manual_seed(0)
    model = torch.nn.Sequential(Q.QuantStub(), torch.nn.Linear(64, 128), torch.nn.ReLU(),
                                torch.nn.Linear(128, 32), Q.DeQuantStub())
    qat = Q.prepare_qat(model)
    assert type(qat[1]) is nnqat.Linear and isinstance(qat[1].weight_fake_quant, Q.FakeQuantize)
    assert isinstance(qat[0].activation_post_process, Q.FakeQuantize) and qat.training
    x = torch.randn(256, 64)
    target = model(x).detach() * 1.5
    opt = torch.optim.SGD(qat.parameters(), lr=1e-2)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(qat(x), target)
        loss.backward()
        assert torch.isfinite(qat[1].weight.grad).all()
        opt.step()
        losses.append(loss.item())
    assert all(b < a for a, b in zip(losses, losses[1:]))
    qat.eval()
    y_qat = qat(x)
    qmodel = Q.convert(qat)
    assert [type(m) for m in qmodel] == [nnq.Quantize, nnq.Linear, nnq.ReLU, nnq.Linear, nnq.DeQuantize]
    assert qmodel[1].weight_int8.dtype == torch.int8 and "weight" not in qmodel[1].state_dict()
    assert float(qmodel[0].scale) == float(qat[0].activation_post_process.scale)
    assert float(qmodel[1].scale) == float(qat[1].activation_post_process.scale)
    # under the reference engine the converted model IS what QAT simulated
    assert _rel(qmodel(x), y_qat) < 1e-6


@pytest.mark.parametrize("rank", [1, 2, 3])
def test_conv_bn_fusion_trains_and_converts(rank):
    conv_t = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)[rank - 1]
    bn_t = (torch.nn.BatchNorm1d, torch.nn.BatchNorm2d, torch.nn.BatchNorm3d)[rank - 1]
    torch.manual_seed(5 + rank)
    net = torch.nn.Sequential(Q.QuantStub(), conv_t(16, 32, 3, padding=1, bias=False), bn_t(32), torch.nn.ReLU(),
                              conv_t(32, 32, 3, stride=2, padding=1), bn_t(32), Q.DeQuantStub()).train()
    with torch.no_grad():
        for bn in (net[2], net[5]):
            bn.running_mean.normal_(0, 0.2)
            bn.running_var.uniform_(0.5, 1.5)
            bn.weight.uniform_(0.5, 1.5)
            bn.bias.normal_(0, 0.2)
    qcfg = Q.get_default_qat_qconfig()
    qat = Q.prepare_qat(Q.fuse_modules_qat(net, [["1", "2", "3"], ["4", "5"]], qcfg), qcfg)
    assert type(qat[1]) is getattr(nniqat, f"ConvBnReLU{rank}d") and type(qat[4]) is getattr(nniqat, f"ConvBn{rank}d")
    x = torch.randn(4, 16, *([10] * rank))
    opt = torch.optim.SGD(qat.parameters(), lr=1e-3)
    mean0 = qat[1].bn.running_mean.clone()
    for _ in range(2):
        opt.zero_grad()
        qat(x).square().mean().backward()
        assert qat[1].conv.weight.grad is not None and qat[1].bn.weight.grad is not None
        opt.step()
    assert not torch.equal(qat[1].bn.running_mean, mean0)  # the statistics kept learning
    qat.eval()
    with torch.no_grad():
        y_qat = qat(x)
    qnet = Q.convert(qat)
    assert type(qnet[1]) is getattr(nnq, f"ConvReLU{rank}d") and type(qnet[4]) is getattr(nnq, f"Conv{rank}d")
    w_fold, b_fold = qat[1]._fold()
    assert torch.equal(qnet[1].bias, b_fold.detach())
    w_hat = Q.dequantize(qnet[1].weight_int8, qnet[1].weight_scale, qnet[1].weight_zero_point, ch_axis=0)
    assert torch.equal(w_hat.reshape(w_fold.shape), qat[1].weight_fake_quant(w_fold.detach()))  # the FOLDED weight's grid
    assert qnet[1].state_dict()["weight_int8"].shape == w_fold.shape  # the reference's buffer shape
    with torch.no_grad():
        assert _rel(qnet(x), y_qat) < 1e-6


@pytest.mark.parametrize("rank", [1, 2, 3])
def test_fused_relu_layers_train_and_convert(rank):
    conv_t = (torch.nn.Conv1d, torch.nn.Conv2d, torch.nn.Conv3d)[rank - 1]
    torch.manual_seed(20 + rank)
    net = torch.nn.Sequential(Q.QuantStub(), conv_t(16, 32, 3, padding=1), torch.nn.ReLU(), conv_t(32, 16, 1),
                              torch.nn.Flatten(), torch.nn.LazyLinear(16), torch.nn.ReLU(), Q.DeQuantStub())
    x = torch.randn(4, 16, *([6] * rank))
    net(x)
    qcfg = Q.get_default_qat_qconfig()
    qat = Q.prepare_qat(Q.fuse_modules_qat(net, [["1", "2"], ["5", "6"]], qcfg), qcfg)
    assert [type(qat[i]) for i in (1, 3, 5)] == [getattr(nnqat, f"ConvReLU{rank}d"), getattr(nnqat, f"Conv{rank}d"),
                                                 nnqat.LinearReLU]
    qat(x).square().mean().backward()
    assert qat[1].weight.grad is not None and qat[5].weight.grad is not None
    qat.eval()
    with torch.no_grad():
        y_qat = qat(x)
    assert float(y_qat.min()) >= 0.0  # the fused ReLU sits ahead of the output grid
    assert float(qat[5].activation_post_process.zero_point) == 0.0  # so the grid covers [0, max] only
    qnet = Q.convert(qat)
    assert [type(qnet[i]) for i in (0, 1, 3, 5)] == [nnq.Quantize, getattr(nnq, f"ConvReLU{rank}d"),
                                                    getattr(nnq, f"Conv{rank}d"), nnq.LinearReLU]
    with torch.no_grad():
        assert _rel(qnet(x), y_qat) < 1e-6


def test_embedding_tables_convert_without_calibration_and_through_qat():
    torch.manual_seed(9)
    model = torch.nn.Sequential(torch.nn.Embedding(500, 64, padding_idx=0), torch.nn.Linear(64, 32))
    idx = torch.randint(0, 500, (4, 10))
    y = model(idx).detach()
    qstatic = Q.convert(model)
    assert type(qstatic[0]) is nnq.Embedding and type(qstatic[1]) is torch.nn.Linear
    assert _rel(qstatic(idx), y) < 0.02
    assert bool((qstatic[0](torch.tensor([0, 0])) == 0).all())  # the padding row reads as zeros
    qat = Q.prepare_qat(model)
    assert type(qat[0]) is nnqat.Embedding and type(qat[1]) is nnqat.Linear
    qat(idx).square().mean().backward()
    assert qat[0].weight.grad is not None
    qnet = Q.convert(qat.eval())
    assert type(qnet[0]) is nnq.Embedding and qnet[0].padding_idx == 0
    assert list(qnet[0].state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point"]
    assert qnet[0].weight_scale.shape == (500,)  # one scale per row
    assert _rel(qnet(idx), y) < 0.05


def test_static_ptq_with_a_mapping_leaves_the_excluded_head_in_float():
    """prepare -> calibrate -> convert with a QConfigMapping (lucid/quantization/_quantize.py:291-305;
    gates of test_static_ptq.py:60-99): stubs become Quantize / DeQuantize, the mapped layers become
    integer layers with the observed grids, the excluded one stays float, the checkpoint round-trips."""
    torch.manual_seed(3)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.quant, self.dequant = Q.QuantStub(), Q.DeQuantStub()
            self.fc1, self.act, self.fc2 = torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 16)
            self.head = torch.nn.Linear(16, 4)

        def forward(self, x):
            return self.head(self.dequant(self.fc2(self.act(self.fc1(self.quant(x))))))

    net = Net().eval()
    x = torch.randn(64, 32)
    mapping = Q.QConfigMapping().set_global(_minmax_qconfig()).set_module_name("head", None)
    fused = Q.fuse_modules(net, [["fc1", "act"]])
    prepared = Q.prepare(fused, mapping)
    with torch.no_grad():
        assert torch.equal(prepared(x), net(x))  # observers change nothing
    qnet = Q.convert(prepared)
    assert type(qnet.quant) is nnq.Quantize and type(qnet.dequant) is nnq.DeQuantize
    assert type(qnet.fc1) is nnq.LinearReLU and type(qnet.fc2) is nnq.Linear and type(qnet.head) is torch.nn.Linear
    lo, hi = float(x.min()), float(x.max())
    assert float(qnet.quant.scale) == pytest.approx((max(hi, 0) - min(lo, 0)) / 255, rel=1e-6)
    with torch.no_grad():
        y, y_q = net(x), qnet(x)
    assert _rel(y_q, y) < 0.05
    state = qnet.state_dict()
    assert {"fc1.weight_int8", "fc1.weight_scale", "fc1.weight_zero_point", "fc1.scale", "fc1.zero_point",
            "fc1.bias", "head.weight"} <= set(state)
    other = Q.prepare(Q.fuse_modules(Net().eval(), [["fc1", "act"]]), mapping)  # different weights and grids
    with torch.no_grad():
        other(x * 3)
    clone = Q.convert(other)
    with torch.no_grad():
        assert not torch.equal(clone(x), y_q)
    clone.load_state_dict(state)
    with torch.no_grad():
        assert torch.equal(clone(x), y_q)


def test_graph_mode_needs_no_hand_placed_stubs():
    """prepare_fx -> calibrate -> convert_fx (lucid/quantization/_quantize_fx.py; gates of
    test_graph_mode.py:20-60)."""
    torch.manual_seed(4)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).eval()
    x = torch.randn(128, 32)
    prepared = Q.prepare_fx(net, _minmax_qconfig(), example_inputs=x[:1])
    assert isinstance(prepared, nnq.QuantWrapper)
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert_fx(prepared)
    assert type(qnet.quant) is nnq.Quantize and type(qnet.dequant) is nnq.DeQuantize
    assert type(qnet.module[0]) is nnq.Linear and qnet.module[0].weight_int8.dtype == torch.int8
    with torch.no_grad():
        assert _rel(qnet(x), net(x)) < 0.05


def test_the_package_itself_has_no_cpu_path(monkeypatch):
    """Without the stand-in a CPU tensor is refused: the fixture is what makes the tests above run."""
    from lucid_b200 import _lib

    monkeypatch.undo()
    with pytest.raises(_lib.LucidError):
        Q.quantize(torch.randn(4, 4), 0.1, 0.0, Q.qint8)


def _steps_apart(y_a, y_b, scale):
    """Distance of two tensors on one output grid, in grid steps."""
    return torch.round((y_a - y_b) / scale).abs()


@pytest.mark.parametrize("fuse", [False, True])
def test_integer_linear_wiring_against_the_float_form(monkeypatch, fuse):
    """Engine "auto" over the stand-in: the stub's codes feed the first contraction, its output
    codes ride through the (code-preserving) ReLU into the second one, and what comes out equals
    the reference's float sequence on the same converted model up to isolated one-step
    differences -- i.e. scales, zero points, row sums and bias reach the epilogue in the right
    places.  (The rate and size of the differences is the gate the GPU tests apply to the
    kernels, lucid/test/unit/quantization/test_static_ptq.py:86.)"""
    from lucid_b200 import backends
    from lucid_b200.nn.quantized._utils import codes_of

    fake = abi_standin.install(monkeypatch, pose_as_cuda=True)  # the code-preserving ReLU reads codes off device tensors
    torch.manual_seed(11)
    model = torch.nn.Sequential(Q.QuantStub(), torch.nn.Linear(64, 128), torch.nn.ReLU(),
                                torch.nn.Linear(128, 32), Q.DeQuantStub()).eval()
    x = torch.randn(200, 64) + 0.3  # an asymmetric input range: a non-zero activation zero point
    if fuse:
        model = Q.fuse_modules(model, [["1", "2"]])
    prepared = Q.prepare(model, _minmax_qconfig())
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    assert float(qnet[0].zero_point) != 0.0
    with torch.no_grad():
        y_float_form = qnet(x)
        monkeypatch.setattr(backends.quantized, "_engine", "auto")
        assert qnet[1]._int8_ok() and qnet[3]._int8_ok()
        h = qnet[1](qnet[0](x))
        carried = codes_of(h)
        assert carried is not None and carried.codes.dtype == torch.uint8  # the layer hands its codes on
        assert torch.equal(Q.dequantize(carried.codes, carried.scale, carried.zero_point), h)
        before = fake.calls["gemm"]
        y_int = qnet(x)
        assert fake.calls["gemm"] == before + 2  # both layers took the integer route
    steps = _steps_apart(y_int, y_float_form, qnet[3].scale)
    assert float(steps.max()) <= 1.0 and float((steps > 0).float().mean()) < 2e-3
    assert _rel(y_int, model(x)) < 0.05


def test_dynamic_linear_wiring_against_the_float_form(monkeypatch):
    """``quantize_dynamic`` under engine "auto": the live-range encode, the contraction and the
    float epilogue reproduce the reference's float sequence (lucid/nn/quantized/dynamic/linear.py:84-99)."""
    from lucid_b200 import backends

    torch.manual_seed(12)
    model = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.ReLU(), torch.nn.Linear(96, 16)).eval()
    x = torch.randn(50, 64)
    qnet = Q.quantize_dynamic(model)
    assert type(qnet[0]) is nnq.dynamic.Linear and type(qnet[2]) is nnq.dynamic.Linear
    with torch.no_grad():
        y_float_form = qnet(x)
        monkeypatch.setattr(backends.quantized, "_engine", "auto")
        y_int = qnet(x)
        assert float((y_int - y_float_form).abs().max() / y_float_form.abs().max()) < 1e-5
        assert _rel(y_int, model(x)) < 0.03


@pytest.mark.parametrize("rank,stride,padding", [(2, 1, 1), (2, 2, "same1"), (1, 2, 2), (2, 1, 0)])
def test_integer_conv_wiring_against_the_float_form(monkeypatch, rank, stride, padding):
    """The convolution modules under engine "auto" over the stand-in: a stub with a non-zero zero
    point feeds NHWC (or, for 1-D, N-L-C) codes, padded taps hold the code of 0.0, grouped and
    strided geometries reach the kernel as the module states them, and the result equals the
    float sequence on the same converted model up to isolated one-step differences."""
    from lucid_b200 import backends

    fake = abi_standin.install(monkeypatch, pose_as_cuda=True)
    conv_t = (torch.nn.Conv1d, torch.nn.Conv2d)[rank - 1]
    same = padding == "same1"
    torch.manual_seed(30 + rank + stride)
    first = conv_t(16, 32, 3, stride=1 if same else stride, padding="same" if same else padding)
    net = torch.nn.Sequential(Q.QuantStub(), first, torch.nn.ReLU(),
                              conv_t(32, 32, 3, stride=stride, padding=1, groups=2), Q.DeQuantStub()).eval()
    x = torch.randn(3, 16, *([11] * rank)) + 0.4
    prepared = Q.prepare(Q.fuse_modules(net, [["1", "2"]]), _minmax_qconfig())
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    assert float(qnet[0].zero_point) != 0.0
    with torch.no_grad():
        y_float_form = qnet(x)
        monkeypatch.setattr(backends.quantized, "_engine", "auto")
        assert qnet[1]._int8_ok() and qnet[3]._int8_ok()
        y_int = qnet(x)
        assert fake.calls["conv"] >= 2  # both layers took the integer route
        y = net(x)
    assert y_int.shape == y.shape
    steps = _steps_apart(y_int, y_float_form, qnet[3].scale)
    assert float(steps.max()) <= 1.0 and float((steps > 0).float().mean()) < 2e-3
    assert _rel(y_int, y) < 0.06


@pytest.mark.parametrize("stride,pad,opad,groups", [(2, 1, 1, 1), (1, 0, 0, 2), (3, 2, 1, 1)])
def test_integer_conv_transpose_wiring_against_the_float_form(monkeypatch, stride, pad, opad, groups):
    """``ConvTranspose2d`` on the integer convolution (input codes laid at stride distance into a
    frame of the zero point's code, flipped / channel-swapped filters): the frame geometry and the
    filter re-layout are host code, checked here against the float sequence of the same module."""
    from lucid_b200 import backends

    fake = abi_standin.install(monkeypatch, pose_as_cuda=True)
    torch.manual_seed(40 + stride)
    net = torch.nn.Sequential(Q.QuantStub(),
                              torch.nn.ConvTranspose2d(32, 32, 3, stride, pad, opad, groups, True),
                              Q.DeQuantStub()).eval()
    x = torch.randn(2, 32, 7, 9) + 0.5
    prepared = Q.prepare(net, _minmax_qconfig())
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    assert type(qnet[1]) is nnq.ConvTranspose2d and float(qnet[0].zero_point) != 0.0
    with torch.no_grad():
        y_float_form = qnet(x)
        monkeypatch.setattr(backends.quantized, "_engine", "auto")
        y_int = qnet(x)
        assert fake.calls["conv"] >= 1  # the integer convolution ran
        y = net(x)
    assert y_int.shape == y.shape
    steps = _steps_apart(y_int, y_float_form, qnet[1].scale)
    assert float(steps.max()) <= 1.0 and float((steps > 0).float().mean()) < 2e-3
    assert _rel(y_int, y) < 0.05


class _Residual(torch.nn.Module):
    """conv -> relu -> conv, + identity, relu: the block whose merge ``FloatFunctional`` marks."""

    def __init__(self):
        super().__init__()
        self.quant, self.dequant = Q.QuantStub(), Q.DeQuantStub()
        self.conv1, self.relu1 = torch.nn.Conv2d(16, 16, 3, padding=1), torch.nn.ReLU()
        self.conv2 = torch.nn.Conv2d(16, 16, 3, padding=1)
        self.skip = nnq.FloatFunctional()
        self.act = torch.nn.Hardswish()

    def forward(self, x):
        x = self.quant(x)
        y = self.conv2(self.relu1(self.conv1(x)))
        return self.dequant(self.act(self.skip.add_relu(y, x)))


def test_residual_block_with_merge_and_activation_tables(monkeypatch):
    """A residual block end to end under engine "auto" over the stand-in: the merge reads both
    operands as codes (the identity straight from the stub, on another grid than the branch), the
    activation runs through its byte table, and the result equals the float sequence of the same
    converted model up to isolated one-step differences
    (lucid/nn/quantized/functional_module.py:230-258, activation.py:22-60)."""
    from lucid_b200 import backends

    fake = abi_standin.install(monkeypatch, pose_as_cuda=True)
    torch.manual_seed(50)
    net = _Residual().eval()
    x = torch.randn(2, 16, 9, 9) + 0.2
    prepared = Q.prepare(Q.fuse_modules(net, [["conv1", "relu1"]]), _minmax_qconfig())
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    assert type(qnet.skip) is nnq.QFunctional and type(qnet.act) is nnq.Hardswish
    with torch.no_grad():
        y_float_form = qnet(x)
        monkeypatch.setattr(backends.quantized, "_engine", "auto")
        y_int = qnet(x)
        y = net(x)
    assert fake.calls["conv"] >= 2 and (fake.calls["merge"] or fake.calls["lut2"]) and fake.calls["lut"] >= 1
    steps = _steps_apart(y_int, y_float_form, qnet.act.scale)
    assert float(steps.max()) <= 1.0 and float((steps > 0).float().mean()) < 5e-3
    assert _rel(y_int, y) < 0.06


def test_group_wise_engine_routes_the_linear_family(monkeypatch):
    """``engine = "mlx_group"`` (lucid/quantization/_quantize.py:116-179, lucid/backends/__init__.py:90-96):
    ``convert`` builds the weight-only layer for Linear / LinearReLU with the bit width of the
    qconfig's weight observer and the first of the group sizes 64, 128, 32 that divides
    ``in_features``; a layer none divides keeps the calibrated layer; ``quantize_dynamic`` routes by
    its ``dtype``.  Other modules are untouched by the engine."""
    from lucid_b200 import backends
    from lucid_b200.quantization import _qgemm
    from lucid_b200.quantization._quantize import _mlx_group_size

    assert [_mlx_group_size(k) for k in (64, 128, 192, 96, 32, 48, 100)] == [64, 64, 64, 32, 32, None, None]
    assert _qgemm.is_available() is False  # no CUDA device here; the call itself must work
    fake = abi_standin.install(monkeypatch, engine="mlx_group")
    assert backends.quantized.use_mlx() and not backends.quantized.use_int8()
    torch.manual_seed(60)
    net = torch.nn.Sequential(Q.QuantStub(), torch.nn.Linear(96, 128), torch.nn.ReLU(), torch.nn.Linear(128, 48),
                              torch.nn.Linear(48, 8), Q.DeQuantStub()).eval()
    x = torch.randn(20, 96)
    w4 = Q.QConfig(activation=Q.MinMaxObserver,
                   weight=Q.PerChannelMinMaxObserver.with_args(qdtype=Q.qint4, qscheme=Q.per_channel_symmetric))
    mapping = Q.QConfigMapping().set_global(_minmax_qconfig()).set_module_name("3", w4)
    prepared = Q.prepare(Q.fuse_modules(net, [["1", "2"]]), mapping)
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    first, second, third = qnet[1], qnet[3], qnet[4]
    assert type(first) is nnq.QuantizedLinearMLX and (first.bits, first.group_size, first.relu) == (8, 32, True)
    assert type(second) is nnq.QuantizedLinearMLX and (second.bits, second.group_size, second.relu) == (4, 64, False)
    assert type(third) is nnq.Linear  # 48 input features: no group size divides them
    assert second.packed_weight.shape == (48, 128 * 4 // 32) and second.scales.shape == (48, 2)
    with torch.no_grad():
        y, y_q = net(x), qnet(x)
    assert fake.calls["groupwise"] == 2
    assert _rel(y_q, y) < 0.25  # the 4-bit layer dominates the error
    dyn = Q.quantize_dynamic(torch.nn.Sequential(torch.nn.Linear(64, 16), torch.nn.Linear(48, 4)).eval())
    assert type(dyn[0]) is nnq.QuantizedLinearMLX and type(dyn[1]) is nnq.dynamic.Linear


class _CatMul(torch.nn.Module):
    """Two branches concatenated, a 1x1 mix, and a gate: cat / mul merges and a table activation."""

    def __init__(self):
        super().__init__()
        self.quant, self.dequant = Q.QuantStub(), Q.DeQuantStub()
        self.a, self.b = torch.nn.Conv2d(16, 16, 1), torch.nn.Conv2d(16, 16, 3, padding=1)
        self.join, self.gate = nnq.FloatFunctional(), nnq.FloatFunctional()
        self.sig, self.mix = torch.nn.Sigmoid(), torch.nn.Conv2d(32, 16, 1)

    def forward(self, x):
        x = self.quant(x)
        y = self.mix(self.join.cat([self.a(x), self.b(x)], dim=1))
        return self.dequant(self.gate.mul(y, self.sig(y)))


def _sweep_cases():
    seq, stub, unstub = torch.nn.Sequential, Q.QuantStub, Q.DeQuantStub
    return {
        "conv1d": (seq(stub(), torch.nn.Conv1d(16, 32, 5, padding=2), torch.nn.ReLU(), torch.nn.Conv1d(32, 16, 3, stride=2),
                       unstub()), (2, 16, 20), [["1", "2"]]),
        "conv3d": (seq(stub(), torch.nn.Conv3d(16, 16, 3, padding=1), torch.nn.ReLU(), unstub()), (2, 16, 5, 6, 7), [["1", "2"]]),
        "conv_transpose1d": (seq(stub(), torch.nn.ConvTranspose1d(16, 16, 3, 2), unstub()), (2, 16, 9), None),
        "conv_transpose3d": (seq(stub(), torch.nn.ConvTranspose3d(16, 8, 3, 2), unstub()), (2, 16, 4, 4, 4), None),
        "cat_mul_sigmoid": (_CatMul(), (2, 16, 8, 8), None),
        "activations": (seq(stub(), torch.nn.Linear(32, 32), torch.nn.Hardswish(), torch.nn.Linear(32, 32), torch.nn.Tanh(),
                            torch.nn.Linear(32, 32), torch.nn.ELU(), torch.nn.Linear(32, 32), torch.nn.LeakyReLU(0.1),
                            torch.nn.Linear(32, 16), torch.nn.Hardsigmoid(), unstub()), (40, 32), None),
        "depthwise": (seq(stub(), torch.nn.Conv2d(16, 16, 3, padding=1, groups=16), torch.nn.Conv2d(16, 32, 1), unstub()),
                      (2, 16, 8, 8), None),
        "reflect_padding": (seq(stub(), torch.nn.Conv2d(16, 16, 3, padding=1, padding_mode="reflect"), unstub()),
                            (2, 16, 8, 8), None),
    }


@pytest.mark.parametrize("engine", ["reference", "auto"])
@pytest.mark.parametrize("case", sorted(_sweep_cases()))
def test_every_module_family_converts_runs_and_round_trips(monkeypatch, case, engine):
    """fuse -> prepare -> calibrate -> convert -> state_dict round trip -> forward for each module
    family ``convert`` maps (lucid/quantization/_quantize.py:66-113), under the float engine and
    under the integer one (layers outside the integer kernels' reach -- depthwise, reflect padding,
    volumes, 1-D / 3-D transposed -- take their float route there)."""
    import warnings

    from lucid_b200 import backends

    abi_standin.install(monkeypatch, pose_as_cuda=True)
    torch.manual_seed(70)
    net, shape, fuse = _sweep_cases()[case]
    net.eval()
    x = torch.randn(*shape)
    prepared = Q.prepare(Q.fuse_modules(net, fuse) if fuse else net, _minmax_qconfig())
    with torch.no_grad():
        prepared(x)
    qnet = Q.convert(prepared)
    state = qnet.state_dict()
    assert not any(k.endswith(".weight") for k in state)  # float weights are gone
    qnet.load_state_dict(state)
    monkeypatch.setattr(backends.quantized, "_engine", engine)
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")  # layers outside the integer path say so once
        y, y_q = net(x), qnet(x)
    assert y_q.shape == y.shape and bool(torch.isfinite(y_q).all())
    assert _rel(y_q, y) < 0.05


def test_default_static_ptq_uses_the_histogram_observer():
    """``prepare(model)`` with no qconfig (lucid/quantization/qconfig.py:180-192): activations get a
    ``HistogramObserver``, weights a per-channel min/max one; after two calibration batches with
    different ranges the grids ``convert`` bakes are the ones the oracle derives from the same
    batches (state kept on the module, clip search on the host)."""
    import numpy as np

    from oracle import lucid_oracle as O

    torch.manual_seed(80)
    net = torch.nn.Sequential(Q.QuantStub(), torch.nn.Linear(32, 16), Q.DeQuantStub()).eval()
    prepared = Q.prepare(net)
    assert isinstance(prepared[0].activation_post_process, Q.HistogramObserver)
    assert isinstance(prepared[1].activation_post_process, Q.HistogramObserver)
    batches = [torch.randn(64, 32), torch.randn(64, 32) * 3 + 1]
    with torch.no_grad():
        for b in batches:
            prepared(b)
    qnet = Q.convert(prepared)
    state = None
    for b in batches:
        state = O.histogram_observe(b.numpy(), state, 2048)
    s, z = O.histogram_qparams(state[0], state[1], state[2], False, O.QUINT8)
    assert float(qnet[0].scale) == float(s) and float(qnet[0].zero_point) == float(z)
    obs = prepared[0].activation_post_process
    assert np.array_equal(obs.histogram.numpy(), state[2]) and float(obs.histogram.sum()) == 2 * 64 * 32
    with torch.no_grad():
        assert _rel(qnet(batches[1]), net(batches[1])) < 0.05


@pytest.mark.parametrize("layers,bidirectional,batch_first", [(1, False, False), (2, True, True)])
def test_dynamic_lstm_host_loop_against_the_float_layer(standin, layers, bidirectional, batch_first):
    """The weight-only LSTM (lucid/nn/quantized/dynamic/rnn.py:27-111): layer / direction / time
    loops, state hand-over and the reversed direction are host code around the cell kernel;
    with the decoded weights loaded into a float ``nn.LSTM`` the two must agree to rounding."""
    torch.manual_seed(90 + layers)
    lstm = torch.nn.LSTM(12, 16, layers, batch_first=batch_first, bidirectional=bidirectional).eval()
    model = torch.nn.Sequential()
    model.add_module("rnn", lstm)
    q = Q.quantize_dynamic(model).rnn
    assert type(q) is nnq.dynamic.LSTM and q.weight_ih_l0_int8.dtype == torch.int8
    twin = torch.nn.LSTM(12, 16, layers, batch_first=batch_first, bidirectional=bidirectional).eval()
    with torch.no_grad():
        for name, p in twin.named_parameters():
            p.copy_(q._weight(name)[1] if name.startswith("weight") else getattr(q, name))
    x = torch.randn(5, 7, 12)  # (batch, time, ...) or (time, batch, ...): both are 3-D
    h0 = torch.randn(layers * (2 if bidirectional else 1), 5 if batch_first else 7, 16)
    c0 = torch.randn_like(h0)
    with torch.no_grad():
        y, (h, c) = q(x, (h0, c0))
        y_t, (h_t, c_t) = twin(x, (h0, c0))
    n_dir = 2 if bidirectional else 1
    assert standin.calls["lstm_cell"] == layers * n_dir * (7 if batch_first else 5)
    for got, want in ((y, y_t), (h, h_t), (c, c_t)):
        assert got.shape == want.shape and float((got - want).abs().max()) < 1e-5
    with torch.no_grad():  # and the float layer it came from, to the weights' 8-bit grid
        assert _rel(y, lstm(x, (h0, c0))[0]) < 0.05
