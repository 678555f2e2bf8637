"""GPU parity: NHWC implicit-GEMM convolution vs the exact integer oracle."""

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

import lucid_b200.nn.quantized as nnq  # noqa: E402
import lucid_b200.quantization as Q  # noqa: E402
from gpu_util import dev, host  # noqa: E402
from lucid_b200 import _lib  # noqa: E402
from lucid_b200.nn.quantized import functional as QF  # noqa: E402


def _sync_status():
    _lib.check_device_status(torch.device("cuda", torch.cuda.current_device()))


CASES = [  # n, h, w, c, k, r, pad
    (2, 28, 28, 256, 256, 3, 1),
    (1, 8, 8, 16, 16, 3, 1),
    (3, 14, 14, 64, 96, 3, 1),
    (2, 7, 9, 32, 40, 3, 0),
    (2, 28, 28, 512, 256, 1, 0),
    (1, 5, 130, 16, 32, 3, 1),
    (2, 12, 12, 144, 272, 5, 2),
]


@pytest.fixture(params=["auto", "pair", "single256", "auto-sk", "pair-sk"])
def tile_shape(request, monkeypatch):
    """Tile policy of the contraction; `-sk` forces the stream-K schedule (tiles cut across CTAs)."""
    spec = request.param
    if spec.endswith("-sk"):
        spec = spec[:-3]
        monkeypatch.setenv("LQ_GEMM_STREAMK", "1")
    if spec != "auto":
        monkeypatch.setenv("LQ_GEMM_SHAPE", spec)
    _lib.load().lq_reload_env()
    yield spec
    monkeypatch.undo()
    _lib.load().lq_reload_env()


@pytest.mark.parametrize("n,h,w,c,k,r,pad", CASES)
@pytest.mark.parametrize("signed", [False, True])
def test_conv_accumulators_exact(n, h, w, c, k, r, pad, signed, tile_shape):
    rng = np.random.default_rng(n + h + c + k + r)
    x = rng.integers(-128 if signed else 0, 128 if signed else 256, (n, h, w, c)).astype(
        np.int8 if signed else np.uint8)
    wt = rng.integers(-128, 128, (k, r, r, c)).astype(np.int8)
    acc = QF.conv2d_nhwc_s8(dev(x), dev(wt), pad=pad, out_dtype=torch.int32)
    _sync_status()
    assert np.array_equal(host(acc), O.int_conv2d_nhwc_exact(x, wt, 1, pad))


def test_conv_stack_resnet_stage3_reduced(tile_shape):
    """Config-4 chain at batch 4: codes between layers bit-exact against the
    kernel-order epilogue on exact accumulators."""
    rng = np.random.default_rng(3)
    n, h, w = 4, 28, 28
    x = rng.standard_normal((n, h, w, 512)).astype(np.float32)
    s_in = np.float32(np.abs(x).max() / 127)
    codes = O.quantize(x, s_in, 0.0, O.QINT8)
    layers = [(512, 256, 1, 0), (256, 256, 3, 1), (256, 1024, 1, 0)]
    a_np, a_scale, a_dev = codes, s_in, dev(codes)
    for li, (cin, cout, r, pad) in enumerate(layers):
        wf = (rng.standard_normal((cout, r, r, cin)) * 0.05).astype(np.float32)
        b = (rng.standard_normal(cout) * 0.01).astype(np.float32)
        wq, ws, _ = O.quantize_weight_per_channel(wf.reshape(cout, -1))
        wq = wq.reshape(cout, r, r, cin)
        acc = O.int_conv2d_nhwc_exact(a_np, wq, 1, pad).reshape(-1, cout)
        y = O.epilogue_f32(acc, a_scale, 0, None, ws, b, relu=True)
        os_, oz = O.calculate_qparams(y.min(), y.max(), False, O.QUINT8)
        assert oz == 0.0  # post-ReLU affine grid: zero point is exactly 0
        ref = O.requantize_f32(y, os_, oz, 0, 255).astype(np.uint8).reshape(n, h, w, cout)
        out = QF.conv2d_nhwc_s8(a_dev, dev(wq), pad=pad, out_dtype=torch.uint8, a_scale=dev(a_scale),
                                b_scale=dev(ws), bias=dev(b), act=_lib.ACT_RELU, out_scale=dev(os_),
                                out_zp=dev(oz), qmin=0, qmax=255)
        _sync_status()
        assert np.array_equal(host(out), ref), f"layer {li}"
        a_np, a_scale, a_dev = ref, os_, out


def test_conv_module_matches_reference_float_form():
    rng = np.random.default_rng(5)
    conv = torch.nn.Conv2d(32, 48, 3, padding=1).cuda()
    x = rng.standard_normal((2, 32, 10, 10)).astype(np.float32)
    xs, xz = Q.calculate_qparams(float(x.min()), float(x.max()), Q.per_tensor_affine, Q.quint8)
    xin = nnq.Quantize(xs, xz, Q.quint8, nhwc=True)(dev(x))
    obs = Q.MinMaxObserver()
    obs(torch.relu(conv(xin)).contiguous())
    conv.activation_post_process = obs
    qm = nnq.ConvReLU2d.from_float(conv)
    y = qm(xin)  # non-zero input zero point with padding: the explicit-frame route
    _sync_status()
    y_ref = O.quantized_conv2d_forward(host(xin), host(qm.weight_int8), host(qm.weight_scale),
                                       host(qm.weight_zero_point), host(conv.bias.detach()),
                                       host(qm.scale), host(qm.zero_point), relu=True, pad=1)
    assert y.shape == (2, 48, 10, 10)
    diff = np.abs(host(y) - y_ref)
    assert (diff > 0).mean() < 2e-3 and diff.max() <= float(qm.scale) * 1.001
    # second layer consumes the first layer's codes (zero point 0 after ReLU)
    conv2 = torch.nn.Conv2d(48, 32, 3, padding=1).cuda()
    obs2 = Q.MinMaxObserver()
    obs2(conv2(y).contiguous())
    conv2.activation_post_process = obs2
    qm2 = nnq.Conv2d.from_float(conv2)
    y2 = qm2(y)
    _sync_status()
    y2_ref = O.quantized_conv2d_forward(host(y), host(qm2.weight_int8), host(qm2.weight_scale),
                                        host(qm2.weight_zero_point), host(conv2.bias.detach()),
                                        host(qm2.scale), host(qm2.zero_point), relu=False, pad=1)
    d2 = np.abs(host(y2) - y2_ref)
    assert (d2 > 0).mean() < 2e-3 and d2.max() <= float(qm2.scale) * 1.001


GEOMETRIES = [  # n, h, w, c, k, (r, s), stride, pad_lo, pad_hi, dilation, groups
    (2, 56, 56, 64, 128, (3, 3), (2, 2), (1, 1), (1, 1), (1, 1), 1),    # ResNet down-sampling 3x3
    (2, 56, 56, 64, 128, (1, 1), (2, 2), (0, 0), (0, 0), (1, 1), 1),    # ... and its 1x1 projection
    (1, 224, 224, 16, 64, (7, 7), (2, 2), (3, 3), (3, 3), (1, 1), 1),   # stem-shaped 7x7 stride 2
    (3, 15, 17, 32, 48, (3, 3), (2, 2), (1, 1), (1, 1), (1, 1), 1),     # odd H x W
    (2, 14, 14, 64, 96, (3, 3), (1, 1), (1, 1), (1, 1), (1, 1), 2),     # groups 2
    (2, 13, 13, 128, 128, (3, 3), (2, 2), (1, 1), (1, 1), (1, 1), 4),   # groups 4, stride 2, odd
    (1, 20, 20, 32, 32, (3, 3), (1, 1), (2, 2), (2, 2), (2, 2), 1),     # dilation 2
    (2, 12, 12, 16, 32, (4, 4), (1, 1), (1, 1), (2, 2), (1, 1), 1),     # "same" with an even kernel: asymmetric
    (1, 9, 40, 48, 16, (3, 5), (3, 2), (0, 2), (1, 2), (1, 1), 1),      # mixed strides / kernel / padding
    (1, 130, 300, 16, 16, (3, 3), (2, 2), (1, 1), (1, 1), (1, 1), 1),   # rows wider than one tile
]


@pytest.mark.parametrize("n,h,w,c,k,rs,stride,plo,phi,dil,groups", GEOMETRIES)
def test_conv_general_geometry_exact(n, h, w, c, k, rs, stride, plo, phi, dil, groups, tile_shape):
    """Stride, dilation, groups and asymmetric padding (what lucid/nn/quantized/conv.py:119-184
    accepts): accumulators bit-exact against the exact integer convolution."""
    rng = np.random.default_rng(h * 31 + w + c + k)
    x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8)
    wt = rng.integers(-128, 128, (k, rs[0], rs[1], c // groups)).astype(np.int8)
    ref = O.int_conv2d_nhwc_general(x, wt, stride, plo, phi, dil, groups)
    acc = QF.conv2d_nhwc_s8(dev(x), dev(wt), pad=plo, stride=stride, dilation=dil, groups=groups,
                            out_hw=ref.shape[1:3], out_dtype=torch.int32)
    _sync_status()
    assert acc.shape == ref.shape
    assert np.array_equal(host(acc), ref)


def test_conv_zero_point_inside_kernel():
    """A non-zero activation zero point with a geometry that reads no out-of-image tap takes the
    kernel's correction term (one launch, requantised codes out)."""
    rng = np.random.default_rng(21)
    n, h, w, c, k = 2, 12, 12, 32, 48
    x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8)
    wt = rng.integers(-128, 128, (k, 3, 3, c)).astype(np.int8)
    ws = (rng.random(k) * 1e-3 + 1e-4).astype(np.float32)
    b = (rng.standard_normal(k) * 0.1).astype(np.float32)
    zp, sa = np.float32(117), np.float32(0.02)
    acc = O.int_conv2d_nhwc_general(x, wt, (2, 2)).reshape(-1, k)
    rowsum = wt.reshape(k, -1).astype(np.int64).sum(axis=1).astype(np.int32)
    y = O.epilogue_f32(acc, sa, zp, rowsum, ws, b, relu=True)
    os_, oz = O.calculate_qparams(y.min(), y.max(), False, O.QUINT8)
    ref = O.requantize_f32(y, os_, oz, 0, 255).astype(np.uint8).reshape(n, 5, 5, k)
    out = QF.conv2d_nhwc_s8(dev(x), dev(wt), stride=2, out_dtype=torch.uint8, a_scale=dev(sa), a_zp=dev(zp),
                            b_rowsum=dev(rowsum), b_scale=dev(ws), bias=dev(b), act=_lib.ACT_RELU,
                            out_scale=dev(os_), out_zp=dev(oz), qmin=0, qmax=255)
    _sync_status()
    assert np.array_equal(host(out), ref)
    with pytest.raises(NotImplementedError):  # with padding the zero point must be 0
        QF.conv2d_nhwc_s8(dev(x), dev(wt), pad=1, out_dtype=torch.int32, a_zp=dev(zp), b_rowsum=dev(rowsum))


class _CountConv:
    """Counts calls of the library's float convolution while a block runs."""

    def __enter__(self):
        import torch.nn.functional as F

        self.n, self._orig = 0, F.conv2d

        def counted(*a, **k):
            self.n += 1
            return self._orig(*a, **k)

        F.conv2d = counted
        return self

    def __exit__(self, *exc):
        import torch.nn.functional as F

        F.conv2d = self._orig


def _resnet18_shaped_stack(gen):
    """The conv geometries of a ResNet-18 (stem 7x7/2, 3x3/1, 3x3/2 + 1x1/2 projections), 16-channel
    aligned and reduced in width, with unfused in-place ReLUs between some layers."""
    import torch.nn as nn

    def conv(ci, co, k, s, p):
        m = nn.Conv2d(ci, co, k, s, p)
        with torch.no_grad():
            m.weight.copy_(torch.randn(m.weight.shape, generator=gen) * (2.0 / (ci * k * k)) ** 0.5)
            m.bias.copy_(torch.randn(co, generator=gen) * 0.05)
        return m

    return nn.Sequential(
        Q.QuantStub(), conv(16, 32, 7, 2, 3), nn.ReLU(inplace=True),
        conv(32, 32, 3, 1, 1), nn.ReLU(inplace=True), conv(32, 32, 3, 1, 1), nn.ReLU(inplace=True),
        conv(32, 64, 3, 2, 1), nn.ReLU(inplace=True), conv(64, 64, 3, 1, 1),
        conv(64, 128, 1, 2, 0), nn.ReLU(inplace=True),
        conv(128, 128, 3, 2, 1), nn.ReLU(inplace=True), Q.DeQuantStub(),
    )


def test_resnet18_shaped_stack_runs_on_the_integer_path():
    """Reference gate lucid/test/unit/quantization/test_static_ptq.py:180-199 (a ResNet-18 through
    prepare / calibrate / convert): every convolution -- strided ones and unfused in-place ReLUs
    included -- runs the integer kernel (no call of the library's float convolution), and the
    result agrees with the reference's float route (engine "reference")."""
    import lucid_b200

    gen = torch.Generator().manual_seed(0)
    model = _resnet18_shaped_stack(gen).cuda().eval()
    x = torch.randn(2, 16, 64, 64, generator=gen).cuda()
    prepared = Q.prepare(model, Q.QConfig(activation=Q.MinMaxObserver, weight=Q.get_default_qconfig().weight))
    with torch.no_grad():
        prepared(x)
    qmodel = Q.convert(prepared)
    convs = [m for m in qmodel.modules() if isinstance(m, nnq.Conv2d)]
    assert len(convs) == 7 and all(c._int8_ok() for c in convs)
    with _CountConv() as counter, torch.no_grad():
        y = qmodel(x)
    _sync_status()
    assert counter.n == 0 and y.shape == (2, 128, 4, 4)
    # Layer by layer on the same input: the integer kernel against the reference's float route
    # (engine "reference": decode the weight, float convolution, fake-quantize).  The two differ
    # only where the float convolution's rounding moves a value across a grid edge: a tiny rate,
    # one code.  (Across a deep stack such flips compound, so the end-to-end rate says little.)
    t = x
    with torch.no_grad():
        for mod in qmodel:
            if isinstance(mod, nnq.Conv2d):
                lucid_b200.backends.quantized.engine = "reference"
                try:
                    y_ref = mod(t)
                finally:
                    lucid_b200.backends.quantized.engine = "auto"
                t = mod(t)
                diff = (t - y_ref).abs()
                assert float((diff > 0).float().mean()) < 1e-3, mod
                assert float(diff.max()) <= 1.001 * float(mod.scale), mod
            else:
                t = mod(t)
    assert torch.equal(t, y)
    _sync_status()


def test_inplace_ops_and_carried_codes():
    """quantized Conv2d -> nn.ReLU(inplace=True) -> quantized Conv2d.  An in-place op keeps the
    Python attribute that carries the first layer's codes but changes the values: stale codes must
    never be consumed.  The converted model's ReLU re-derives the codes of the rectified values
    (max(code, zero_point): exact); any other in-place op drops them, and the next layer encodes
    what the tensor holds now, as the reference (which only sees floats) does."""
    import lucid_b200
    from lucid_b200.nn.quantized._utils import codes_of

    gen = torch.Generator().manual_seed(1)
    c1 = torch.nn.Conv2d(16, 32, 3, padding=1)
    c2 = torch.nn.Conv2d(32, 16, 3, padding=1)
    model = torch.nn.Sequential(Q.QuantStub(), c1, torch.nn.ReLU(inplace=True), c2).cuda().eval()
    x = torch.randn(2, 16, 12, 12, generator=gen).cuda()
    prepared = Q.prepare(model, Q.QConfig(activation=Q.MinMaxObserver, weight=Q.get_default_qconfig().weight))
    with torch.no_grad():
        prepared(x)
    qmodel = Q.convert(prepared)
    assert type(qmodel[2]) is nnq.ReLU and qmodel[2].inplace
    with torch.no_grad():
        mid = qmodel[1](qmodel[0](x))
        qc = codes_of(mid)
        assert qc is not None and float(mid.min()) < 0
        codes_before = qc.codes.clone()
        out = qmodel[2](mid)
        assert out is mid and float(mid.min()) == 0.0
        qc2 = codes_of(mid)
        assert qc2 is not None and torch.equal(qc2.codes, torch.maximum(codes_before, qc.zero_point.to(torch.uint8)))
        assert torch.equal(Q.dequantize(qc2.codes, qc2.scale, qc2.zero_point).permute(0, 3, 1, 2), mid)
        y = qmodel(x)
        lucid_b200.backends.quantized.engine = "reference"
        try:
            y_ref = qmodel(x)
        finally:
            lucid_b200.backends.quantized.engine = "auto"
        diff = (y - y_ref).abs()
        assert float((diff > 0).float().mean()) < 5e-3 and float(diff.max()) <= 1.001 * float(qmodel[3].scale)
        # a functional in-place op the module layer cannot see: the codes are dropped, not reused
        mid = qmodel[1](qmodel[0](x))
        torch.relu_(mid)
        assert codes_of(mid) is None
        y_fn = qmodel[3](mid)  # encodes the rectified floats on their live 8-bit grid
        assert float((y_fn - y_ref).abs().mean() / y_ref.abs().mean()) < 0.02
        stale = qmodel[3](qmodel[1](qmodel[0](x)))  # what consuming the un-rectified codes would give
        assert float((stale - y_ref).abs().mean() / y_ref.abs().mean()) > 0.1
    _sync_status()


@pytest.mark.parametrize("cin,cout,k,stride,pad,opad,dil,groups", [
    (32, 48, 3, 2, 1, 1, 1, 1),    # the usual 2x up-sampling layer
    (32, 32, 4, 2, 1, 0, 1, 1),    # even kernel
    (64, 32, 3, 1, 0, 0, 1, 2),    # groups, stride 1
    (16, 16, 3, 3, 2, 2, 2, 1),    # stride 3, dilation 2
])
def test_conv_transpose2d_integer_route(cin, cout, k, stride, pad, opad, dil, groups):
    """nn.quantized.ConvTranspose2d (lucid/nn/quantized/conv_transpose.py:45-160) on the integer
    kernel: exact accumulators against the float transposed convolution of the codes evaluated in
    float64, and the module output against the reference's float route."""
    import lucid_b200

    torch.manual_seed(cin + k + stride)
    ct = torch.nn.ConvTranspose2d(cin, cout, k, stride, pad, opad, groups, True, dil).cuda()
    x = torch.randn(2, cin, 9, 11, device="cuda")
    xs, xz = Q.calculate_qparams(float(x.min()), float(x.max()), Q.per_tensor_affine, Q.quint8)
    xin = nnq.Quantize(xs, xz, Q.quint8)(x)
    obs = Q.MinMaxObserver()
    obs(ct(xin).detach().contiguous())
    ct.activation_post_process = obs
    qm = nnq.ConvTranspose2d.from_float(ct)
    assert qm._int8_ok()
    with _CountConvT() as counter:
        y = qm(xin)
    _sync_status()
    assert counter.n == 0 and y.shape == ct(xin).shape
    # exact integer accumulators: conv_transpose of (codes - zp) with the weight codes, in float64
    qc = xin._lq_codes
    a = (qc.codes.double() - float(xz)).permute(0, 3, 1, 2)
    acc_ref = torch.nn.functional.conv_transpose2d(a, qm.weight_int8.double(), None, stride, pad, opad, groups, dil)
    wk, rowsum, wscale = qm._weight_krsc()
    scale_k = (float(xs) * wscale.double()).reshape(1, -1, 1, 1)
    y_exact = acc_ref * scale_k + qm.bias.double().reshape(1, -1, 1, 1)
    codes_ref = torch.clamp(torch.round(y_exact / float(qm.scale)) + float(qm.zero_point), 0, 255)
    got = y._lq_codes.codes.permute(0, 3, 1, 2).double()
    assert float((got != codes_ref).double().mean()) < 1e-3 and float((got - codes_ref).abs().max()) <= 1
    lucid_b200.backends.quantized.engine = "reference"
    try:
        y_ref = qm(xin)
    finally:
        lucid_b200.backends.quantized.engine = "auto"
    diff = (y - y_ref).abs()
    assert float((diff > 0).float().mean()) < 1e-3 and float(diff.max()) <= 1.001 * float(qm.scale)


class _CountConvT:
    def __enter__(self):
        import torch.nn.functional as F

        self.n, self._orig = 0, F.conv_transpose2d

        def counted(*a, **k):
            self.n += 1
            return self._orig(*a, **k)

        F.conv_transpose2d = counted
        return self

    def __exit__(self, *exc):
        import torch.nn.functional as F

        F.conv_transpose2d = self._orig


@pytest.mark.parametrize("cin,cout,k,stride,pad,dil,groups", [(32, 48, 3, 1, 1, 1, 1), (64, 64, 5, 2, 2, 1, 2),
                                                              (16, 32, 3, 1, "same", 2, 1)])
def test_conv1d_integer_route_equals_float_form(cin, cout, k, stride, pad, dil, groups):
    """Conv1d on the implicit GEMM (a signal is a one-row image): the integer route and the
    reference's dequantize -> float conv -> fake-quantize route agree up to one output step at a
    few positions, and the state dict keeps the reference's 3-D weight."""
    import lucid_b200.backends as backends

    g = torch.Generator(device="cuda").manual_seed(cin + k)
    conv = torch.nn.Conv1d(cin, cout, k, stride=stride, padding=pad, dilation=dil, groups=groups).cuda()
    x0 = torch.randn(3, cin, 97, device="cuda", generator=g)
    xs, xz = Q.calculate_qparams(float(x0.min()), float(x0.max()), Q.per_tensor_affine, Q.quint8)
    x = nnq.Quantize(xs, xz, Q.quint8)(x0)  # on a grid, carrying its codes, like a stub's output
    with _lib.ieee_float32(), torch.no_grad():
        y_float = torch.relu(conv(x))
    obs = Q.MinMaxObserver()
    obs(y_float.contiguous())
    conv.activation_post_process = obs
    qm = nnq.ConvReLU1d.from_float(conv)
    assert qm.state_dict()["weight_int8"].shape == (cout, cin // groups, k)
    clone = nnq.ConvReLU1d(cin, cout, k, stride=stride, padding=0 if isinstance(pad, str) else pad, dilation=dil,
                           groups=groups).cuda()
    clone.load_state_dict(qm.state_dict())
    clone.padding_str, clone.out_qdtype = qm.padding_str, qm.out_qdtype
    y = qm(x)
    _sync_status()
    assert y.shape == y_float.shape and torch.equal(clone(x), y)
    old = backends.quantized.engine
    backends.quantized.engine = "reference"
    try:
        y_ref = qm(x)
    finally:
        backends.quantized.engine = old
    diff = (y - y_ref).abs()
    assert float((diff > 0).float().mean()) < 0.02 and float(diff.max()) <= float(qm.scale) * 1.001
    assert float((y - y_float).abs().max()) <= float(qm.scale) * 3


def test_conv3d_float_route_and_convert_mapping():
    g = torch.Generator(device="cuda").manual_seed(3)
    model = torch.nn.Sequential(Q.QuantStub(), torch.nn.Conv3d(8, 16, 3, padding=1), torch.nn.ReLU(), Q.DeQuantStub()).cuda()
    x = torch.randn(2, 8, 6, 10, 10, device="cuda", generator=g)
    prepared = Q.prepare(model)
    prepared(x)
    qmodel = Q.convert(prepared)
    assert isinstance(qmodel[1], nnq.Conv3d)
    with _lib.ieee_float32():
        y_float = model(x)
    y = qmodel(x)
    _sync_status()
    assert y.shape == y_float.shape
    assert float((y - y_float).abs().max()) <= 4 * float(qmodel[1].scale) + 4 * float(qmodel[0].scale)
