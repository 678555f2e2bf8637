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


@pytest.fixture(params=["auto", "pair", "single256"])
def tile_shape(request, monkeypatch):
    if request.param != "auto":
        monkeypatch.setenv("LQ_GEMM_SHAPE", request.param)
    return request.param


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
