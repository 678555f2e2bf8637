"""The BASELINE configurations at full size: sampled rows / images against the oracle plus
size-independent properties.  Config 1 and 2 live in test_gpu_stream.py / test_gpu_gemm.py."""

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

import lucid_b200.nn.quantized as nnq  # noqa: E402
import lucid_b200.quantization as Q  # noqa: E402
from gpu_util import dev, host, rel_max  # noqa: E402
from lucid_b200 import _lib  # noqa: E402
from lucid_b200.nn.quantized import functional as QF  # noqa: E402


def _status():
    _lib.check_device_status(torch.device("cuda", torch.cuda.current_device()))


def _exact_rows(xq, w, slab=4096):
    """O.int_gemm_exact with the weight taken in slabs of rows (bounds the float64 staging)."""
    return np.concatenate([O.int_gemm_exact(xq, w[n0:n0 + slab]) for n0 in range(0, w.shape[0], slab)], axis=1)


def test_config3_gated_mlp_bf16_full_size():
    """x (8 x 512 tokens, d = 4096) -> int8 gate/up 4096 -> 11008 (SiLU-gated) -> int8 down;
    bf16 in/out, per-channel weights ~ N(0, 0.02^2), per-token activation scales."""
    d, ff, m = 4096, 11008, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(8, 512, d, device="cuda", generator=g).to(torch.bfloat16)
    wg = torch.randn(ff, d, device="cuda", generator=g) * 0.02
    wu = torch.randn(ff, d, device="cuda", generator=g) * 0.02
    wd = torch.randn(d, ff, device="cuda", generator=g) * 0.02
    mlp = nnq.dynamic.GatedMLP.from_float(wg, wu, wd)
    y = mlp(x)
    _status()
    assert y.shape == (8, 512, d) and y.dtype == torch.bfloat16
    rows = np.random.default_rng(0).choice(m, 48, replace=False)
    xs = host(x.reshape(m, d))[rows]
    # weight codes as the module holds them, de-interleaved
    gu = host(mlp.gate_up_int8).reshape(ff // 128, 2, 128, d)
    gs = host(mlp.gate_up_scale).reshape(ff // 128, 2, 128)
    gq, uq = gu[:, 0].reshape(ff, d), gu[:, 1].reshape(ff, d)
    gsc, usc = gs[:, 0].reshape(ff), gs[:, 1].reshape(ff)
    rq, rs, _ = O.quantize_weight_per_channel(host(wg))
    assert np.array_equal(gq, rq) and np.array_equal(gsc, rs)
    xq, xsc = O.per_token_quantize(xs)
    yg = O.epilogue_f32(O.int_gemm_exact(xq, gq), xsc, 0, None, gsc, None)
    yu = O.epilogue_f32(O.int_gemm_exact(xq, uq), xsc, 0, None, usc, None)
    h = O.bf16_round(O.silu_f32(yg) * yu)
    hq, hsc = O.per_token_quantize(h)
    ref = O.epilogue_f32(O.int_gemm_exact(hq, host(mlp.down_int8)), hsc, 0, None, host(mlp.down_scale), None)
    got = host(y.reshape(m, d))[rows]
    assert rel_max(got, ref) < 1e-2
    # against the unquantized float MLP the int8 block stays within the usual PTQ error
    xf = torch.from_numpy(xs).cuda()
    yf = (torch.nn.functional.silu(xf @ wg.T) * (xf @ wu.T)) @ wd.T
    err = float((torch.from_numpy(got).cuda() - yf).abs().mean() / yf.abs().mean())
    assert err < 0.05


def test_config4_conv_stack_full_batch():
    """ResNet-50 stage-3 shaped stack on NHWC int8 codes, N = 64, 28 x 28, C = 512:
    1x1 512->256, 3x3 256->256 (pad 1), 1x1 256->1024, fused bias + ReLU + requantise."""
    rng = np.random.default_rng(4)
    n, h, w = 64, 28, 28
    x = rng.standard_normal((n, h, w, 512)).astype(np.float32)
    s_in = np.float32(np.abs(x).max() / 127)
    codes = O.quantize(x, s_in, 0.0, O.QINT8)
    layers = [(512, 256, 1, 0), (256, 256, 3, 1), (256, 1024, 1, 0)]
    sample = [0, 17, 63]  # images checked against the oracle
    a_dev, a_scale = dev(codes), s_in
    a_ref = codes[sample]
    for li, (cin, cout, r, pad) in enumerate(layers):
        wf = (rng.standard_normal((cout, r, r, cin)) * 0.05).astype(np.float32)
        b = (rng.standard_normal(cout) * 0.01).astype(np.float32)
        wq, ws, _ = O.quantize_weight_per_channel(wf.reshape(cout, -1))
        wq = wq.reshape(cout, r, r, cin)
        acc = O.int_conv2d_nhwc_exact(a_ref, wq, 1, pad).reshape(-1, cout)
        yr = O.epilogue_f32(acc, a_scale, 0, None, ws, b, relu=True)
        os_, oz = O.calculate_qparams(yr.min(), yr.max(), False, O.QUINT8)
        assert oz == 0.0
        ref = O.requantize_f32(yr, os_, oz, 0, 255).astype(np.uint8).reshape(len(sample), h, w, cout)
        out = QF.conv2d_nhwc_s8(a_dev, dev(wq), pad=pad, out_dtype=torch.uint8, a_scale=dev(a_scale),
                                b_scale=dev(ws), bias=dev(b), act=_lib.ACT_RELU, out_scale=dev(os_),
                                out_zp=dev(oz), qmin=0, qmax=255)
        _status()
        assert out.shape == (n, h, w, cout)
        assert np.array_equal(host(out[sample]), ref), f"layer {li}"
        # property: the batch is independent per image -> running the sampled images alone
        # reproduces the same codes
        alone = QF.conv2d_nhwc_s8(a_dev[sample].contiguous(), dev(wq), pad=pad, out_dtype=torch.uint8,
                                  a_scale=dev(a_scale), b_scale=dev(ws), bias=dev(b), act=_lib.ACT_RELU,
                                  out_scale=dev(os_), out_zp=dev(oz), qmin=0, qmax=255)
        assert torch.equal(alone, out[sample])
        a_dev, a_scale, a_ref = out, os_, ref


@pytest.mark.parametrize("name,n,k", [("qkv", 10240, 8192), ("o", 8192, 8192), ("down", 8192, 28672)])
def test_config5_llama70b_linears(name, n, k):
    """M = 4096 tokens, bf16 activations quantized per token, int8 per-channel weights."""
    m = 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    lin = nnq.dynamic.PerTokenLinear(k, n).cuda()
    for r0 in range(0, n, 2048):  # encode in slabs to bound the float staging
        wf = torch.randn(2048, k, device="cuda", generator=g) * 0.02
        obs = Q.PerChannelMinMaxObserver(ch_axis=0)
        obs(wf)
        s, z = obs.calculate_qparams()
        lin.weight_int8[r0:r0 + 2048] = Q.quantize(wf, s, z, Q.qint8, ch_axis=0)
        lin.weight_scale[r0:r0 + 2048] = s
    y = lin(x)
    _status()
    rows = np.random.default_rng(1).choice(m, 32, replace=False)
    xq, xs = O.per_token_quantize(host(x)[rows])
    acc = O.int_gemm_exact(xq, host(lin.weight_int8))
    ref = O.epilogue_f32(acc, xs, 0, None, host(lin.weight_scale), None)
    got = host(y)[rows]
    assert np.array_equal(got, O.bf16_round(ref))
    assert rel_max(got, O.epilogue_f64(acc, xs, 0, None, host(lin.weight_scale), None)) < 1e-2
    # properties at full size: exact accumulators are linear in the activation codes, and a
    # column permutation of the weight permutes the output columns
    a1 = torch.randint(-60, 60, (m, k), dtype=torch.int8, device="cuda", generator=g)
    a2 = torch.randint(-60, 60, (m, k), dtype=torch.int8, device="cuda", generator=g)
    w = lin.weight_int8
    s12 = QF.gemm_s8(a1 + a2, w, out_dtype=torch.int32)
    assert torch.equal(QF.gemm_s8(a1, w, out_dtype=torch.int32) + QF.gemm_s8(a2, w, out_dtype=torch.int32), s12)
    perm = torch.randperm(n, device="cuda", generator=g)
    assert torch.equal(QF.gemm_s8(a1, w[perm].contiguous(), out_dtype=torch.int32), QF.gemm_s8(a1, w, out_dtype=torch.int32)[:, perm])
    _status()


def test_config5_gate_up_full_size():
    """The gate / up projections of config 5 as the bench runs them: one GEMM over the
    [gate; up] weight interleaved in blocks of 128 rows (N = 2 x 28672), SiLU-gate epilogue, bf16
    out.  Sampled rows against the oracle (the SiLU goes through a library exp: 1e-2 relative on
    bf16), and the epilogue-free accumulators of the same operands bit for bit."""
    m, d, ff = 4096, 8192, 28672
    g = torch.Generator(device="cuda").manual_seed(55)
    x = torch.randn(m, d, device="cuda", generator=g).to(torch.bfloat16)
    w_gu = torch.empty((2 * ff, d), dtype=torch.int8, device="cuda")
    s_gu = torch.empty(2 * ff, dtype=torch.float32, device="cuda")
    slab = 2048
    for r0 in range(0, ff, slab):  # encode gate and up in slabs, interleaved as the kernel pairs them
        parts = []
        for _ in range(2):
            wf = torch.randn(slab, d, device="cuda", generator=g) * 0.02
            obs = Q.PerChannelMinMaxObserver(ch_axis=0)
            obs(wf)
            s, z = obs.calculate_qparams()
            parts.append((Q.quantize(wf, s, z, Q.qint8, ch_axis=0), s))
        w_gu[2 * r0:2 * (r0 + slab)] = nnq.dynamic.interleave_gate_up(parts[0][0], parts[1][0])
        s_gu[2 * r0:2 * (r0 + slab)] = nnq.dynamic.interleave_gate_up(parts[0][1], parts[1][1])
    a, sa = Q.quantize_per_token(x, Q.qint8)
    h = QF.gemm_s8(a, w_gu, out_dtype=torch.bfloat16, a_scale=sa, b_scale=s_gu, act=_lib.ACT_SILU_GATE)
    _status()
    assert h.shape == (m, ff)
    rows = np.random.default_rng(2).choice(m, 32, replace=False)
    xq, xs = O.per_token_quantize(host(x)[rows])
    assert np.array_equal(host(a)[rows], xq) and np.array_equal(host(sa)[rows], xs.astype(np.float32))
    gu = host(w_gu).reshape(ff // 128, 2, 128, d)
    gs = host(s_gu).reshape(ff // 128, 2, 128)
    yg = O.epilogue_f32(_exact_rows(xq, gu[:, 0].reshape(ff, d)), xs, 0, None, gs[:, 0].reshape(ff), None)
    yu = O.epilogue_f32(_exact_rows(xq, gu[:, 1].reshape(ff, d)), xs, 0, None, gs[:, 1].reshape(ff), None)
    assert rel_max(host(h)[rows], O.silu_f32(yg) * yu) < 1e-2
    rows_t = torch.from_numpy(np.sort(rows)).cuda()
    acc = QF.gemm_s8(a[rows_t].contiguous(), w_gu, out_dtype=torch.int32)
    assert np.array_equal(host(acc), _exact_rows(host(a)[np.sort(rows)], host(w_gu)))
    _status()
