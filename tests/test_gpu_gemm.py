"""GPU parity: the tcgen05 integer contraction and its epilogues vs the oracle.

int32 accumulators and requantised codes are bit-exact; float outputs are
bit-exact against the oracle's kernel-order f32 epilogue and within 1e-6
(norm-wise: max|err| / max|y|) of the float64 evaluation of the same formula;
bf16 outputs equal the f32 result rounded once (tolerance 1e-2 vs float64)."""

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

import lucid_b200  # noqa: E402
import lucid_b200.nn.quantized as nnq  # noqa: E402
import lucid_b200.quantization as Q  # noqa: E402
from gpu_util import dev, host, rel_max  # noqa: E402
from lucid_b200 import _lib  # noqa: E402
from lucid_b200.nn.quantized import functional as QF  # noqa: E402


def _codes(rng, shape, signed=True, full_range=True):
    lo, hi = (-128, 128) if signed else (0, 256)
    if not full_range:
        lo, hi = (-127, 128) if signed else (0, 256)
    return rng.integers(lo, hi, shape).astype(np.int8 if signed else np.uint8)


def _sync_status():
    _lib.check_device_status(torch.device("cuda", torch.cuda.current_device()))


SHAPES = [(128, 128, 128), (128, 256, 128), (256, 512, 256), (1, 16, 16), (130, 200, 144),
          (77, 129, 4096), (384, 640, 1040), (512, 1024, 2048), (128, 96, 32), (300, 257, 48)]


@pytest.fixture(params=["auto", "pair", "single256", "single128", "pair-epi8", "pair-epi16",
                        "single256-epi8", "single256-epi16", "auto-sk", "pair-sk", "single256-sk",
                        "single128-sk", "pair-epi16-sk"])
def tile_shape(request, monkeypatch):
    """Forces the GEMM's tile policy (CTA pair 256x256 / single 128x256 / single 128x128), the
    epilogue build (8 or 16 epilogue warps) and the schedule (`-sk`: stream-K, i.e. tiles cut
    across CTAs and completed from partial sums, even for these small shapes)."""
    spec = request.param
    sk = spec.endswith("-sk")
    if sk:
        spec = spec[:-3]
        monkeypatch.setenv("LQ_GEMM_STREAMK", "1")
    shape, _, epi = spec.partition("-epi")
    if shape != "auto":
        monkeypatch.setenv("LQ_GEMM_SHAPE", shape)
    if epi:
        monkeypatch.setenv("LQ_GEMM_EPI_WARPS", epi)
    _lib.load().lq_reload_env()
    yield shape
    monkeypatch.undo()
    _lib.load().lq_reload_env()


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("a_signed", [True, False])
def test_accumulators_exact(m, n, k, a_signed, tile_shape):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a = _codes(rng, (m, k), a_signed)
    b = _codes(rng, (n, k), True)
    acc = QF.gemm_s8(dev(a), dev(b), out_dtype=torch.int32)
    _sync_status()
    assert np.array_equal(host(acc), O.int_gemm_exact(a, b))


def test_accumulator_extremes():
    # every product at its largest magnitude: |acc| = K * 128 * 128 and K * 255 * 128
    k = 8192
    a = np.full((128, k), -128, np.int8)
    b = np.full((256, k), -128, np.int8)
    acc = QF.gemm_s8(dev(a), dev(b), out_dtype=torch.int32)
    assert int(acc.min()) == int(acc.max()) == k * 128 * 128
    au = np.full((128, k), 255, np.uint8)
    acc = QF.gemm_s8(dev(au), dev(b), out_dtype=torch.int32)
    assert int(acc.min()) == int(acc.max()) == -k * 255 * 128
    _sync_status()


@pytest.mark.parametrize("m,n,k", [(2048, 3072, 1024), (4096, 4864, 512), (2176, 5120, 384)])
def test_many_tiles_persistent_schedule(m, n, k, tile_shape):
    # more tiles than SMs / clusters, several K blocks: exercises both TMEM stages, the ring
    # wrap-around and (paired) an odd number of M sub-tiles
    rng = np.random.default_rng(11)
    a, b = _codes(rng, (m, k)), _codes(rng, (n, k))
    acc = QF.gemm_s8(dev(a), dev(b), out_dtype=torch.int32)
    _sync_status()
    assert np.array_equal(host(acc), O.int_gemm_exact(a, b))


@pytest.mark.parametrize("m,n,k", [(4096, 1280, 8192), (4096, 1024, 8192), (4096, 1024, 28672), (2048, 4096, 4096),
                                   (4096, 2560, 8192)])
def test_stream_k_shard_shapes_bit_equal(m, n, k, monkeypatch):
    """The shapes whose tile count does not fill whole waves of SMs (the per-rank shards of the
    Llama-2-70B projections at 4 and 8 ranks, config 2): the stream-K schedule the policy picks
    for them gives the same bits as the tile-by-tile schedule, for raw accumulators and for the
    bf16 epilogue, and the accumulators equal torch's integer GEMM."""
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=g)
    b = torch.randint(-128, 128, (n, k), dtype=torch.int8, device="cuda", generator=g)
    sa = torch.rand(m, device="cuda", generator=g) * 1e-2
    sb = torch.rand(n, device="cuda", generator=g) * 1e-2
    acc = QF.gemm_s8(a, b, out_dtype=torch.int32)
    y = QF.gemm_s8(a, b, out_dtype=torch.bfloat16, a_scale=sa, b_scale=sb)
    monkeypatch.setenv("LQ_GEMM_STREAMK", "0")
    _lib.load().lq_reload_env()
    try:
        acc_dp = QF.gemm_s8(a, b, out_dtype=torch.int32)
        y_dp = QF.gemm_s8(a, b, out_dtype=torch.bfloat16, a_scale=sa, b_scale=sb)
    finally:
        monkeypatch.undo()
        _lib.load().lq_reload_env()
    _sync_status()
    assert torch.equal(acc, acc_dp) and torch.equal(y, y_dp)
    rows = torch.arange(0, m, 37, device="cuda")
    ref = (a[rows].double() @ b.double().T).to(torch.int32)
    assert torch.equal(acc[rows], ref)
    # the scratch is left clean: a second launch reuses it
    assert torch.equal(QF.gemm_s8(a, b, out_dtype=torch.int32), acc)
    _sync_status()


def test_concurrent_contractions_in_one_graph_use_their_own_scratch():
    """Two stream-K contractions forked over two streams inside one CUDA graph may run at the
    same time; each branch names its own workspace (`workspace_tag`), and the replayed results
    equal the eager ones."""
    g = torch.Generator(device="cuda").manual_seed(5)
    ops = []
    for m, n, k in ((4096, 1280, 8192), (4096, 1024, 8192)):  # both cut their partial wave across CTAs
        a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda", generator=g)
        b = torch.randint(-128, 128, (n, k), dtype=torch.int8, device="cuda", generator=g)
        ops.append((a, b, QF.gemm_s8(a, b, out_dtype=torch.int32), torch.empty((m, n), dtype=torch.int32, device="cuda")))
    side = torch.cuda.Stream()

    def both():
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(cur)
        with torch.cuda.stream(side), _lib.workspace_tag("side"):
            side.wait_event(fork)
            QF.gemm_s8(ops[1][0], ops[1][1], out_dtype=torch.int32, out=ops[1][3])
            join = torch.cuda.Event()
            join.record(side)
        QF.gemm_s8(ops[0][0], ops[0][1], out_dtype=torch.int32, out=ops[0][3])
        cur.wait_event(join)

    warm = torch.cuda.Stream()
    warm.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(warm):
        both()  # creates the workspaces eagerly
    torch.cuda.current_stream().wait_stream(warm)
    torch.cuda.synchronize()
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gph):
        both()
    for _ in range(5):
        for _, _, _, out in ops:
            out.zero_()
        gph.replay()
        torch.cuda.synchronize()
        assert all(torch.equal(out, ref) for _, _, ref, out in ops)
    _sync_status()


def _c2_like(m, k, n, seed=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.01).astype(np.float32)
    return x, w, b


def test_dynamic_linear_epilogue_f32_bit_exact():
    x, w, b = _c2_like(512, 1024, 768)
    wq, ws, wz = O.quantize_weight_per_channel(w)
    xs, xz = O.calculate_qparams(x.min(), x.max(), False, O.QUINT8)
    xq = O.quantize(x, xs, xz, O.QUINT8).astype(np.uint8)
    acc = O.int_gemm_exact(xq, wq)
    rowsum = wq.astype(np.int64).sum(axis=1).astype(np.int32)
    y_ref = O.epilogue_f32(acc, xs, xz, rowsum, ws, b)
    rs = QF.rowsum_s8(dev(wq))
    assert np.array_equal(host(rs), rowsum)
    y = QF.gemm_s8(dev(xq), dev(wq), out_dtype=torch.float32, a_scale=dev(xs), a_zp=dev(xz),
                   b_rowsum=rs, b_scale=dev(ws), bias=dev(b))
    _sync_status()
    assert np.array_equal(host(y), y_ref)
    assert rel_max(host(y), O.epilogue_f64(acc, xs, xz, rowsum, ws, b)) < 1e-6
    # and against the reference's own float form (dequantize -> f32 GEMM), norm-wise
    y_float = O.dynamic_linear_forward(x, wq, ws, wz, b)
    assert rel_max(host(y), y_float) < 2e-6


def test_dynamic_linear_module_matches_reference_fixture(golden):
    lin = torch.nn.Linear(64, 32).cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(golden["dyn_w"]))
        lin.bias.copy_(dev(golden["dyn_b"]))
    q = nnq.dynamic.Linear.from_float(lin)
    assert np.array_equal(host(q.weight_int8), golden["dyn_wq"])
    assert np.array_equal(host(q.weight_scale), golden["dyn_ws"])
    y = q(dev(golden["dyn_x"]))
    _sync_status()
    assert y.dtype == torch.float32
    assert rel_max(host(y), golden["dyn_y"]) < 1e-6


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_per_token_epilogue(out_dtype):
    rng = np.random.default_rng(5)
    m, k, n = 256, 512, 640
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    wq, ws, _ = O.quantize_weight_per_channel(w)
    xq, xs = O.per_token_quantize(x)
    acc = O.int_gemm_exact(xq, wq)
    y_ref = O.epilogue_f32(acc, xs, 0, None, ws, None)
    y = QF.gemm_s8(dev(xq), dev(wq), out_dtype=out_dtype, a_scale=dev(xs), b_scale=dev(ws))
    _sync_status()
    if out_dtype == torch.float32:
        assert np.array_equal(host(y), y_ref)
    else:
        assert np.array_equal(host(y), O.bf16_round(y_ref))
        assert rel_max(host(y), O.epilogue_f64(acc, xs, 0, None, ws, None)) < 1e-2


@pytest.mark.parametrize("unsigned_out,relu", [(True, True), (True, False), (False, False), (False, True)])
def test_requantising_epilogue_bit_exact(unsigned_out, relu, tile_shape):
    x, w, b = _c2_like(300, 256, 520, seed=7)
    wq, ws, _ = O.quantize_weight_per_channel(w)
    xs, xz = O.calculate_qparams(x.min(), x.max(), False, O.QUINT8)
    xq = O.quantize(x, xs, xz, O.QUINT8).astype(np.uint8)
    acc = O.int_gemm_exact(xq, wq)
    rowsum = wq.astype(np.int64).sum(axis=1).astype(np.int32)
    y = O.epilogue_f32(acc, xs, xz, rowsum, ws, b, relu=relu)
    qd = O.QUINT8 if unsigned_out else O.QINT8
    os_, oz = O.calculate_qparams(y.min(), y.max(), False, qd)
    ref = O.requantize_f32(y, os_, oz, qd[3], qd[4])
    out = QF.gemm_s8(dev(xq), dev(wq), out_dtype=torch.uint8 if unsigned_out else torch.int8,
                     a_scale=dev(xs), a_zp=dev(xz), b_rowsum=dev(rowsum), b_scale=dev(ws),
                     bias=dev(b), act=_lib.ACT_RELU if relu else _lib.ACT_NONE,
                     out_scale=dev(os_), out_zp=dev(oz), qmin=qd[3], qmax=qd[4])
    _sync_status()
    assert np.array_equal(host(out).astype(np.int32), ref.astype(np.int32))


@pytest.mark.parametrize("case", ["narrow_grid_relu", "zp_above_qmin_relu", "fractional_zp", "tiny_scale"])
def test_requantising_epilogue_corners_full_tiles(case):
    """N a multiple of the tile width (the kernel that holds the requantising loop alone): a grid
    narrower than the storage type, a ReLU whose floor is the zero point, and output grids outside
    the short division's domain (fractional zero point, subnormal scale), which every block
    answers through the full-range sequence."""
    x, w, b = _c2_like(300, 256, 512, seed=11)
    wq, ws, _ = O.quantize_weight_per_channel(w)
    xs, xz = O.calculate_qparams(x.min(), x.max(), False, O.QUINT8)
    xq = O.quantize(x, xs, xz, O.QUINT8).astype(np.uint8)
    acc = O.int_gemm_exact(xq, wq)
    rowsum = wq.astype(np.int64).sum(axis=1).astype(np.int32)
    relu = case in ("narrow_grid_relu", "zp_above_qmin_relu")
    y = O.epilogue_f32(acc, xs, xz, rowsum, ws, b, relu=relu)
    span = float(np.abs(y).max())
    os_, oz, qmin, qmax, store = {
        "narrow_grid_relu": (np.float32(span / 90), np.float32(0.0), -100, 100, torch.int8),
        "zp_above_qmin_relu": (np.float32(span / 100), np.float32(-20.0), -128, 127, torch.int8),
        "fractional_zp": (np.float32(span / 100), np.float32(2.5), -128, 127, torch.int8),
        "tiny_scale": (np.float32(3e-41), np.float32(0.0), 0, 255, torch.uint8),
    }[case]
    with np.errstate(over="ignore", invalid="ignore"):
        ref = O.requantize_f32(y, os_, oz, qmin, qmax)
    out = QF.gemm_s8(dev(xq), dev(wq), out_dtype=store, a_scale=dev(xs), a_zp=dev(xz), b_rowsum=dev(rowsum),
                     b_scale=dev(ws), bias=dev(b), act=_lib.ACT_RELU if relu else _lib.ACT_NONE,
                     out_scale=dev(os_), out_zp=dev(oz), qmin=qmin, qmax=qmax)
    _sync_status()
    assert np.array_equal(host(out).astype(np.int32), ref.astype(np.int32))


def test_static_linear_module_vs_reference_float_form(golden):
    """Module-level: mismatch rate against the reference's float path must be tiny
    and every mismatch +-1 code (the float GEMM's rounding, not ours)."""
    x, w, b = _c2_like(256, 512, 384, seed=9)
    lin = torch.nn.Linear(512, 384).cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(w))
        lin.bias.copy_(dev(b))
    obs = Q.MinMaxObserver()
    xin = nnq.Quantize(*[t for t in Q.calculate_qparams(float(x.min()), float(x.max()),
                                                         Q.per_tensor_affine, Q.quint8)])(dev(x))
    obs(torch.relu(lin(xin)))
    lin.activation_post_process = obs
    qm = nnq.LinearReLU.from_float(lin)
    y = qm(xin)
    _sync_status()
    assert y.dtype == torch.float32 and hasattr(y, "_lq_codes")
    # oracle: the reference's float sequence on the same fake-quantized input
    y_ref = O.quantized_linear_forward(host(xin), host(qm.weight_int8), host(qm.weight_scale),
                                       host(qm.weight_zero_point), b, host(qm.scale),
                                       host(qm.zero_point), relu=True)
    s = float(qm.scale)
    diff = np.abs(host(y) - y_ref)
    assert (diff > 0).mean() < 1e-3
    assert diff.max() <= s * 1.001
    # the engine switch routes to the float sequence and reproduces it
    lucid_b200.backends.quantized.engine = "reference"
    try:
        yf = qm(xin)
    finally:
        lucid_b200.backends.quantized.engine = "auto"
    d2 = np.abs(host(yf) - y_ref)
    assert (d2 > 0).mean() < 1e-3 and d2.max() <= s * 1.001


def test_gated_epilogue(tile_shape):
    if tile_shape == "single128":
        pytest.skip("gated tiles are 256 wide")
    rng = np.random.default_rng(13)
    m, k, f = 200, 256, 384
    x = rng.standard_normal((m, k)).astype(np.float32)
    wg = (rng.standard_normal((f, k)) * 0.05).astype(np.float32)
    wu = (rng.standard_normal((f, k)) * 0.05).astype(np.float32)
    gq, gs, _ = O.quantize_weight_per_channel(wg)
    uq, us, _ = O.quantize_weight_per_channel(wu)
    xq, xs = O.per_token_quantize(x)
    yg = O.epilogue_f32(O.int_gemm_exact(xq, gq), xs, 0, None, gs, None)
    yu = O.epilogue_f32(O.int_gemm_exact(xq, uq), xs, 0, None, us, None)
    ref = O.silu_f32(yg) * yu
    w_gu = nnq.dynamic.interleave_gate_up(dev(gq), dev(uq))
    s_gu = nnq.dynamic.interleave_gate_up(dev(gs), dev(us))
    h = QF.gemm_s8(dev(xq), w_gu, out_dtype=torch.float32, a_scale=dev(xs), b_scale=s_gu,
                   act=_lib.ACT_SILU_GATE)
    _sync_status()
    assert h.shape == (m, f)
    assert rel_max(host(h), ref) < 2e-6  # library exp differs in the last ulp
    hb = QF.gemm_s8(dev(xq), w_gu, out_dtype=torch.bfloat16, a_scale=dev(xs), b_scale=s_gu,
                    act=_lib.ACT_SILU_GATE)
    assert rel_max(host(hb), ref) < 1e-2


def test_config2_full_size_sampled_rows_and_linearity():
    x, w, b = _c2_like(2048, 4096, 4096, seed=1)
    lin = torch.nn.Linear(4096, 4096).cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(w))
        lin.bias.copy_(dev(b))
    q = nnq.dynamic.Linear.from_float(lin)
    y = q(dev(x))
    _sync_status()
    wq, ws = host(q.weight_int8), host(q.weight_scale)
    xs, xz = O.calculate_qparams(x.min(), x.max(), False, O.QUINT8)
    rows = np.random.default_rng(2).choice(2048, 96, replace=False)
    xq = O.quantize(x[rows], xs, xz, O.QUINT8).astype(np.uint8)
    acc = O.int_gemm_exact(xq, wq)
    rowsum = wq.astype(np.int64).sum(axis=1)
    y_ref = O.epilogue_f32(acc, xs, xz, rowsum, ws, b)
    assert np.array_equal(host(y)[rows], y_ref)
    # size-independent property: integer accumulators are linear in the activation codes
    a1 = _codes(np.random.default_rng(3), (2048, 4096), False) // 2
    a2 = _codes(np.random.default_rng(4), (2048, 4096), False) // 2
    wt = dev(wq)
    s1 = QF.gemm_s8(dev(a1), wt, out_dtype=torch.int32)
    s2 = QF.gemm_s8(dev(a2), wt, out_dtype=torch.int32)
    s12 = QF.gemm_s8(dev((a1 + a2).astype(np.uint8)), wt, out_dtype=torch.int32)
    _sync_status()
    assert torch.equal(s1 + s2, s12)


def test_bad_arguments_raise():
    a = torch.zeros((16, 24), dtype=torch.int8, device="cuda")
    b = torch.zeros((16, 24), dtype=torch.int8, device="cuda")
    with pytest.raises(lucid_b200.ShapeMismatch):  # K % 16 != 0 -> alignment class
        QF.gemm_s8(a, b)
    with pytest.raises(lucid_b200.ShapeMismatch):
        QF.gemm_s8(a, torch.zeros((16, 32), dtype=torch.int8, device="cuda"))
    with pytest.raises(lucid_b200.DtypeMismatch):
        QF.gemm_s8(a.float(), b)
    with pytest.raises(lucid_b200.DeviceMismatch):
        QF.gemm_s8(a.cpu(), b)
