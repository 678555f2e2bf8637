"""GPU parity: streaming kernels (through the C ABI) vs the CPU oracle, bit for bit."""

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

import lucid_b200 as L  # noqa: E402
import lucid_b200.quantization as Q  # noqa: E402
from gpu_util import dev, host, qd_of  # noqa: E402

PT_CASES = ["pt_s8", "pt_s8_b", "pt_s8_c", "pt_u8", "pt_sat", "pt_big"]


@pytest.mark.parametrize("name", PT_CASES)
def test_golden_per_tensor(golden, name):
    x = golden[f"{name}_x"]
    s = golden[f"{name}_scale"]
    z = float(golden[f"{name}_zp"])
    qmin, qmax = (int(v) for v in golden[f"{name}_qrange"])
    qd = qd_of(qmin, qmax)
    s_arg = float(s) if s.dtype == np.float64 else dev(s)  # python float or 0-d device tensor
    q = Q.quantize(dev(x), s_arg, z, qd)
    assert q.dtype == (torch.int16 if qmin >= 0 else torch.int8)
    assert np.array_equal(host(q), golden[f"{name}_q"])
    assert np.array_equal(host(Q.dequantize(q, s_arg, z)), golden[f"{name}_dq"])
    assert np.array_equal(host(Q.fake_quantize(dev(x), s_arg, z, qmin, qmax)), golden[f"{name}_fq"])


def test_golden_ties(golden):
    x = dev(golden["ties_x"])
    assert np.array_equal(host(Q.quantize(x, 0.5, 0.0, Q.qint8)), golden["ties_q"])
    assert np.array_equal(host(Q.quantize(x, 0.5, 3.0, Q.quint8)), golden["ties_q_u8"])


def test_golden_per_channel(golden):
    x, s, z = golden["pc_x"], dev(golden["pc_scale"]), dev(golden["pc_zp"])
    q = Q.quantize(dev(x), s, z, Q.qint8, ch_axis=0)
    assert np.array_equal(host(q), golden["pc_q"])
    assert np.array_equal(host(Q.dequantize(q, s, z, ch_axis=0)), golden["pc_dq"])
    assert np.array_equal(host(Q.fake_quantize(dev(x), s, z, -128, 127, ch_axis=0)), golden["pc_fq"])
    z1 = dev(golden["pc1_zp"])
    q1 = Q.quantize(dev(golden["pc1_x"]), s, z1, Q.quint8, ch_axis=1)
    assert q1.dtype == torch.int16
    assert np.array_equal(host(q1), golden["pc1_q"])
    assert np.array_equal(host(Q.dequantize(q1, s, z1, ch_axis=1)), golden["pc1_dq"])


@pytest.mark.parametrize("sname,scheme", [("aff", Q.per_tensor_affine), ("sym", Q.per_tensor_symmetric)])
@pytest.mark.parametrize("dname,qd", [("s8", Q.qint8), ("u8", Q.quint8), ("s4", Q.qint4)])
def test_golden_qparams(golden, sname, scheme, dname, qd):
    s, z = Q.calculate_qparams(dev(golden["qp_min"]), dev(golden["qp_max"]), scheme, qd)
    assert np.array_equal(host(s), golden[f"qp_{sname}_{dname}_scale"])
    assert np.array_equal(host(z), golden[f"qp_{sname}_{dname}_zp"])
    s0, z0 = Q.calculate_qparams(float(golden["qp_min"][0]), float(golden["qp_max"][0]), scheme, qd)
    assert s0.item() == golden[f"qp_{sname}_{dname}_scale"][0]


def test_golden_observers(golden):
    obs = Q.MinMaxObserver()
    obs(dev(golden["obs_xa"]))
    obs(dev(golden["obs_xb"]))
    assert obs.min_val.item() == golden["obs_min"] and obs.max_val.item() == golden["obs_max"]
    s, z = obs.calculate_qparams()
    assert s.item() == golden["obs_scale"] and z.item() == golden["obs_zp"]
    pobs = Q.PerChannelMinMaxObserver(ch_axis=0)
    pobs(dev(golden["obs_xa"]))
    assert np.array_equal(host(pobs.min_val), golden["pobs_min"])
    assert np.array_equal(host(pobs.max_val), golden["pobs_max"])
    ps, pz = pobs.calculate_qparams()
    assert np.array_equal(host(ps), golden["pobs_scale"]) and np.array_equal(host(pz), golden["pobs_zp"])


def test_reference_unit_values():
    # values of lucid/test/unit/quantization/test_functional.py
    q = Q.quantize(dev(np.array([-1000.0, 1000.0], np.float32)), 0.1, 0.0, Q.qint8)
    assert host(q).tolist() == [-128, 127]
    q = Q.quantize(dev(np.array([0.0], np.float32)), 0.02, 128.0, Q.quint8)
    assert q.dtype == torch.int16 and q.item() == 128
    x = np.array([-1.0, -0.3, 0.0, 0.7, 2.0], np.float32)
    q = Q.quantize(dev(x), 0.05, 0.0, Q.qint8)
    assert q.dtype == torch.int8
    assert np.allclose(host(Q.dequantize(q, 0.05, 0.0)), x, atol=1e-6)


def test_ste_gradient():
    xg = dev(np.array([-100.0, 0.2, 0.5, 100.0], np.float32)).requires_grad_(True)
    Q.fake_quantize(xg, 0.05, 0.0, -128, 127).sum().backward()
    assert host(xg.grad).tolist() == [0.0, 1.0, 1.0, 0.0]
    w = dev(np.array([[1.0, 2.0, 300.0], [-400.0, 0.5, 0.1]], np.float32)).requires_grad_(True)
    Q.fake_quantize(w, dev(np.array([0.02, 0.03], np.float32)), dev(np.zeros(2, np.float32)),
                    -128, 127, ch_axis=0).sum().backward()
    assert host(w.grad).tolist() == [[1.0, 1.0, 0.0], [0.0, 1.0, 1.0]]


# ---- config 1 at full size -----------------------------------------------------
@pytest.fixture(scope="module")
def c1():
    return np.random.default_rng(0).standard_normal((4096, 4096)).astype(np.float32)


@pytest.mark.parametrize("variant", ["narrow_127", "native_127_5"])
def test_config1_round_trip_bit_exact(c1, variant):
    x = dev(c1)
    if variant == "narrow_127":
        s_host = (np.abs(c1).max() / np.float32(127)).astype(np.float32)
        qd = Q.QDtype("qint8_narrow", 8, True, -127, 127, "int8")
        mn, mx = Q.minmax(x)
        absmax = torch.maximum(mn.abs(), mx.abs())
        s = absmax / 127
        assert s.item() == s_host
    else:
        obs = Q.MinMaxObserver(Q.per_tensor_symmetric, Q.qint8)
        obs(x)
        s, z = obs.calculate_qparams()
        mn, mx = O.minmax_observe(c1)
        s_host, z_host = O.calculate_qparams(mn, mx, True, O.QINT8)
        assert s.item() == s_host and z.item() == 0.0
        qd = Q.qint8
    q = Q.quantize(x, s, 0.0, qd)
    ref_q = O.quantize(c1, s_host, 0.0, (qd.name, 8, True, qd.quant_min, qd.quant_max, "int8"))
    assert np.array_equal(host(q), ref_q)
    xh = Q.dequantize(q, s, 0.0)
    assert np.array_equal(host(xh), O.dequantize(ref_q, s_host, 0.0))
    # size-independent properties: idempotence and fake_quantize == dequantize(quantize)
    assert torch.equal(Q.quantize(xh, s, 0.0, qd), q)
    assert torch.equal(Q.fake_quantize(x, s, 0.0, qd.quant_min, qd.quant_max), xh)
    # checksum of checksums against the oracle
    assert int(q.to(torch.int64).sum().item()) == int(ref_q.astype(np.int64).sum())


@pytest.mark.parametrize("shape", [(1,), (7,), (3, 5), (17, 33), (4, 16), (5, 1000), (2, 3, 4, 5), (0, 8)])
def test_odd_shapes_and_empty(shape):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(shape) * 2).astype(np.float32)
    q = Q.quantize(dev(x), 0.031, 7.0, Q.quint8)
    assert q.shape == torch.Size(shape)
    assert np.array_equal(host(q), O.quantize(x, 0.031, 7.0, O.QUINT8))
    dq = Q.dequantize(q, 0.031, 7.0)
    assert np.array_equal(host(dq), O.dequantize(host(q), 0.031, 7.0))


def test_unaligned_views():
    x = np.random.default_rng(4).standard_normal(4099).astype(np.float32)
    t = dev(x)[3:]  # 12-byte offset: the scalar path
    q = Q.quantize(t.clone()[0:4096], 0.02, 0.0, Q.qint8)
    assert np.array_equal(host(q), O.quantize(x[3:], 0.02, 0.0, O.QINT8))


@pytest.mark.parametrize("axis", [0, 1, 2, -1])
def test_per_channel_any_axis(axis):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 32, 16)).astype(np.float32)
    c = x.shape[axis]
    s = (np.abs(rng.standard_normal(c)) * 0.02 + 0.01).astype(np.float32)
    z = rng.integers(0, 255, c).astype(np.float32)
    q = Q.quantize(dev(x), dev(s), dev(z), Q.quint8, ch_axis=axis)
    assert np.array_equal(host(q), O.quantize(x, s, z, O.QUINT8, ch_axis=axis))
    dq = Q.dequantize(q, dev(s), dev(z), ch_axis=axis)
    assert np.array_equal(host(dq), O.dequantize(host(q), s, z, ch_axis=axis))
    fq = Q.fake_quantize(dev(x), dev(s), dev(z), 0, 255, ch_axis=axis)
    assert np.array_equal(host(fq), O.fake_quantize(x, s, z, 0, 255, ch_axis=axis))


def test_weight_encode_per_row_config2():
    w = (np.random.default_rng(1).standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    obs = Q.PerChannelMinMaxObserver(ch_axis=0)
    obs(dev(w))
    s, z = obs.calculate_qparams()
    q = Q.quantize(dev(w), s, z, Q.qint8, ch_axis=0)
    rq, rs, rz = O.quantize_weight_per_channel(w)
    assert np.array_equal(host(s), rs) and np.array_equal(host(z), rz)
    assert np.array_equal(host(q), rq)


@pytest.mark.parametrize("n", [1, 31, 4096, 100003, 1 << 22])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_minmax_per_tensor(n, dtype):
    x = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    t = dev(x).to(dtype)
    ref = t.float().cpu().numpy()
    for _ in range(3):  # the workspace re-arms itself between calls
        mn, mx = Q.minmax(t)
        assert mn.item() == ref.min() and mx.item() == ref.max()


@pytest.mark.parametrize("shape", [(5, 7), (64, 1000), (300, 4096), (9, 8192), (4, 28672)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_minmax_per_row(shape, dtype):
    x = np.random.default_rng(shape[1]).standard_normal(shape).astype(np.float32)
    t = dev(x).to(dtype)
    ref = t.float().cpu().numpy()
    mn, mx = Q.minmax(t, per_row=True)
    assert np.array_equal(host(mn), ref.min(axis=1)) and np.array_equal(host(mx), ref.max(axis=1))


@pytest.mark.parametrize("shape", [(3, 16), (100, 4096), (16, 11008), (5, 28672), (7, 100)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_token_encode(shape, dtype):
    x = np.random.default_rng(shape[0]).standard_normal(shape).astype(np.float32)
    t = dev(x).to(dtype)
    ref_in = t.float().cpu().numpy()
    q, s = Q.quantize_per_token(t, Q.qint8)
    rq, rs = O.per_token_quantize(ref_in)
    assert np.array_equal(host(s), rs)
    assert np.array_equal(host(q), rq)


def test_bf16_input_and_output():
    x = np.random.default_rng(9).standard_normal((64, 256)).astype(np.float32)
    t = dev(x).to(torch.bfloat16)
    xin = t.float().cpu().numpy()
    q = Q.quantize(t, 0.03, 0.0, Q.qint8)
    assert np.array_equal(host(q), O.quantize(xin, 0.03, 0.0, O.QINT8))
    dq = Q.dequantize(q, 0.03, 0.0, out_dtype=torch.bfloat16)
    assert np.array_equal(host(dq), O.bf16_round(O.dequantize(host(q), 0.03, 0.0)))


def test_cpu_tensor_is_rejected():
    import lucid_b200 as L

    with pytest.raises(L.DeviceMismatch):
        Q.quantize(torch.zeros(4), 0.1, 0.0, Q.qint8)


def _near_ties(rng, scale, n):
    """Inputs whose quotient by `scale` sits on or next to a .5 tie."""
    k = rng.integers(-300, 300, n).astype(np.float32)
    x = ((k + np.float32(0.5)) * np.float32(scale)).astype(np.float32)
    lo = np.nextafter(x, np.float32(-np.inf))
    hi = np.nextafter(x, np.float32(np.inf))
    return np.concatenate([x, lo, hi, np.nextafter(lo, np.float32(-np.inf)), np.nextafter(hi, np.float32(np.inf))])


def test_division_is_correctly_rounded_around_ties():
    """The kernels divide with a hoisted reciprocal plus residual corrections; the result
    must be the correctly rounded quotient everywhere, most visibly next to .5 ties."""
    rng = np.random.default_rng(21)
    for scale in np.exp(rng.uniform(np.log(1e-6), np.log(1e3), 40)).astype(np.float32):
        x = np.concatenate([_near_ties(rng, scale, 4096),
                            (rng.standard_normal(4096) * scale * 100).astype(np.float32)])
        x = x[: (x.size // 16) * 16].reshape(-1, 16)
        for qd, oqd, z in ((Q.qint8, O.QINT8, 0.0), (Q.quint8, O.QUINT8, 131.0)):
            got = host(Q.quantize(dev(x), float(scale), z, qd))
            assert np.array_equal(got, O.quantize(x, float(scale), z, oqd)), scale
        fq = host(Q.fake_quantize(dev(x), float(scale), 3.0, -128, 127))
        assert np.array_equal(fq, O.fake_quantize(x, float(scale), 3.0, -128, 127)), scale


def test_division_exact_per_channel_random_scales():
    rng = np.random.default_rng(22)
    rows, cols = 512, 1024
    s_col = np.exp(rng.uniform(np.log(1e-5), np.log(10.0), cols)).astype(np.float32)
    s_row = np.exp(rng.uniform(np.log(1e-5), np.log(10.0), rows)).astype(np.float32)
    k = rng.integers(-200, 200, (rows, cols)).astype(np.float32) + np.float32(0.5)
    for s, axis in ((s_col, 1), (s_row, 0)):
        sb = s.reshape(1, -1) if axis == 1 else s.reshape(-1, 1)
        x = (k * sb).astype(np.float32)
        x[::2] = np.nextafter(x[::2], np.float32(np.inf))
        x[1::4] = np.nextafter(x[1::4], np.float32(-np.inf))
        z = np.zeros_like(s)
        got = host(Q.quantize(dev(x), dev(s), dev(z), Q.qint8, ch_axis=axis))
        assert np.array_equal(got, O.quantize(x, s, z, O.QINT8, ch_axis=axis))


def test_extreme_scales_and_values_take_the_full_division():
    x = np.array([0.0, -0.0, 1e-45, -1e-40, 1e-30, 3.0e38, -3.0e38, 1.0, -1.0, 123.456, 1e20, -1e-20,
                  5e-39, 2.5, 3.5, -2.5], np.float32).reshape(1, 16)
    for scale in (1e-42, 1e-30, 1e-8, 1.0, 1e30, 3e38):
        got = host(Q.quantize(dev(x), float(scale), 0.0, Q.qint8))
        with np.errstate(over="ignore", divide="ignore"):
            ref = O.quantize(x, float(scale), 0.0, O.QINT8)
        assert np.array_equal(got, ref), scale


def test_back_to_back_dependent_launches_see_each_others_results():
    """The encode reads the grid that the range reduction launched just before it derived, and
    both kernels may become resident while their predecessor drains.  A long unsynchronised chain
    over inputs of alternating magnitude (all links share the reduction's workspace) must give
    every link the grid of ITS input."""
    rng = np.random.default_rng(29)
    shapes = [(1024, 1024), (96, 4096), (2048, 512)]
    xs = [(rng.standard_normal(shapes[i % 3]) * (0.01 if i % 2 else 37.0)).astype(np.float32) for i in range(6)]
    dx = [dev(x) for x in xs]
    outs = []
    for rep in range(40):
        for i, x in enumerate(dx):
            outs.append((i, *Q.quantize_dynamic_per_tensor(x, Q.quint8)))
    torch.cuda.synchronize()
    refs = {}
    for i, x in enumerate(xs):
        s, z = O.calculate_qparams(x.min(), x.max(), False, O.QUINT8)
        refs[i] = (O.quantize(x, s, z, O.QUINT8), np.float32(s), np.float32(z))
    for i, codes, s, z in outs:
        assert float(s) == refs[i][1] and float(z) == refs[i][2]
        assert np.array_equal(host(codes), refs[i][0])


def test_outliers_inside_a_large_tensor_and_ragged_last_span():
    """The per-tensor encode redoes only the spans that hold a value outside the short division's
    domain; the rest of the tensor, the spans next to them and a last span that is not whole must
    all equal the oracle."""
    rng = np.random.default_rng(23)
    for shape in ((37, 1028), (1024, 4096), (3, 16)):
        x = (rng.standard_normal(shape) * 3).astype(np.float32)
        flat = x.reshape(-1)
        pos = rng.choice(flat.size, size=min(64, flat.size // 2), replace=False)
        flat[pos] = rng.choice(np.array([1e30, -1e30, np.inf, -np.inf, 3e38, 1e9, -4.2e6 * 0.05, 4194304.0 * 0.05],
                                        np.float32), size=pos.size)
        for qd, oqd, z in ((Q.qint8, O.QINT8, 0.0), (Q.quint8, O.QUINT8, 131.0)):
            got = host(Q.quantize(dev(x), 0.05, z, qd))
            with np.errstate(over="ignore", invalid="ignore"):
                ref = O.quantize(x, 0.05, z, oqd)
            assert np.array_equal(got, ref), (shape, qd)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_shard_encode_with_broadcast_equals_unsharded_per_token_encode(dtype):
    """Column shards encoded separately with the all-reduced abs-max and stored into the
    slices of two destination buffers reproduce quantize_per_token of the whole tensor."""
    from lucid_b200.nn.quantized.sharded import quantize_shard_bcast, shard_absmax

    torch.manual_seed(4)
    rows, cols, shards = 257, 1024, 4
    x = (torch.randn(rows, cols, device="cuda") * torch.rand(rows, 1, device="cuda") * 3).to(dtype)
    x[5] = 0  # an all-zero token takes the eps scale
    want_codes, want_scales = Q.quantize_per_token(x, Q.qint8)
    per = cols // shards
    parts = [x[:, i * per:(i + 1) * per].contiguous() for i in range(shards)]
    # what the MAX all-reduce leaves on every rank
    am = torch.stack([shard_absmax(p) for p in parts]).max(dim=0).values
    bufs = [torch.full((rows, cols), 99, dtype=torch.int8, device="cuda") for _ in range(2)]
    for i, p in enumerate(parts):
        scales = quantize_shard_bcast(p, am, [b.data_ptr() for b in bufs], cols, i * per)
        assert torch.equal(scales, want_scales)
    assert torch.equal(bufs[0], want_codes) and torch.equal(bufs[1], want_codes)
    with pytest.raises(L.ShapeMismatch):
        quantize_shard_bcast(parts[0], am, [bufs[0].data_ptr()], cols, 3)  # column offset off the vector grid
