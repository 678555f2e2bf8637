"""The oracle is pinned here: NumPy and C restatements against (1) fixtures made by
executing the reference's own Python sources (tests/golden/make_golden.py) and
(2) the known answers in the reference's unit tests
(lucid/test/unit/quantization/test_functional.py, test_observer.py, and the
docstring examples of lucid/quantization/_qparams.py)."""

import numpy as np
import pytest

from oracle import c_oracle as CO
from oracle import lucid_oracle as O

PT_CASES = ["pt_s8", "pt_s8_b", "pt_s8_c", "pt_u8", "pt_sat", "pt_big"]


@pytest.mark.parametrize("name", PT_CASES)
def test_per_tensor_against_reference_execution(golden, name):
    x = golden[f"{name}_x"]
    s = golden[f"{name}_scale"]
    z = float(golden[f"{name}_zp"])
    qmin, qmax = (int(v) for v in golden[f"{name}_qrange"])
    storage = "int16" if qmin == 0 else "int8"
    qd = ("t", 8, qmin < 0, qmin, qmax, storage)
    s = float(s) if s.dtype == np.float64 else s  # Python-float scales stay Python floats
    q = O.quantize(x, s, z, qd)
    assert q.dtype == golden[f"{name}_q"].dtype
    assert np.array_equal(q, golden[f"{name}_q"])
    assert np.array_equal(O.dequantize(q, s, z), golden[f"{name}_dq"])
    assert np.array_equal(O.fake_quantize(x, s, z, qmin, qmax), golden[f"{name}_fq"])
    assert np.array_equal(O.fake_quantize_ste_mask(x, s, z, qmin, qmax), golden[f"{name}_mask"])
    # C restatement agrees bit for bit
    s32 = np.float32(s)
    cq = CO.quantize(x, s32, z, 0, qmin, qmax, np.dtype(storage).type)
    assert np.array_equal(cq, golden[f"{name}_q"])
    assert np.array_equal(CO.dequantize(cq, s32, z, 0), golden[f"{name}_dq"])
    assert np.array_equal(CO.fake_quantize(x, s32, z, 0, qmin, qmax), golden[f"{name}_fq"])


def test_ties_round_half_to_even(golden):
    x = golden["ties_x"]
    assert np.array_equal(O.quantize(x, 0.5, 0.0, O.QINT8), golden["ties_q"])
    assert np.array_equal(O.quantize(x, 0.5, 3.0, O.QUINT8), golden["ties_q_u8"])
    # the property itself: k + 0.5 goes to the even neighbour
    k = np.arange(-100, 100)
    q = O.quantize(((k + 0.5) * 0.5).astype(np.float32), 0.5, 0.0, O.QINT8).astype(np.int64)
    assert np.all(q % 2 == 0)
    assert np.array_equal(CO.quantize(x.reshape(1, -1), 0.5, 0.0, 0, -128, 127)[0], golden["ties_q"])


def test_per_channel(golden):
    x, s, z = golden["pc_x"], golden["pc_scale"], golden["pc_zp"]
    q = O.quantize(x, s, z, O.QINT8, ch_axis=0)
    assert np.array_equal(q, golden["pc_q"])
    assert np.array_equal(O.dequantize(q, s, z, ch_axis=0), golden["pc_dq"])
    assert np.array_equal(O.fake_quantize(x, s, z, -128, 127, ch_axis=0), golden["pc_fq"])
    assert np.array_equal(CO.quantize(x, s, z, 1, -128, 127), golden["pc_q"])
    x1, z1 = golden["pc1_x"], golden["pc1_zp"]
    q1 = O.quantize(x1, s, z1, O.QUINT8, ch_axis=1)
    assert q1.dtype == np.int16
    assert np.array_equal(q1, golden["pc1_q"])
    assert np.array_equal(O.dequantize(q1, s, z1, ch_axis=1), golden["pc1_dq"])
    assert np.array_equal(CO.quantize(x1, s, z1, 2, 0, 255, np.int16), golden["pc1_q"])
    assert np.array_equal(CO.dequantize(q1, s, z1, 2), golden["pc1_dq"])


@pytest.mark.parametrize("sname,sym", [("aff", False), ("sym", True)])
@pytest.mark.parametrize("dname,qd", [("s8", O.QINT8), ("u8", O.QUINT8), ("s4", O.QINT4)])
def test_calculate_qparams(golden, sname, sym, dname, qd):
    mn, mx = golden["qp_min"], golden["qp_max"]
    s, z = O.calculate_qparams(mn, mx, sym, qd)
    assert np.array_equal(s, golden[f"qp_{sname}_{dname}_scale"])
    assert np.array_equal(z, golden[f"qp_{sname}_{dname}_zp"])
    assert np.array_equal(s, golden[f"qp_{sname}_{dname}_scale_scalar"])
    cs, cz = CO.calculate_qparams(mn, mx, sym, qd[2], qd[3], qd[4])
    assert np.array_equal(cs, s) and np.array_equal(cz, z)


def test_observers(golden):
    mn, mx = O.minmax_observe(golden["obs_xa"])
    mn, mx = O.minmax_observe(golden["obs_xb"], mn, mx)
    assert mn == golden["obs_min"] and mx == golden["obs_max"]
    s, z = O.calculate_qparams(mn, mx, False, O.QUINT8)
    assert s == golden["obs_scale"] and z == golden["obs_zp"]
    pmn, pmx = O.per_channel_minmax_observe(golden["obs_xa"], 0)
    assert np.array_equal(pmn, golden["pobs_min"]) and np.array_equal(pmx, golden["pobs_max"])
    ps, pz = O.calculate_qparams(pmn, pmx, True, O.QINT8)
    assert np.array_equal(ps, golden["pobs_scale"]) and np.array_equal(pz, golden["pobs_zp"])
    cmn, cmx = CO.minmax_rows(golden["obs_xa"])
    assert np.array_equal(cmn, pmn) and np.array_equal(cmx, pmx)


def test_dynamic_linear_module(golden):
    wq, ws, wz = O.quantize_weight_per_channel(golden["dyn_w"])
    assert np.array_equal(wq, golden["dyn_wq"])
    assert np.array_equal(ws, golden["dyn_ws"]) and np.array_equal(wz, golden["dyn_wz"])
    y = O.dynamic_linear_forward(golden["dyn_x"], wq, ws, wz, golden["dyn_b"])
    assert np.array_equal(y, golden["dyn_y"])  # same NumPy matmul on both sides
    x = golden["dyn_x"]
    xs, xz = O.calculate_qparams(x.min(), x.max(), False, O.QUINT8)
    assert xs == golden["dyn_xs"] and xz == golden["dyn_xz"]
    assert np.array_equal(O.quantize(x, xs, xz, O.QUINT8), golden["dyn_xq"])


def test_static_linear_module(golden):
    y = O.quantized_linear_forward(golden["dyn_x"], golden["dyn_wq"], golden["dyn_ws"],
                                   golden["dyn_wz"], golden["dyn_b"], golden["ql_os"],
                                   golden["ql_oz"])
    assert np.array_equal(y, golden["ql_y"])


def test_integer_form_matches_reference_float_form(golden):
    """The integer form the kernels compute equals the reference's float form up
    to SGEMM rounding (norm-wise 1e-6) on the reference-generated module case."""
    x = golden["dyn_x"]
    xs, xz = golden["dyn_xs"], golden["dyn_xz"]
    xq = O.quantize(x, xs, xz, O.QUINT8)
    wq, ws = golden["dyn_wq"], golden["dyn_ws"]
    acc = O.int_gemm_exact(xq, wq)
    assert np.array_equal(acc, CO.gemm_i8(xq.astype(np.uint8), wq))
    rs = wq.astype(np.int64).sum(axis=1)
    y = O.epilogue_f32(acc, xs, xz, rs, ws, golden["dyn_b"])
    ref = golden["dyn_y"]
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-6


# ---- known answers copied as VALUES from the reference's unit tests ----------

def test_reference_unit_known_answers():
    # test_functional.py: saturation
    assert O.quantize(np.array([-1000.0, 1000.0], np.float32), 0.1, 0.0, O.QINT8).tolist() == [-128, 127]
    # affine zero point
    q = O.quantize(np.array([0.0], np.float32), 0.02, 128.0, O.QUINT8)
    assert q.dtype == np.int16 and q.item() == 128
    # on-grid round trip
    x = np.array([-1.0, -0.3, 0.0, 0.7, 2.0], np.float32)
    q = O.quantize(x, 0.05, 0.0, O.QINT8)
    assert q.dtype == np.int8
    assert np.allclose(O.dequantize(q, 0.05, 0.0), x, atol=1e-6)
    # fake_quantize == dequantize(quantize)
    x = np.array([-1.0, -0.31, 0.0, 0.72, 2.0], np.float32)
    assert np.array_equal(O.fake_quantize(x, 0.05, 0.0, -128, 127),
                          O.dequantize(O.quantize(x, 0.05, 0.0, O.QINT8), 0.05, 0.0))
    # STE masks
    assert O.fake_quantize_ste_mask(np.array([-100.0, 0.2, 0.5, 100.0], np.float32),
                                    0.05, 0.0, -128, 127).tolist() == [0.0, 1.0, 1.0, 0.0]
    w = np.array([[1.0, 2.0, 300.0], [-400.0, 0.5, 0.1]], np.float32)
    m = O.fake_quantize_ste_mask(w, np.array([0.02, 0.03], np.float32), np.zeros(2, np.float32),
                                 -128, 127, ch_axis=0)
    assert m.tolist() == [[1.0, 1.0, 0.0], [0.0, 1.0, 1.0]]
    # per-channel error bound
    w = np.array([[1.0, 2.0, 3.0], [-4.0, 0.5, 0.1]], np.float32)
    sc = np.array([0.03, 0.05], np.float32)
    dq = O.dequantize(O.quantize(w, sc, np.zeros(2), O.QINT8, ch_axis=0), sc, np.zeros(2), ch_axis=0)
    assert (np.abs(dq - w) <= np.array([[0.015], [0.025]]) + 1e-6).all()


def test_reference_qparams_known_answers():
    s, z = O.calculate_qparams(-1.0, 3.0, False, O.QUINT8)
    assert s.item() == pytest.approx(4.0 / 255.0, rel=1e-5) and 0.0 <= z.item() <= 255.0
    s, z = O.calculate_qparams(-2.5, 2.0, True, O.QINT8)
    assert z.item() == 0.0 and s.item() > 0.0
    s, _ = O.calculate_qparams(0.0, 0.0, False, O.QINT8)
    assert s.item() > 0.0
    # _qparams.py docstring examples
    s, z = O.calculate_qparams(-2.0, 6.0, False, O.QUINT8)
    assert round(float(s), 4) == 0.0314 and int(z) == 64
    _, z = O.calculate_qparams(-0.8, 0.5, True, O.QINT8)
    assert int(z) == 0


def test_reference_observer_known_answers():
    mn, mx = O.minmax_observe(np.array([[-1.0, 2.0], [0.5, 3.0]], np.float32))
    mn, mx = O.minmax_observe(np.array([[-2.0, 1.0]], np.float32), mn, mx)
    assert mn == -2.0 and mx == 3.0
    pmn, pmx = O.per_channel_minmax_observe(np.array([[1.0, 2.0, 3.0], [-4.0, 0.5, 0.1]], np.float32))
    assert pmn.tolist() == [1.0, -4.0] and pmx.tolist() == [3.0, 0.5]


def test_bf16_helpers():
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    import torch

    ref = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(O.bf16_round(x), ref)
    assert np.array_equal(O.from_bf16_bits(O.to_bf16_bits(x)), ref)


def test_int_conv_matches_float_conv_on_codes():
    rng = np.random.default_rng(1)
    x = rng.integers(0, 255, (2, 6, 5, 8)).astype(np.uint8)
    w = rng.integers(-127, 127, (4, 3, 3, 8)).astype(np.int8)
    acc = O.int_conv2d_nhwc_exact(x, w, 1, 1)
    yf = O.conv2d_f32_nchw(x.transpose(0, 3, 1, 2).astype(np.float32),
                           w.transpose(0, 3, 1, 2).astype(np.float32), None, 1, 1)
    assert np.array_equal(acc, yf.transpose(0, 2, 3, 1).astype(np.int32))


def test_moving_average_observers(golden):
    mn, mx = np.inf, -np.inf
    cmn = cmx = None
    for i in range(3):
        x = golden[f"ma_x{i}"]
        mn, mx = O.moving_average_minmax_observe(x, mn, mx, c=0.05)
        assert mn == golden[f"ma_min{i}"] and mx == golden[f"ma_max{i}"]
        cmn, cmx = O.moving_average_per_channel_observe(x, 0, cmn, cmx, c=0.05)
        assert np.array_equal(cmn, golden[f"mac_min{i}"])
        assert np.array_equal(cmx, golden[f"mac_max{i}"])
    s, z = O.calculate_qparams(mn, mx, False, O.QUINT8)
    assert s == golden["ma_scale"] and z == golden["ma_zp"]
    s, z = O.calculate_qparams(cmn, cmx, True, O.QINT8)
    assert np.array_equal(s, golden["mac_scale"]) and np.array_equal(z, golden["mac_zp"])
    # lucid/test/unit/quantization/test_observer.py:34-39
    a = O.moving_average_minmax_observe(np.array([-2.0, 2.0]), np.inf, -np.inf, c=0.5)
    b = O.moving_average_minmax_observe(np.array([-4.0, 4.0]), *a, c=0.5)
    assert b == (-3.0, 3.0)


HIST_CASES = [("hg", 4, 2048, False, O.QUINT8), ("hs", 3, 128, True, O.QINT8),
              ("hc", 2, 256, False, O.QUINT8), ("hr", 2, 2048, False, O.QUINT8),
              ("ht", 1, 2048, False, O.QUINT8)]


@pytest.mark.parametrize("tag,batches,bins,sym,qd", HIST_CASES)
def test_histogram_observer(golden, tag, batches, bins, sym, qd):
    state = None
    for i in range(batches):
        state = O.histogram_observe(golden[f"{tag}_x{i}"], state, bins)
        assert np.array_equal(state[2], golden[f"{tag}_hist{i}"]), (tag, i)
        assert [state[0], state[1]] == golden[f"{tag}_range{i}"].tolist()
    clip = O.histogram_search_clip_range(state[0], state[1], state[2], qd[4] - qd[3])
    assert list(clip) == golden[f"{tag}_clip"].tolist()
    s, z = O.histogram_qparams(state[0], state[1], state[2], sym, qd)
    assert s == golden[f"{tag}_scale"] and z == golden[f"{tag}_zp"]


def test_histogram_observer_reference_properties(golden):
    """The two facts the reference's own tests assert
    (lucid/test/unit/quantization/test_observer.py:54-77)."""
    g = np.random.default_rng(0)
    x = g.standard_normal(2000).astype(np.float32)
    st = O.histogram_observe(x, None, 256)
    assert st[2].sum() == 2000
    data = np.concatenate([g.standard_normal(3000), g.uniform(5.0, 12.0, 150)]).astype(np.float32)
    st = O.histogram_observe(data, None, 512)
    s_h, _ = O.histogram_qparams(st[0], st[1], st[2], False, O.QUINT8)
    s_m, _ = O.calculate_qparams(*O.minmax_observe(data), False, O.QUINT8)
    assert s_h <= s_m
    # the heavy-tailed fixture really is clipped
    assert golden["ht_clip"][1] < golden["ht_range0"][1]


@pytest.mark.parametrize("tag", ["u8", "s8"])
def test_qfunctional_merges(golden, tag):
    sc, zp, qmin, qmax = golden[f"qf_{tag}_grid"].tolist()
    xf = O.dequantize(golden["qf_xq"], 0.04, 120.0)
    yf = O.dequantize(golden["qf_yq"], 0.025, 0.0)
    args = (sc, zp, int(qmin), int(qmax))
    assert np.array_equal(O.qfunctional("add", xf, yf, *args), golden[f"qf_{tag}_add"])
    assert np.array_equal(O.qfunctional("mul", xf, yf, *args), golden[f"qf_{tag}_mul"])
    assert np.array_equal(O.qfunctional("add_relu", xf, yf, *args), golden[f"qf_{tag}_add_relu"])
    assert np.array_equal(O.qfunctional("add", xf, 0.75, *args), golden[f"qf_{tag}_add_scalar"])
    assert np.array_equal(O.qfunctional("mul", xf, -1.5, *args), golden[f"qf_{tag}_mul_scalar"])
    assert np.array_equal(O.qfunctional("cat", xf, [yf], *args, dim=1), golden[f"qf_{tag}_cat"])
    assert np.array_equal(O.qfunctional("add", golden["qf_xraw"], golden["qf_yraw"], *args),
                          golden[f"qf_{tag}_add_raw"])


def test_fake_quantize_module(golden):
    """FakeQuantize.forward (lucid/quantization/_fake_quantize.py:182-199): observe, refresh the
    qparams, fake-quantize; a frozen observer keeps them."""
    mn, mx = np.inf, -np.inf
    for i in range(3):
        x = golden[f"fqm_x{i}"]
        mn, mx = O.moving_average_minmax_observe(x, mn, mx, c=0.1)
        s, z = O.calculate_qparams(mn, mx, False, O.QUINT8)
        assert [s, z] == golden[f"fqm_qp{i}"].tolist()
        assert np.array_equal(O.fake_quantize(x, s, z, 0, 255), golden[f"fqm_y{i}"])
    assert [s, z] == golden["fqm_qpwide"].tolist()
    assert np.array_equal(O.fake_quantize(golden["fqm_xwide"], s, z, 0, 255), golden["fqm_ywide"])
    ws, wz = O.calculate_qparams(*O.per_channel_minmax_observe(golden["fqm_w"]), True, O.QINT8)
    assert np.array_equal(ws, golden["fqm_wscale"]) and np.array_equal(wz, golden["fqm_wzp"])
    assert np.array_equal(O.fake_quantize(golden["fqm_w"], ws, wz, -128, 127, ch_axis=0), golden["fqm_wy"])


def test_c_restatement_of_histogram_and_merges(golden):
    """The plain-C restatements agree with the NumPy ones and with the reference-made fixtures."""
    g = np.random.default_rng(70)
    for n, bins, lo, hi in [(10_000, 2048, 0.0, 0.0), (5_000, 100, -1.5, 2.25), (333, 7, -0.1, 0.1),
                            (64, 16, 0.75, 0.75)]:
        x = (g.standard_normal(n) * 2).astype(np.float32)
        assert np.array_equal(CO.histc(x, bins, lo, hi), O.histc(x, bins, lo, hi))
    assert np.array_equal(CO.histc(np.full(9, 0.75, np.float32), 8, 0, 0), O.histc(np.full(9, 0.75), 8, 0, 0))
    # the fixtures' second batch widened the range: first histogram re-binned + second counts
    lo0, hi0 = golden["hg_range0"].tolist()
    lo1, hi1 = golden["hg_range1"].tolist()
    reb = CO.histogram_rebin(golden["hg_hist0"], lo0, hi0, lo1, hi1)
    assert np.array_equal(reb, O.histogram_rebin(golden["hg_hist0"], lo0, hi0, lo1, hi1))
    assert np.array_equal(CO.histc(golden["hg_x1"], 2048, lo1, hi1) + reb, golden["hg_hist1"])
    lo0, hi0 = golden["hc_range0"].tolist()  # a constant first batch: zero-width old range
    lo1, hi1 = golden["hc_range1"].tolist()
    assert np.array_equal(CO.histc(golden["hc_x1"], 256, lo1, hi1) +
                          CO.histogram_rebin(golden["hc_hist0"], lo0, hi0, lo1, hi1), golden["hc_hist1"])
    xf = O.dequantize(golden["qf_xq"], 0.04, 120.0)
    yf = O.dequantize(golden["qf_yq"], 0.025, 0.0)
    for tag in ("u8", "s8"):
        sc, zp, qmin, qmax = golden[f"qf_{tag}_grid"].tolist()
        for op in ("add", "mul", "add_relu"):
            assert np.array_equal(CO.qfunctional(op, xf, yf, sc, zp, int(qmin), int(qmax)), golden[f"qf_{tag}_{op}"])
        assert np.array_equal(CO.qfunctional("add", xf, 0.75, sc, zp, int(qmin), int(qmax)),
                              golden[f"qf_{tag}_add_scalar"])


def test_groupwise_codes_round_trip_and_packing():
    """Group-wise weight codes (formulas of lucid/quantization/_qgemm.py:84-97): the round-trip
    error stays within half a step, a constant group is exact, and the packing is little-endian."""
    rng = np.random.default_rng(3)
    w = rng.standard_normal((6, 256)).astype(np.float32)
    w[2, :64] = -0.75
    for bits in (4, 8):
        packed, s, b = O.groupwise_quantize(w, 64, bits)
        assert packed.shape == (6, 256 * bits // 32) and s.shape == (6, 4)
        w_hat = O.groupwise_dequantize(packed, s, b, 64, bits)
        assert np.all(np.abs(w_hat - w) <= np.repeat(s, 64, axis=1) * 0.5000001 + 1e-7)
        assert np.all(w_hat[2, :64] == np.float32(-0.75))
        codes = O.groupwise_codes(packed, bits)
        assert codes.max() <= (1 << bits) - 1
        assert int(packed[0, 0] & ((1 << bits) - 1)) == int(codes[0, 0])
        x = rng.standard_normal((3, 256)).astype(np.float32)
        ref = O.groupwise_matmul_f64(x, packed, s, b, 64, bits)
        assert np.allclose(ref, x.astype(np.float64) @ w_hat.astype(np.float64).T, atol=1e-5)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("group", [32, 64, 128])
def test_c_restatement_of_groupwise_codes(bits, group):
    """The two restatements of the group-wise codes (NumPy and plain C) agree bit for bit,
    constant groups and ties included."""
    rng = np.random.default_rng(100 * bits + group)
    w = rng.standard_normal((9, 4 * group)).astype(np.float32)
    w[1, :group] = 0.5                                   # constant group: scale 1, codes 0
    w[2, group:2 * group] = np.linspace(0, 1, group)     # an evenly spaced group
    w[3] = np.round(w[3] * 8) / 8                        # coarse values: exact ties after the divide
    packed, s, b = O.groupwise_quantize(w, group, bits)
    cpacked, cs, cb = CO.groupwise_quantize(w, group, bits)
    assert np.array_equal(packed, cpacked) and np.array_equal(s, cs) and np.array_equal(b, cb)
    assert np.array_equal(O.groupwise_dequantize(packed, s, b, group, bits),
                          CO.groupwise_dequantize(cpacked, cs, cb, group, bits))


@pytest.mark.parametrize("relu", [False, True])
def test_c_restatement_of_the_integer_linear(relu):
    """The north-star composition (per-token encode -> exact int32 accumulation -> f32 epilogue ->
    bf16 rounding or requantisation) in plain C equals the NumPy restatement bit for bit."""
    rng = np.random.default_rng(41 + relu)
    m, n, k = 37, 29, 96
    x = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    x[3] = 0.0                                            # an all-zero token: scale = eps
    x[5, :8] = [127.5, -127.5, 0.5, -0.5, 1.5, 2.5, -1.5, 63.75]  # ties after the divide (scale 1)
    x[5, 8:] = 0.0
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    w_scale = (rng.random(n) * 0.01 + 1e-3).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    q, s = O.per_token_quantize(x, O.QINT8)
    cq, cs = CO.per_token_quantize(x)
    assert np.array_equal(np.asarray(q, dtype=np.int8), cq) and np.array_equal(np.asarray(s, dtype=np.float32).reshape(-1), cs)
    acc = O.int_gemm_exact(cq, w)
    assert np.array_equal(acc, CO.int_gemm(cq, w))
    y = O.epilogue_f32(acc, cs, 0, None, w_scale, bias, relu=relu)
    assert np.array_equal(y, CO.linear_epilogue(acc, cs, w_scale, bias, relu=relu))
    assert np.array_equal(O.bf16_round(y), CO.linear_epilogue(acc, cs, w_scale, bias, relu=relu, out_bf16=True))
    for scale, zp, qmin, qmax in ((0.05, 128.0, 0, 255), (0.11, 0.0, -128, 127)):
        assert np.array_equal(O.requantize_f32(y, scale, zp, qmin, qmax), CO.requantize(y, scale, zp, qmin, qmax))
