"""Calibration observers on the GPU against the oracle and the fixtures made by executing the
reference's observer.py: histc (bit-equal counts), the histogram observer's range growth,
re-binning, clip search and qparams, and the moving-average observers."""

import io

import numpy as np
import pytest
import torch

import lucid_b200 as L
import lucid_b200.quantization as Q
from gpu_util import dev, host
from oracle import lucid_oracle as O
from test_oracle_golden import HIST_CASES

pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.mark.parametrize("n", [1, 5, 1023, 4096, 100_003, 1 << 20])
@pytest.mark.parametrize("bins", [1, 7, 100, 2048, 4096])
def test_histc_matches_oracle(n, bins):
    g = np.random.default_rng(n + bins)
    x = (g.standard_normal(n) * 3).astype(F32)
    # the reference's default: the range comes from the data
    assert np.array_equal(host(Q.histc(dev(x), bins)), O.histc(x, bins, 0, 0))
    # an explicit range that leaves elements outside
    got = Q.histc(dev(x), bins, -1.5, 2.25)
    want = O.histc(x, bins, -1.5, 2.25)
    assert np.array_equal(host(got), want)
    assert want.sum() == np.count_nonzero((x >= -1.5) & (x <= 2.25))


def test_histc_bf16_unaligned_and_2d():
    g = np.random.default_rng(3)
    x = g.standard_normal((37, 129)).astype(F32)
    xb = dev(x, torch.bfloat16)
    want = O.histc(host(xb), 512, -2.0, 2.0)
    assert np.array_equal(host(Q.histc(xb, 512, -2.0, 2.0)), want)
    # a view that starts 4 bytes into the allocation: the scalar path
    big = dev(np.concatenate([[0.0], x.ravel()]).astype(F32))
    assert np.array_equal(host(Q.histc(big[1:], 512, -2.0, 2.0)), O.histc(x, 512, -2.0, 2.0))


def test_histc_values_on_bin_edges():
    """Elements on, just below and just above every bin edge: the quotient sits at an integer,
    where a multiply by the reciprocal and the true division may disagree."""
    for lo, hi, bins in [(-1.0, 1.0, 2048), (0.1, 0.7, 1000), (-3.3, 9.1, 4096), (1e-3, 1.1e-3, 100)]:
        step = (hi - lo) / bins
        edges = (lo + np.arange(bins + 1, dtype=np.float64) * step).astype(F32)
        x = np.concatenate([edges, np.nextafter(edges, F32(np.inf)), np.nextafter(edges, F32(-np.inf)),
                            # thirds and other quotients with long binary expansions
                            (lo + (np.arange(3 * bins) / 3.0) * step).astype(F32)]).astype(F32)
        assert np.array_equal(host(Q.histc(dev(x), bins, lo, hi)), O.histc(x, bins, lo, hi)), (lo, hi, bins)


def test_histc_low_precision_data_sits_on_edges():
    """bfloat16 activations and quantized grids put a large share of the elements exactly on
    bin edges (the quotient is an integer): every one of them needs the exact tie-break."""
    g = np.random.default_rng(17)
    xb = dev((g.standard_normal(300_000) * 1.5).astype(F32), torch.bfloat16)
    xh = host(xb)
    for lo, hi, bins in [(-5.5, 5.5, 2048), (-4.0, 4.0, 2048), (-8.0, 8.0, 4096), (-3.0, 5.0, 1000)]:
        want = O.histc(xh, bins, lo, hi)
        assert np.array_equal(host(Q.histc(xb, bins, lo, hi)), want)
        assert np.array_equal(host(Q.histc(xb.float(), bins, lo, hi)), want)
    grid = (g.integers(-128, 128, 200_000) * 0.0625).astype(F32)  # all on edges of [-8, 8] / 2048
    assert np.array_equal(host(Q.histc(dev(grid), 2048, -8.0, 8.0)), O.histc(grid, 2048, -8.0, 8.0))
    assert np.array_equal(host(Q.histc(dev(grid), 2048)), O.histc(grid, 2048, 0, 0))
    third = (g.integers(0, 3000, 100_000) / 3.0).astype(F32)
    assert np.array_equal(host(Q.histc(dev(third), 1000, 0.0, 1000.0)), O.histc(third, 1000, 0.0, 1000.0))


def test_histc_constant_and_rectified():
    x = np.full(1000, 0.75, dtype=F32)
    want = O.histc(x, 64, 0, 0)
    assert want[0] == 1000  # [v, v + 1]
    assert np.array_equal(host(Q.histc(dev(x), 64)), want)
    g = np.random.default_rng(5)
    r = np.maximum(g.standard_normal(200_000), 0).astype(F32)
    assert np.array_equal(host(Q.histc(dev(r), 2048)), O.histc(r, 2048, 0, 0))
    nan = r.copy()
    nan[::7] = np.nan
    got = host(Q.histc(dev(nan), 256, 0.0, 4.0))
    assert np.array_equal(got, O.histc(nan[~np.isnan(nan)], 256, 0.0, 4.0))


def test_histc_large_is_exact():
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(1 << 26, device="cuda", generator=g)  # 256 MB: larger than L2
    h = Q.histc(x, 2048)
    assert float(h.double().sum()) == x.numel()
    part = x[: 1 << 24]
    lo, hi = float(x.min()), float(x.max())
    assert np.array_equal(host(Q.histc(part, 2048, lo, hi)), O.histc(host(part), 2048, lo, hi))


def test_histc_rejects():
    x = torch.randn(64, device="cuda")
    with pytest.raises(NotImplementedError):
        Q.histc(x, 1 << 20)
    with pytest.raises(L.ShapeMismatch):
        Q.histc(x, 16, 2.0, 1.0)
    with pytest.raises(L.ShapeMismatch):
        Q.histc(x, 16, 0.0, float("inf"))
    with pytest.raises(L.DeviceMismatch):
        Q.histc(x.cpu(), 16)
    with pytest.raises(L.DtypeMismatch):
        Q.histc(x.to(torch.int32), 16)


@pytest.mark.parametrize("tag,batches,bins,sym,qd", HIST_CASES)
def test_histogram_observer_golden(golden, tag, batches, bins, sym, qd):
    scheme = Q.per_tensor_symmetric if sym else Q.per_tensor_affine
    obs = Q.HistogramObserver(bins=bins, qscheme=scheme, qdtype=Q.qint8 if qd[2] else Q.quint8)
    for i in range(batches):
        obs(dev(golden[f"{tag}_x{i}"]))
        assert np.array_equal(host(obs.histogram), golden[f"{tag}_hist{i}"]), (tag, i)
        assert [float(obs.min_val), float(obs.max_val)] == golden[f"{tag}_range{i}"].tolist()
    assert list(obs._search_clip_range()) == golden[f"{tag}_clip"].tolist()
    s, z = obs.calculate_qparams()
    assert s.item() == golden[f"{tag}_scale"] and z.item() == golden[f"{tag}_zp"]


def test_histogram_observer_long_run_against_oracle():
    """Twelve batches with drifting scale: single-pass folds, range growth and re-binning mixed."""
    g = np.random.default_rng(21)
    obs = Q.HistogramObserver()
    state = None
    for i in range(12):
        scale = [1.0, 0.5, 2.0, 1.5, 0.2, 3.0, 3.0, 0.1, 4.5, 1.0, 2.0, 6.0][i]
        x = (g.standard_normal(50_000) * scale + 0.1 * i).astype(F32)
        obs(dev(x))
        state = O.histogram_observe(x, state, 2048)
        assert np.array_equal(host(obs.histogram), state[2]), i
        assert (float(obs.min_val), float(obs.max_val)) == (state[0], state[1])
    assert obs.histogram.sum().item() == 12 * 50_000
    s, z = obs.calculate_qparams()
    so, zo = O.histogram_qparams(state[0], state[1], state[2], False, O.QUINT8)
    assert s.item() == so and z.item() == zo


def test_histogram_observer_step_is_asynchronous_and_capturable():
    """A step never reads anything back: three steps captured in a CUDA graph (range held,
    range grew, range held again) replay to the oracle's state."""
    g = np.random.default_rng(23)
    xs = [(g.standard_normal(30_000) * s).astype(F32) for s in (1.0, 0.5, 2.0, 0.7)]
    obs = Q.HistogramObserver()
    obs(dev(xs[0]))  # seeds the state and allocates the workspace
    state = O.histogram_observe(xs[0], None, 2048)
    bufs = [dev(x) for x in xs[1:]]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for b in bufs:
                obs(b)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    for x in xs[1:]:
        state = O.histogram_observe(x, state, 2048)
    assert np.array_equal(host(obs.histogram), state[2])
    assert (float(obs.min_val), float(obs.max_val)) == (state[0], state[1])


def test_histogram_observer_ignores_batches_without_finite_values():
    obs = Q.HistogramObserver(bins=64)
    x = torch.randn(1000, device="cuda")
    obs(x)
    before = (obs.histogram.clone(), float(obs.min_val), float(obs.max_val))
    obs(torch.full((50,), float("nan"), device="cuda"))
    assert torch.equal(obs.histogram, before[0])
    assert (float(obs.min_val), float(obs.max_val)) == before[1:]
    fresh = Q.HistogramObserver(bins=64)
    fresh(torch.full((50,), float("nan"), device="cuda"))
    assert float(fresh.min_val) == float("inf") and fresh.histogram.sum().item() == 0
    fresh(x)
    assert torch.equal(fresh.histogram, before[0])


def test_histogram_observer_state_dict_round_trip():
    g = np.random.default_rng(22)
    a, b = Q.HistogramObserver(bins=512), Q.HistogramObserver(bins=512)
    x0, x1 = (g.standard_normal(4000).astype(F32) for _ in range(2))
    a(dev(x0))
    buf = io.BytesIO()
    torch.save(a.state_dict(), buf)
    buf.seek(0)
    b.load_state_dict(torch.load(buf))
    a(dev(x1 * 2))
    b(dev(x1 * 2))
    assert torch.equal(a.histogram, b.histogram.to(a.histogram.device))
    assert float(a.min_val) == float(b.min_val) and float(a.max_val) == float(b.max_val)


def test_moving_average_observers_golden(golden):
    ma = Q.MovingAverageMinMaxObserver(averaging_constant=0.05)
    mac = Q.MovingAveragePerChannelMinMaxObserver(ch_axis=0, averaging_constant=0.05)
    for i in range(3):
        x = dev(golden[f"ma_x{i}"])
        ma(x)
        mac(x)
        assert ma.min_val.item() == golden[f"ma_min{i}"] and ma.max_val.item() == golden[f"ma_max{i}"]
        assert np.array_equal(host(mac.min_val), golden[f"mac_min{i}"])
        assert np.array_equal(host(mac.max_val), golden[f"mac_max{i}"])
    s, z = ma.calculate_qparams()
    assert s.item() == golden["ma_scale"] and z.item() == golden["ma_zp"]
    s, z = mac.calculate_qparams()
    assert np.array_equal(host(s), golden["mac_scale"]) and np.array_equal(host(z), golden["mac_zp"])


def test_fixed_and_placeholder_observers():
    f = Q.FixedQParamsObserver(1.0 / 256.0, 0)
    x = torch.randn(8, device="cuda")
    assert f(x) is x
    s, z = f.calculate_qparams()
    assert s.item() == 1.0 / 256.0 and z.item() == 0.0
    with pytest.raises(RuntimeError):
        Q.PlaceholderObserver().calculate_qparams()
    assert Q.NoopObserver()(x) is x


def test_default_qconfig_uses_histogram_observer():
    qc = Q.get_default_qconfig()
    assert isinstance(qc.activation(), Q.HistogramObserver)
    assert isinstance(qc.weight(), Q.PerChannelMinMaxObserver)
