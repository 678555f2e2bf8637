"""CPU-only checks of the drop-in boundary: the C-ABI library loads and exports
every declared symbol, the Python surface mirrors the reference's names, and
argument errors are raised before any device work."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import lucid_b200
import lucid_b200.nn.quantized as nnq
import lucid_b200.quantization as Q
from lucid_b200 import _lib
from lucid_b200.quantization import _functional as QFn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "lucid_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert {"lq_quantize", "lq_dequantize", "lq_gemm_s8", "lq_conv2d_nhwc_s8", "lq_minmax"} <= set(names)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/lucid_b200.h but not exported"
    # the shim binds exactly the declared set
    assert sorted(_lib._SIGNATURES) == names
    assert _lib.load().lq_version() == 100


def test_host_side_argument_errors_need_no_gpu():
    lib = _lib.load()
    e = _lib.Epilogue()
    assert lib.lq_quantize(None, 0, 4, 4, None, None, 1.0, 0.0, 0, -128, 127, None, 2, None) == 3
    assert "null" in _lib.last_error()
    assert lib.lq_quantize(None, 0, 0, 4, None, None, 1.0, 0.0, 0, -128, 127, None, 2, None) == 0  # empty
    one = ctypes.c_void_p(16)
    assert lib.lq_gemm_s8(one, 1, one, 8, 8, 24, ctypes.byref(e), one, 8, None, None) == 4  # K % 16
    assert lib.lq_gemm_s8(one, 1, one, 8, 8, 32, None, one, 8, None, None) == 3
    e.out_dtype = 99
    assert lib.lq_gemm_s8(one, 1, one, 8, 8, 32, ctypes.byref(e), one, 8, None, None) == 2
    e.out_dtype = _lib.F32
    assert lib.lq_gemm_s8(one, 1, one, 8, 8, 32, ctypes.byref(e), one, 8, None, None) == 3  # scales missing
    assert lib.lq_minmax(one, 0, 0, 4, 0, one, one, one, 1 << 20, None) == 1  # empty has no range
    assert lib.lq_minmax(one, 0, 4, 4, 0, one, one, one, 8, None) == 6  # workspace too small
    assert lib.lq_conv2d_nhwc_s8(one, 1, one, 1, 8, 8, 16, 16, 3, 3, 9, 1, ctypes.byref(e), one, None, None) == 5  # stride > 8
    assert lib.lq_conv2d_nhwc_s8(one, 1, one, 1, 8, 8, 16, 16, 3, 3, 0, 1, ctypes.byref(e), one, None, None) == 1
    geo = _lib.ConvGeometry(N=1, H=8, W=8, C=32, K=16, R=3, S=3, P=8, Q=8, stride_h=1, stride_w=1, pad_h=1, pad_w=1,
                            dil_h=1, dil_w=1, groups=3)
    conv_ex = lambda: lib.lq_conv2d_nhwc_s8_ex(one, 1, one, ctypes.byref(geo), ctypes.byref(e), one, None, 0, None, None)
    assert conv_ex() == 1  # groups must divide C and K
    geo.groups, geo.K = 4, 16
    assert conv_ex() == 4  # 8 channels per group: not a multiple of 16
    geo.groups, geo.P = 1, 40
    assert conv_ex() == 1  # output larger than the padded input allows
    # workspace-carrying and sharded contraction, exchange flags
    e.out_dtype = _lib.S32
    assert lib.lq_gemm_s8_ws(one, 1, one, 8, 8, 32, ctypes.byref(e), one, 8, one, 64, None, None) == 6
    assert lib.lq_gemm_workspace_bytes() >= 148 * 128 * 256 * 4
    ptrs = (ctypes.c_void_p * 2)(16, 32)
    assert lib.lq_gemm_s8_sharded(one, 1, one, 8, 8, 32, ctypes.byref(e), ptrs, 2, 8, 0, ptrs, 2, one, None, 0,
                                  None, None) == 3  # signalling needs the workspace
    assert lib.lq_gemm_s8_sharded(one, 1, one, 8, 8, 32, ctypes.byref(e), ptrs, 9, 8, 0, None, 0, None, None, 0,
                                  None, None) == 1  # at most 8 destinations
    assert lib.lq_peer_wait(one, 0, one, 0, None, None) == 1
    assert lib.lq_peer_wait(None, 2, one, 0, None, None) == 3
    assert lib.lq_peer_signal(ptrs, 9, one, None) == 1
    assert lib.lq_absmax_rows_bcast(one, 7, 4, 16, 16, ptrs, 2, 0, None) == 2
    assert lib.lq_quantize_per_token_bcast(one, 1, 4, 24, -128, 127, 1e-8, ptrs, ptrs, 2, None, 0, None) == 4  # cols % 16
    assert lib.lq_quantize_rows_bcast(one, 1, 4, 16, 16, one, 0, 4, -128, 127, 1e-8, ptrs, 2, 16, 0, None, None) == 1  # parts
    e.out_dtype = _lib.F32
    hist = (one, 0, 64, 0.0, 1.0, 16, None, 0.0, 0.0, one, None, None, one, 1 << 20, None)
    assert lib.lq_histc(*hist[:5], lib.lq_histc_max_bins() + 1, *hist[6:]) == 5
    assert lib.lq_histc(*hist[:3], 1.0, 1.0, *hist[5:]) == 1  # empty range: the caller derives it
    assert lib.lq_histc(*hist[:3], 0.0, float("inf"), *hist[5:]) == 1
    assert lib.lq_histc(*hist[:2], 0, *hist[3:]) == 1
    assert lib.lq_histc(*hist[:13], 64, None) == 6  # workspace too small
    assert lib.lq_histc_workspace_bytes() >= 8 * lib.lq_histc_max_bins()
    assert lib.lq_histogram_observe(one, 0, 64, 16, None, one, one, one, 1 << 20, None) == 3
    # element-wise merges, tables, embeddings
    merge = [0, one, 0, None, None, None, 0, None, None, 0.0, 8, one, one, 0, 255, one, 3, None, None]
    assert lib.lq_qmerge(*merge[:10], 0, *merge[11:]) == 0  # nothing to do
    assert lib.lq_qmerge(7, *merge[1:]) == 5
    assert lib.lq_qmerge(*merge[:2], 3, *merge[3:]) == 2  # codes need their scale / zero point
    assert lib.lq_qmerge(*merge[:3], one, None, *merge[5:]) == 3  # ... both of them
    assert lib.lq_qmerge(*merge[:15], None, 3, None, None) == 3  # no output requested
    assert lib.lq_qmerge(*merge[:13], 5, 4, *merge[15:]) == 1  # qmin > qmax
    assert lib.lq_lut_u8(one, 8, None, one, None) == 3
    assert lib.lq_lut2_u8(one, one, 8, ctypes.c_void_p(24), one, None, None, None, 0, None) == 4  # table alignment
    assert lib.lq_lut2_u8(one, one, 8, one, one, one, None, None, 0, None) == 3  # f32 output needs the grid
    emb = [one, one, one, 10, 16, one, 64, 4, None, 0, 0, 0, -1, one, 0, None, None]
    assert lib.lq_embedding_s8(*emb[:6], 16, *emb[7:]) == 2  # index width
    assert lib.lq_embedding_s8(*emb[:4], 0, *emb[5:]) == 1  # empty table
    assert lib.lq_embedding_s8(*emb[:14], 2, *emb[15:]) == 2  # lookups leave as f32 / bf16
    assert lib.lq_embedding_s8(*emb[:8], one, 2, 0, 3, *emb[12:]) == 5  # pooling mode
    assert lib.lq_embedding_s8(*emb[:8], one, 2, 0, 0, -1, one, 1, None, None) == 2  # bags pool in f32
    assert lib.lq_histogram_observe(one, 0, 64, 0, one, one, one, one, 1 << 20, None) == 5
    assert lib.lq_histogram_observe(one, 9, 64, 16, one, one, one, one, 1 << 20, None) == 2


def test_cpu_tensors_are_rejected_not_emulated():
    x = torch.randn(4, 16)
    with pytest.raises(lucid_b200.DeviceMismatch):
        Q.quantize(x, 0.1, 0.0, Q.qint8)
    with pytest.raises(lucid_b200.DeviceMismatch):
        Q.dequantize(torch.zeros(4, dtype=torch.int8), 0.1, 0.0)
    with pytest.raises(lucid_b200.DeviceMismatch):
        Q.MinMaxObserver()(x)
    with pytest.raises(lucid_b200.DeviceMismatch):
        nnq.dynamic.Linear(16, 8)(x)


def test_histogram_clip_search_is_host_logic(golden):
    """The clip search runs on the host from the histogram alone
    (lucid/quantization/observer.py:840-870): feed it the reference-made histograms."""
    for tag, last, bins, qd in (("hg", 3, 2048, Q.quint8), ("hs", 2, 128, Q.qint8),
                                ("hc", 1, 256, Q.quint8), ("hr", 1, 2048, Q.quint8),
                                ("ht", 0, 2048, Q.quint8)):
        obs = Q.HistogramObserver(bins=bins, qdtype=qd)
        lo, hi = golden[f"{tag}_range{last}"].tolist()
        obs.load_state_dict({"min_val": torch.tensor(lo), "max_val": torch.tensor(hi),
                             "histogram": torch.from_numpy(golden[f"{tag}_hist{last}"])})
        assert list(obs._search_clip_range()) == golden[f"{tag}_clip"].tolist()
    with pytest.raises(lucid_b200.DeviceMismatch):
        Q.HistogramObserver()(torch.randn(8))
    assert isinstance(Q.get_default_qconfig().activation(), Q.HistogramObserver)


def test_surface_matches_reference_names():
    assert (Q.qint8.quant_min, Q.qint8.quant_max, Q.qint8.storage) == (-128, 127, "int8")
    assert (Q.quint8.quant_min, Q.quint8.quant_max, Q.quint8.storage) == (0, 255, "int16")
    assert (Q.qint4.quant_min, Q.qint4.quant_max) == (-8, 7)
    assert Q.qint32.storage == "int32" and Q.qint8.signed and not Q.quint8.signed
    assert repr(Q.qint8) == "lucid.quantization.qint8"
    assert Q.per_channel_symmetric.is_per_channel and not Q.per_tensor_affine.is_per_channel
    assert Q.per_tensor_symmetric.is_symmetric and not Q.per_channel_affine.is_symmetric
    lin = nnq.Linear(32, 16)
    assert list(lin.state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point", "bias",
                                      "scale", "zero_point"]
    assert lin.weight_int8.dtype == torch.int8 and lin.out_qdtype is Q.quint8
    assert "qdtype=quint8" in repr(lin)
    conv = nnq.Conv2d(16, 32, 3, padding=1)
    assert tuple(conv.weight_int8.shape) == (32, 16, 3, 3)
    assert list(conv.state_dict()) == list(lin.state_dict())
    dyn = nnq.dynamic.Linear(32, 16, bias=False)
    assert list(dyn.state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point"]
    assert "dynamic=True" in repr(dyn)


def test_engine_switch():
    b = lucid_b200.backends.quantized
    assert b.engine == "auto" and b.use_int8()
    with pytest.raises(ValueError):
        b.engine = "fastest"
    b.engine = "reference"
    assert not b.use_int8()
    assert not b.use_mlx()
    b.engine = "mlx_group"  # the Linear family on the group-wise weight-only layer, the rest float
    assert b.use_mlx() and not b.use_int8()
    try:
        import torch

        from lucid_b200.quantization import _quantize

        assert _quantize._quant_mapping()[torch.nn.Linear].__name__ == "build"
        assert _quantize._mlx_group_size(4096) == 64 and _quantize._mlx_group_size(96) == 32
        assert _quantize._mlx_group_size(100) is None
    finally:
        b.engine = "auto"
    assert not b.use_mlx()
    assert lucid_b200.device("cuda:0").type == "cuda"
    with pytest.raises(RuntimeError):
        lucid_b200.device("metal")
    with pytest.raises(ValueError):
        lucid_b200.device("tpu")


def test_view2d_and_param_broadcast():
    x = torch.empty(6, 32, 16)
    assert QFn._view2d(x, 0, True) == (6, 512, _lib.PER_ROW, 1)
    assert QFn._view2d(x, 2, True) == (192, 16, _lib.PER_COL, 1)
    assert QFn._view2d(x, -1, True) == (192, 16, _lib.PER_COL, 1)
    assert QFn._view2d(x, 1, True) == (192, 16, _lib.PER_ROW, 6)
    assert QFn._view2d(x, None, False) == (192, 16, _lib.PER_TENSOR, 1)
    rows, cols, mode, s, z, sv, zv = QFn._prepare_params(x, 0.5, 3, None)
    assert (s, z, sv, zv, mode) == (None, None, 0.5, 3.0, _lib.PER_TENSOR)
    sc = torch.arange(32, dtype=torch.float32)
    rows, cols, mode, s, z, _, _ = QFn._prepare_params(x, sc, 0.0, 1)
    assert mode == _lib.PER_ROW and s.numel() == 192 and torch.equal(s[:32], sc) and torch.equal(s[32:64], sc)
    assert z.numel() == 192 and float(z.abs().sum()) == 0.0
    with pytest.raises(lucid_b200.ShapeMismatch):
        QFn._prepare_params(x, torch.ones(5), 0.0, 1)
    with pytest.raises(lucid_b200.ShapeMismatch):
        QFn._prepare_params(x, torch.ones(5), 0.0, None)


def test_gate_up_interleave_layout():
    g = torch.arange(256).reshape(256, 1)
    u = g + 1000
    w = nnq.dynamic.interleave_gate_up(g, u)
    assert w.shape == (512, 1)
    assert w[:128, 0].tolist() == list(range(128)) and w[128:256, 0].tolist() == list(range(1000, 1128))
    assert w[256:384, 0].tolist() == list(range(128, 256))
    with pytest.raises(lucid_b200.ShapeMismatch):
        nnq.dynamic.interleave_gate_up(g[:100], u[:100])


def test_shard_bounds():
    from lucid_b200.nn.quantized.sharded import shard_bounds

    assert [shard_bounds(28672, 8, r) for r in (0, 7)] == [(0, 3584), (25088, 28672)]
    assert shard_bounds(10240, 8, 3) == (3840, 5120)
    with pytest.raises(lucid_b200.ShapeMismatch):
        shard_bounds(10, 4, 0)
    with pytest.raises(ValueError):
        shard_bounds(16, 4, 4)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No CPU fallback: without the built extension the package raises instead of emulating."""
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "liblucid_b200.so"))
    assert not _lib.is_available()
    with pytest.raises(lucid_b200.EngineUnavailable):
        _lib.load()
    assert not lucid_b200.backends.quantized.available


def test_package_never_imports_the_oracle():
    import subprocess
    import sys

    code = ("import sys, lucid_b200, lucid_b200.nn.quantized, lucid_b200.quantization;"
            "assert not any(m == 'oracle' or m.startswith('oracle.') for m in sys.modules)")
    subprocess.check_call([sys.executable, "-c", code], cwd=ROOT)


def test_workflow_routing_needs_no_gpu():
    """prepare / prepare_qat / quantize_dynamic decide what to swap on the host."""
    import lucid_b200.nn.qat as nnqat

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(8, 8)
            self.act = torch.nn.Hardswish()
            self.up = torch.nn.ConvTranspose2d(4, 4, 2)
            self.skip = nnq.FloatFunctional()

        def forward(self, x):
            return self.skip.add(self.act(self.fc(x)), x)

    ff = nnq.FloatFunctional()
    a, b = torch.randn(4), torch.randn(4)
    assert torch.equal(ff.add(a, b), a + b) and torch.equal(ff.add_relu(a, b), torch.relu(a + b))
    assert torch.equal(ff.cat([a, b]), torch.cat([a, b])) and torch.equal(ff.mul_scalar(a, 2.0), a * 2.0)
    prepared = Q.prepare(Block())
    for name in ("fc", "act", "up", "skip"):
        assert isinstance(getattr(prepared, name).activation_post_process, Q.HistogramObserver), name
    assert not hasattr(prepared.skip, "_lq_hook") and hasattr(prepared.fc, "_lq_hook")
    qat = Q.prepare_qat(Block())
    assert type(qat.fc) is nnqat.Linear and qat.training
    assert isinstance(qat.fc.weight_fake_quant, Q.FakeQuantize)
    assert isinstance(qat.fc.activation_post_process.activation_post_process, Q.MovingAverageMinMaxObserver)
    assert qat.fc.weight_fake_quant.ch_axis == 0 and qat.fc.activation_post_process.ch_axis is None
    fq = Q.FakeQuantize()
    assert fq.disable_observer() is fq and fq.disable_fake_quant()(a) is a
    with pytest.raises(ValueError):
        nnqat.Linear(4, 4)
    with pytest.raises(ValueError):
        nnq.EmbeddingBag(10, 4, mode="sun")
    with pytest.raises(lucid_b200.DeviceMismatch):
        nnq.QFunctional(0.1, 0.0).add(a, b)
    with pytest.raises(lucid_b200.DeviceMismatch):
        nnq.Embedding(10, 4)(torch.tensor([1, 2]))
    with pytest.raises(lucid_b200.DeviceMismatch):
        nnq.Sigmoid(0.1, 0.0)(a)
    emb = nnq.Embedding(10, 4, padding_idx=0)
    assert list(emb.state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point"]
    ct = nnq.ConvTranspose2d(4, 6, 3, stride=2)
    assert tuple(ct.weight_int8.shape) == (4, 6, 3, 3) and ct.weight_ch_axis == 1
    assert list(ct.state_dict()) == ["weight_int8", "weight_scale", "weight_zero_point", "bias", "scale", "zero_point"]


def test_public_names_of_the_reference_are_all_present():
    """The drop-in surface: every name the reference's packages export for this path
    (``__all__`` of lucid/quantization/__init__.py, lucid/nn/quantized/__init__.py:45-73,
    lucid/nn/quantized/dynamic, lucid/nn/qat, lucid/nn/intrinsic, lucid/nn/intrinsic/qat)
    exists under the same package here."""
    import importlib

    surface = {
        "lucid_b200.quantization": """FakeQuantize FixedQParamsObserver HistogramObserver MinMaxObserver
            MovingAverageMinMaxObserver MovingAveragePerChannelMinMaxObserver NoopObserver ObserverBase
            PerChannelMinMaxObserver PlaceholderObserver QConfig QConfigMapping QDtype QParams QScheme
            calculate_qparams convert convert_fx dequantize fake_quantize fuse_modules fuse_modules_qat
            get_default_qat_qconfig get_default_qat_qconfig_mapping get_default_qconfig
            get_default_qconfig_mapping per_channel_affine per_channel_symmetric per_tensor_affine
            per_tensor_symmetric prepare prepare_fx prepare_qat qint32 qint4 qint8 quantize quantize_dynamic
            quint8""",
        "lucid_b200.nn.quantized": """Conv1d Conv2d Conv3d ConvReLU1d ConvReLU2d ConvReLU3d ConvTranspose1d
            ConvTranspose2d ConvTranspose3d DeQuantStub DeQuantize ELU Embedding EmbeddingBag FloatFunctional
            Hardsigmoid Hardswish LeakyReLU Linear LinearReLU QFunctional QuantStub QuantWrapper Quantize
            QuantizedLinearMLX Sigmoid Tanh""",
        "lucid_b200.nn.quantized.dynamic": "LSTM Linear",
        "lucid_b200.nn.qat": "Conv1d Conv2d Conv3d ConvReLU1d ConvReLU2d ConvReLU3d Embedding Linear LinearReLU",
        "lucid_b200.nn.intrinsic": "ConvReLU1d ConvReLU2d ConvReLU3d LinearReLU",
        "lucid_b200.nn.intrinsic.qat": "ConvBn1d ConvBn2d ConvBn3d ConvBnReLU1d ConvBnReLU2d ConvBnReLU3d",
    }
    for package, names in surface.items():
        mod = importlib.import_module(package)
        missing = [n for n in names.split() if not hasattr(mod, n)]
        assert not missing, (package, missing)
