"""Calibration observers on device (lucid/quantization/observer.py).

Every observation is one pass over the observed tensor: the running min / max observers
(observer.py:364-375, 635-648) and their moving-average forms (:490-505, :1000-1018) run one
fused reduction (the reference runs two), and the histogram observer (:773-880) bins the batch
against its current range while the same kernel measures the batch's own range and folds the
running histogram, so a second pass is needed only when the range grew (the reference makes
three passes and two host read-backs per batch)."""

from __future__ import annotations

import functools
import math

import torch

from .. import _lib
from ._qparams import calculate_qparams
from ._qscheme import (QDtype, QScheme, per_channel_symmetric, per_tensor_affine, qint8, quint8)


def minmax(x: torch.Tensor, per_row: bool = False):
    """(min, max) of a CUDA tensor: scalars, or one pair per row of the 2-D view
    ``(shape[0], -1)``."""
    _lib.require_cuda(x, "observed tensor")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.DtypeMismatch(f"observers take float32/bfloat16, got {x.dtype}")
    if x.numel() == 0:
        raise _lib.ShapeMismatch("cannot observe an empty tensor")
    xc = x.detach().contiguous()
    dev = xc.device
    with torch.cuda.device(dev):
        if per_row:
            rows = xc.shape[0]
            cols = xc.numel() // rows
            mn = torch.empty(rows, dtype=torch.float32, device=dev)
            mx = torch.empty(rows, dtype=torch.float32, device=dev)
            _lib.check(_lib.load().lq_minmax(_lib.ptr(xc), _lib.code_of(xc.dtype), rows, cols,
                                             _lib.PER_ROW, _lib.ptr(mn), _lib.ptr(mx), None, 0,
                                             _lib.stream_ptr(dev)))
        else:
            mn = torch.empty((), dtype=torch.float32, device=dev)
            mx = torch.empty((), dtype=torch.float32, device=dev)
            ws = _lib.minmax_workspace(dev)
            _lib.check(_lib.load().lq_minmax(_lib.ptr(xc), _lib.code_of(xc.dtype), 1, xc.numel(),
                                             _lib.PER_TENSOR, _lib.ptr(mn), _lib.ptr(mx),
                                             _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return mn, mx


class ObserverBase(torch.nn.Module):
    def __init__(self, qscheme: QScheme, qdtype: QDtype, ch_axis=None, eps: float = 1e-8):
        super().__init__()
        self.qscheme = qscheme
        self.qdtype = qdtype
        self.ch_axis = ch_axis if qscheme.is_per_channel else None
        self.eps = eps

    @classmethod
    def with_args(cls, **kwargs):
        return functools.partial(cls, **kwargs)

    def _fold(self, cur_min, cur_max):
        # seeds are +inf / -inf scalars that broadcast on first sight
        self.min_val = torch.minimum(self.min_val.to(cur_min.device), cur_min)
        self.max_val = torch.maximum(self.max_val.to(cur_max.device), cur_max)

    def calculate_qparams(self):
        return calculate_qparams(self.min_val, self.max_val, self.qscheme, self.qdtype, self.eps)


class MinMaxObserver(ObserverBase):
    """Per-tensor running min / max (lucid/quantization/observer.py:352-375)."""

    def __init__(self, qscheme=per_tensor_affine, qdtype=quint8, eps: float = 1e-8):
        super().__init__(qscheme, qdtype, None, eps)
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))

    def forward(self, x):
        self._fold(*minmax(x))
        return x


class PerChannelMinMaxObserver(ObserverBase):
    """Per-channel running min / max (lucid/quantization/observer.py:620-652)."""

    def __init__(self, ch_axis: int = 0, qscheme=per_channel_symmetric, qdtype=qint8,
                 eps: float = 1e-8):
        super().__init__(qscheme, qdtype, ch_axis, eps)
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))

    def forward(self, x):
        axis = self.ch_axis if self.ch_axis is not None else 0
        perm = x if axis % max(x.dim(), 1) == 0 else torch.movedim(x, axis, 0)
        self._fold(*minmax(perm, per_row=True))
        return x


class MovingAverageMinMaxObserver(MinMaxObserver):
    """Per-tensor min / max smoothed by an exponential moving average, seeded by the first
    batch (lucid/quantization/observer.py:479-505)."""

    def __init__(self, qscheme=per_tensor_affine, qdtype=quint8, averaging_constant: float = 0.01,
                 eps: float = 1e-8):
        super().__init__(qscheme, qdtype, eps)
        self.averaging_constant = averaging_constant

    def forward(self, x):
        cur_min, cur_max = minmax(x)
        c = self.averaging_constant
        mn, mx = self.min_val.to(cur_min.device), self.max_val.to(cur_max.device)
        first = torch.isinf(mn)
        self.min_val = torch.where(first, cur_min, mn + c * (cur_min - mn))
        self.max_val = torch.where(first, cur_max, mx + c * (cur_max - mx))
        return x


class MovingAveragePerChannelMinMaxObserver(PerChannelMinMaxObserver):
    """Per-channel min / max smoothed by an exponential moving average
    (lucid/quantization/observer.py:988-1018)."""

    def __init__(self, ch_axis: int = 0, qscheme=per_channel_symmetric, qdtype=qint8,
                 averaging_constant: float = 0.01, eps: float = 1e-8):
        super().__init__(ch_axis, qscheme, qdtype, eps)
        self.averaging_constant = averaging_constant

    def forward(self, x):
        axis = self.ch_axis if self.ch_axis is not None else 0
        perm = x if axis % max(x.dim(), 1) == 0 else torch.movedim(x, axis, 0)
        cur_min, cur_max = minmax(perm, per_row=True)
        if self.min_val.dim() == 0 and math.isinf(float(self.min_val)):
            # the seed is a scalar +inf: the first batch sets the per-channel vectors directly
            self.min_val, self.max_val = cur_min, cur_max
        else:
            c = self.averaging_constant
            mn, mx = self.min_val.to(cur_min.device), self.max_val.to(cur_max.device)
            self.min_val = mn + c * (cur_min - mn)
            self.max_val = mx + c * (cur_max - mx)
        return x


class FixedQParamsObserver(ObserverBase):
    """Fixed (scale, zero_point); observes nothing (lucid/quantization/observer.py:1113-1132)."""

    def __init__(self, scale: float, zero_point: int, qscheme=per_tensor_affine, qdtype=quint8,
                 eps: float = 1e-8):
        super().__init__(qscheme, qdtype, None, eps)
        self.register_buffer("scale", torch.tensor(float(scale)))
        self.register_buffer("zero_point", torch.tensor(float(zero_point)))

    def forward(self, x):
        return x

    def calculate_qparams(self):
        return self.scale, self.zero_point


class PlaceholderObserver(ObserverBase):
    """Identity marker for tensors whose qparams come from elsewhere
    (lucid/quantization/observer.py:1212-1230)."""

    def __init__(self, qscheme=per_tensor_affine, qdtype=quint8, eps: float = 1e-8):
        super().__init__(qscheme, qdtype, None, eps)

    def forward(self, x):
        return x

    def calculate_qparams(self):
        raise RuntimeError(
            f"{type(self).__name__} collects no statistics; qparams are computed at runtime "
            "(dynamic quantization) or supplied elsewhere.")


class NoopObserver(PlaceholderObserver):
    """A tensor that is deliberately not quantized here (lucid/quantization/observer.py:1233)."""


# ---- histogram observer -------------------------------------------------------------------
def _histc_launch(xc, bins, lo, hi, prev=None, prev_range=None, want_range=False):
    """One ``lq_histc`` launch on contiguous ``xc`` over the finite range ``lo < hi``.
    ``prev`` is folded in: added bin by bin when ``prev_range`` is None (same grid), else
    re-binned from ``prev_range`` onto ``[lo, hi]``."""
    dev = xc.device
    with torch.cuda.device(dev):
        out = torch.empty(bins, dtype=torch.float32, device=dev)
        mm = torch.empty(2, dtype=torch.float32, device=dev) if want_range else None
        ws = _lib.histc_workspace(dev)
        p_lo, p_hi = (lo, hi) if prev_range is None else prev_range
        mm_ptr = None if mm is None else mm.data_ptr()
        _lib.check(_lib.load().lq_histc(
            _lib.ptr(xc), _lib.code_of(xc.dtype), xc.numel(), float(lo), float(hi), int(bins),
            _lib.ptr(prev), float(p_lo), float(p_hi), _lib.ptr(out),
            mm_ptr, None if mm_ptr is None else mm_ptr + 4,
            _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return out, mm


def _check_observed(x):
    _lib.require_cuda(x, "observed tensor")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.DtypeMismatch(f"observers take float32/bfloat16, got {x.dtype}")
    if x.numel() == 0:
        raise _lib.ShapeMismatch("cannot observe an empty tensor")
    return x.detach().contiguous()


def _range_of(xc):
    """(min, max) of the tensor as Python floats: one kernel, one read-back."""
    dev = xc.device
    with torch.cuda.device(dev):
        mm = torch.empty(2, dtype=torch.float32, device=dev)
        ws = _lib.minmax_workspace(dev)
        _lib.check(_lib.load().lq_minmax(_lib.ptr(xc), _lib.code_of(xc.dtype), 1, xc.numel(),
                                         _lib.PER_TENSOR, mm.data_ptr(), mm.data_ptr() + 4,
                                         _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    lo, hi = mm.tolist()
    return lo, hi


def histc(x: torch.Tensor, bins: int = 100, min: float = 0.0, max: float = 0.0):  # noqa: A002
    """Counts of ``x`` in ``bins`` equal-width bins over ``[min, max]`` as float32
    (lucid/_C/ops/composite/Stats.cpp:47-91).  An empty range (``min == max``) is taken from
    the data, and a constant tensor gets ``[v, v + 1]``."""
    xc = _check_observed(x)
    lo, hi = float(min), float(max)
    if lo == hi:
        lo, hi = _range_of(xc)
        if lo == hi:
            hi = lo + 1.0
    return _histc_launch(xc, bins, lo, hi)[0]


def _quantile_from_hist(counts, centres, q):
    """Centre of the first bin at which the cumulative mass reaches ``q``
    (lucid/quantization/observer.py:883-894)."""
    total = sum(counts)
    if total <= 0:
        return centres[0]
    target, acc = q * total, 0.0
    for centre, n in zip(centres, counts):
        acc += n
        if acc >= target:
            return centre
    return centres[-1]


class HistogramObserver(ObserverBase):
    """Running histogram of the observed values; the quantization range is the tail clip
    with the smallest clip + rounding L2 error (lucid/quantization/observer.py:773-880).

    The state (``min_val``, ``max_val``, ``histogram``) lives on the device and a step is two
    kernel launches with no host synchronisation: the batch is binned on the current range
    while its own range is measured, and binned again only if the range grew (the reference
    reads both ranges back to the host every batch and makes three passes)."""

    _CLIP_FRACTIONS = (0.0, 1e-5, 1e-4, 1e-3, 5e-3, 1e-2)

    def __init__(self, bins: int = 2048, qscheme=per_tensor_affine, qdtype=quint8,
                 eps: float = 1e-8):
        super().__init__(qscheme, qdtype, None, eps)
        self.bins = bins
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))
        self.register_buffer("histogram", torch.zeros(bins))

    def _host_range(self):
        return float(self.min_val), float(self.max_val)

    def forward(self, x):
        xc = _check_observed(x)
        dev = xc.device
        if self.histogram.device != dev or self.min_val.device != dev or self.max_val.device != dev:
            self.to(dev)
        for name in ("min_val", "max_val", "histogram"):
            t = getattr(self, name)
            if t.dtype != torch.float32 or not t.is_contiguous():
                setattr(self, name, t.to(torch.float32).contiguous())
        with torch.cuda.device(dev):
            ws = _lib.histc_workspace(dev)
            _lib.check(_lib.load().lq_histogram_observe(
                _lib.ptr(xc), _lib.code_of(xc.dtype), xc.numel(), int(self.bins),
                _lib.ptr(self.min_val), _lib.ptr(self.max_val), _lib.ptr(self.histogram),
                _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
        return x

    def _search_clip_range(self):
        lo, hi = self._host_range()
        counts = self.histogram.tolist()
        total = sum(counts)
        if total <= 0.0 or hi <= lo:
            return lo, hi
        bins = self.bins
        width = (hi - lo) / bins
        centres = [lo + (i + 0.5) * width for i in range(bins)]
        levels = self.qdtype.quant_max - self.qdtype.quant_min
        occupied = [(c, n) for c, n in zip(centres, counts) if n != 0.0]
        best_err, best = float("inf"), (lo, hi)
        for frac in self._CLIP_FRACTIONS:
            cmin = _quantile_from_hist(counts, centres, frac)
            cmax = _quantile_from_hist(counts, centres, 1.0 - frac)
            if cmax <= cmin:
                continue
            step = (cmax - cmin) / max(levels, 1)
            rounding = (step * step) / 12.0
            err = 0.0
            for c, n in occupied:
                clipped = cmin if c < cmin else (cmax if c > cmax else c)
                err += n * ((c - clipped) ** 2 + rounding)
            if err < best_err:
                best_err, best = err, (cmin, cmax)
        return best

    def calculate_qparams(self):
        cmin, cmax = self._search_clip_range()
        dev = self.histogram.device
        return calculate_qparams(torch.tensor(float(cmin), device=dev),
                                 torch.tensor(float(cmax), device=dev),
                                 self.qscheme, self.qdtype, self.eps)
