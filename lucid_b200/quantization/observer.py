"""Range observers on device (lucid/quantization/observer.py:364-375, 635-648).

Only the two observers on the hot path are provided: the per-tensor running
min/max and the per-channel running min/max.  Each observation is one
reduction kernel (the reference runs two full reductions per call)."""

from __future__ import annotations

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
        import functools

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
