"""``calculate_qparams`` on device (lucid/quantization/_qparams.py:93-215)."""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _lib
from ._qscheme import QDtype, QScheme


@dataclass(frozen=True)
class QParams:
    """Bundle of a calibrated grid (lucid/quantization/_qparams.py:22-90)."""

    scale: torch.Tensor
    zero_point: torch.Tensor
    qscheme: QScheme
    qdtype: QDtype
    ch_axis: int | None = None


def _as_cuda_f32(v, like=None) -> torch.Tensor:
    if isinstance(v, torch.Tensor):
        _lib.require_cuda(v, "range tensor")
        return v.detach().to(torch.float32).contiguous()
    dev = like.device if like is not None else torch.device("cuda", torch.cuda.current_device())
    return torch.tensor(float(v), dtype=torch.float32, device=dev)


def calculate_qparams(min_val, max_val, qscheme: QScheme, qdtype: QDtype, eps: float = 1e-8):
    """(scale, zero_point) from an observed range; both f32 tensors shaped like
    the inputs, ``zero_point`` integer-valued.  One kernel, same f32 op order as
    the reference's tensor composite."""
    like = min_val if isinstance(min_val, torch.Tensor) else (
        max_val if isinstance(max_val, torch.Tensor) else None)
    mn = _as_cuda_f32(min_val, like)
    mx = _as_cuda_f32(max_val, like)
    if mn.shape != mx.shape:
        mn, mx = torch.broadcast_tensors(mn, mx)
        mn, mx = mn.contiguous(), mx.contiguous()
    scale = torch.empty_like(mn)
    zp = torch.empty_like(mn)
    with torch.cuda.device(mn.device):
        _lib.check(_lib.load().lq_calculate_qparams(
            _lib.ptr(mn), _lib.ptr(mx), mn.numel(), int(qscheme.is_symmetric), int(qdtype.signed),
            qdtype.quant_min, qdtype.quant_max, C.c_float(eps), _lib.ptr(scale), _lib.ptr(zp),
            _lib.stream_ptr(mn.device)))
    return scale, zp
