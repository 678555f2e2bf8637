"""quantize / dequantize / fake_quantize on B200
(lucid/quantization/_functional.py:57-182, 185-281, 284-448).

Each call is ONE pass over HBM (the reference makes six); results are bit-exact
with the reference's f32 composite: true division, ties-to-even, compare clip.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from .. import _lib
from ._qscheme import QDtype


def _view2d(x: torch.Tensor, ch_axis, per_channel: bool):
    """Collapse ``x`` to (rows, cols) so the channel axis is the row or the
    column index.  Returns (rows, cols, mode, repeat) where ``repeat`` says how
    often a per-channel vector must be tiled to index rows directly."""
    n = x.numel()
    if not per_channel or x.dim() == 0:
        cols = x.shape[-1] if x.dim() > 0 else 1
        return (n // cols if cols else 0), cols, _lib.PER_TENSOR, 1
    ax = ch_axis % x.dim()
    ch = x.shape[ax]
    if ax == x.dim() - 1:
        return (n // ch if ch else 0), ch, _lib.PER_COL, 1
    inner = math.prod(x.shape[ax + 1:])
    outer = math.prod(x.shape[:ax])
    return outer * ch, inner, _lib.PER_ROW, outer


def _prepare_params(x, scale, zero_point, ch_axis):
    """Mirror of the reference's device alignment and per-channel broadcast
    (lucid/quantization/_functional.py:166-179)."""
    s_is_t = isinstance(scale, torch.Tensor)
    z_is_t = isinstance(zero_point, torch.Tensor)
    per_channel = ch_axis is not None and s_is_t and scale.numel() > 1
    rows, cols, mode, repeat = _view2d(x, ch_axis, per_channel)
    if not s_is_t and not z_is_t:
        return rows, cols, mode, None, None, float(scale), float(zero_point)
    dev = x.device
    s = scale.detach().to(device=dev, dtype=torch.float32) if s_is_t else \
        torch.tensor(float(scale), dtype=torch.float32, device=dev)
    if z_is_t:
        z = zero_point.detach().to(device=dev, dtype=torch.float32)
    else:
        z = torch.full_like(s, float(zero_point))
    s = s.reshape(-1)
    z = z.reshape(-1)
    if z.numel() != s.numel():
        z = z.expand_as(s) if z.numel() == 1 else z
        s = s.expand_as(z) if s.numel() == 1 else s
    if per_channel:
        ch = x.shape[ch_axis % x.dim()]
        if s.numel() != ch:
            raise _lib.ShapeMismatch(
                f"per-channel scale has {s.numel()} entries but axis {ch_axis} has {ch}")
        if repeat > 1:
            s, z = s.repeat(repeat), z.repeat(repeat)
    elif s.numel() != 1:
        raise _lib.ShapeMismatch("a multi-element scale needs ch_axis")
    return rows, cols, mode, s.contiguous(), z.contiguous(), 0.0, 0.0


def _input(x, what, dtypes):
    _lib.require_cuda(x, what)
    if x.dtype not in dtypes:
        raise _lib.DtypeMismatch(f"{what} has dtype {x.dtype}; expected one of {dtypes}")
    return x.detach().contiguous()


def quantize(x, scale, zero_point, qdtype: QDtype, ch_axis=None) -> torch.Tensor:
    """``clip(round(x / s) + z, qmin, qmax)`` as integer codes in
    ``qdtype.storage`` (int8; int16 for quint8)."""
    xc = _input(x, "quantize input", (torch.float32, torch.bfloat16))
    rows, cols, mode, s, z, sv, zv = _prepare_params(xc, scale, zero_point, ch_axis)
    out = torch.empty(xc.shape, dtype=qdtype.torch_storage, device=xc.device)
    with torch.cuda.device(xc.device):
        _lib.check(_lib.load().lq_quantize(
            _lib.ptr(xc), _lib.code_of(xc.dtype), rows, cols, _lib.ptr(s), _lib.ptr(z),
            C.c_float(sv), C.c_float(zv), mode, qdtype.quant_min, qdtype.quant_max,
            _lib.ptr(out), _lib.code_of(out.dtype), _lib.stream_ptr(xc.device)))
    return out


def quantize_to(x, scale, zero_point, quant_min, quant_max, out_dtype, ch_axis=None):
    """Same arithmetic with an explicit storage dtype (torch.int8 / uint8 /
    int16): the form the integer GEMM consumes (u8 codes stay u8)."""
    xc = _input(x, "quantize input", (torch.float32, torch.bfloat16))
    rows, cols, mode, s, z, sv, zv = _prepare_params(xc, scale, zero_point, ch_axis)
    out = torch.empty(xc.shape, dtype=out_dtype, device=xc.device)
    with torch.cuda.device(xc.device):
        _lib.check(_lib.load().lq_quantize(
            _lib.ptr(xc), _lib.code_of(xc.dtype), rows, cols, _lib.ptr(s), _lib.ptr(z),
            C.c_float(sv), C.c_float(zv), mode, quant_min, quant_max, _lib.ptr(out),
            _lib.code_of(out_dtype), _lib.stream_ptr(xc.device)))
    return out


def dequantize(q, scale, zero_point, ch_axis=None, out_dtype=torch.float32) -> torch.Tensor:
    """``(float32(q) - z) * s``; float32 like the reference (bf16 on request:
    the f32 result rounded once)."""
    qc = _input(q, "dequantize input", (torch.int8, torch.uint8, torch.int16))
    rows, cols, mode, s, z, sv, zv = _prepare_params(qc, scale, zero_point, ch_axis)
    out = torch.empty(qc.shape, dtype=out_dtype, device=qc.device)
    with torch.cuda.device(qc.device):
        _lib.check(_lib.load().lq_dequantize(
            _lib.ptr(qc), _lib.code_of(qc.dtype), rows, cols, _lib.ptr(s), _lib.ptr(z),
            C.c_float(sv), C.c_float(zv), mode, _lib.ptr(out), _lib.code_of(out_dtype),
            _lib.stream_ptr(qc.device)))
    return out


def _fake_quantize_forward(x, scale, zero_point, quant_min, quant_max, ch_axis, want_mask):
    xc = _input(x, "fake_quantize input", (torch.float32,))
    rows, cols, mode, s, z, sv, zv = _prepare_params(xc, scale, zero_point, ch_axis)
    out = torch.empty_like(xc)
    mask = torch.empty_like(xc) if want_mask else None
    with torch.cuda.device(xc.device):
        _lib.check(_lib.load().lq_fake_quantize(
            _lib.ptr(xc), rows, cols, _lib.ptr(s), _lib.ptr(z), C.c_float(sv), C.c_float(zv),
            mode, int(quant_min), int(quant_max), _lib.ptr(out), _lib.ptr(mask),
            _lib.stream_ptr(xc.device)))
    return out, mask


class _FakeQuantizeAffine(torch.autograd.Function):
    """Straight-through estimator: gradient passes where the code did not
    saturate (lucid/quantization/_functional.py:284-331)."""

    @staticmethod
    def forward(ctx, x, scale, zero_point, quant_min, quant_max, ch_axis):
        out, mask = _fake_quantize_forward(x, scale, zero_point, quant_min, quant_max, ch_axis, True)
        ctx.save_for_backward(mask)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (mask,) = ctx.saved_tensors
        return grad_out * mask, None, None, None, None, None


def fake_quantize(x, scale, zero_point, quant_min, quant_max, ch_axis=None) -> torch.Tensor:
    """``dequantize(quantize(x))`` in one pass, float in / float out."""
    if isinstance(x, torch.Tensor) and x.requires_grad and torch.is_grad_enabled():
        return _FakeQuantizeAffine.apply(x, scale, zero_point, quant_min, quant_max, ch_axis)
    out, _ = _fake_quantize_forward(x, scale, zero_point, quant_min, quant_max, ch_axis, False)
    return out


def quantize_dynamic_per_tensor(x, qdtype: QDtype, symmetric: bool = False, eps: float = 1e-8):
    """Per-tensor encode on the live range in one native call: min/max -> calculate_qparams ->
    quantize.  Returns ``(codes (int8 | uint8), scale, zero_point)``, the latter two 0-d device
    tensors (nothing is synchronised)."""
    xc = _input(x, "dynamic encode input", (torch.float32, torch.bfloat16))
    if xc.numel() == 0:
        raise _lib.ShapeMismatch("cannot observe an empty tensor")
    dev = xc.device
    store = torch.int8 if qdtype.signed else torch.uint8
    out = torch.empty(xc.shape, dtype=store, device=dev)
    small = torch.empty(4, dtype=torch.float32, device=dev)  # scale, zp, min, max
    cols = xc.shape[-1] if xc.dim() > 0 else 1
    with torch.cuda.device(dev):
        ws = _lib.minmax_workspace(dev)
        _lib.check(_lib.load().lq_quantize_dynamic(
            _lib.ptr(xc), _lib.code_of(xc.dtype), xc.numel() // cols, cols, int(symmetric),
            int(qdtype.signed), qdtype.quant_min, qdtype.quant_max, C.c_float(eps), _lib.ptr(ws),
            ws.numel(), _lib.ptr(out), _lib.code_of(store), C.c_void_p(small.data_ptr()),
            C.c_void_p(small.data_ptr() + 4), C.c_void_p(small.data_ptr() + 8), _lib.stream_ptr(dev)))
    return out, small[0], small[1]


def quantize_per_token(x, qdtype: QDtype, eps: float = 1e-8):
    """Per-token (row of the last axis) symmetric encode in one HBM pass.

    Equals ``PerChannelMinMaxObserver(ch_axis=0)`` -> ``calculate_qparams`` ->
    ``quantize(ch_axis=0)`` on the ``(tokens, features)`` matrix.  Returns
    ``(int8 codes, f32 scales[tokens])``."""
    if not qdtype.signed or qdtype.quant_min < -128 or qdtype.quant_max > 127:
        raise _lib.DtypeMismatch("per-token encode needs a signed grid inside int8")
    xc = _input(x, "per-token input", (torch.float32, torch.bfloat16))
    cols = xc.shape[-1]
    rows = xc.numel() // cols if cols else 0
    out = torch.empty(xc.shape, dtype=torch.int8, device=xc.device)
    scales = torch.empty(xc.shape[:-1], dtype=torch.float32, device=xc.device)
    with torch.cuda.device(xc.device):
        _lib.check(_lib.load().lq_quantize_per_token(
            _lib.ptr(xc), _lib.code_of(xc.dtype), rows, cols, qdtype.quant_min, qdtype.quant_max,
            C.c_float(eps), _lib.ptr(out), _lib.ptr(scales), _lib.stream_ptr(xc.device)))
    return out, scales
