"""Group-wise weight-only codes and the fused decode matmul
(lucid/quantization/_qgemm.py:24-320).  In the reference these wrap the Metal-only MLX ops; here
they are CUDA kernels of this library: ``quantize`` packs a float ``(out, in)`` weight into
``bits``-wide codes with one affine ``(scale, bias)`` per ``group_size`` input positions,
``dequantize`` inverts the packing, ``quantized_matmul`` contracts a float activation against
the packed weight without materialising it (built for decode shapes: a few activation rows)."""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib

_GROUPS = (32, 64, 128)


def is_available() -> bool:
    """The group-wise kernels are part of the library (lucid/quantization/_qgemm.py:24-66)."""
    return _lib.is_available()


def _check(bits: int, group_size: int, in_features: int) -> None:
    if bits not in (4, 8):
        raise NotImplementedError(f"bits must be 4 or 8, got {bits}")
    if group_size not in _GROUPS:
        raise NotImplementedError(f"group_size must be one of {_GROUPS}, got {group_size}")
    if in_features % group_size != 0:
        raise _lib.ShapeMismatch(f"in_features {in_features} is not a multiple of group_size {group_size}")


def quantize(w: torch.Tensor, group_size: int = 64, bits: int = 8):
    """``(packed_weight int32 (out, in * bits / 32), scales (out, in / group), biases)``
    (lucid/quantization/_qgemm.py:69-152).  The packed words are tagged int32 as in the
    reference; their bit patterns are the little-endian codes."""
    _lib.require_cuda(w, "weight")
    if w.dim() != 2:
        raise _lib.ShapeMismatch(f"weight must be (out, in), got {tuple(w.shape)}")
    n, k = w.shape
    _check(bits, group_size, k)
    wf = w.detach().to(torch.float32).contiguous()
    packed = torch.empty((n, k * bits // 32), dtype=torch.int32, device=w.device)
    scales = torch.empty((n, k // group_size), dtype=torch.float32, device=w.device)
    biases = torch.empty_like(scales)
    with torch.cuda.device(w.device):
        _lib.check(_lib.load().lq_groupwise_quantize(_lib.ptr(wf), n, k, group_size, bits, _lib.ptr(packed),
                                                     _lib.ptr(scales), _lib.ptr(biases), _lib.stream_ptr(w.device)))
    return packed, scales, biases


def dequantize(wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64, bits: int = 8):
    """``w_hat = code * scale + bias`` as float32 ``(out, in)`` (lucid/quantization/_qgemm.py:155-225)."""
    _lib.require_cuda(wq, "packed weight")
    n = wq.shape[0]
    k = wq.shape[1] * 32 // bits
    _check(bits, group_size, k)
    if tuple(scales.shape) != (n, k // group_size) or tuple(biases.shape) != tuple(scales.shape):
        raise _lib.ShapeMismatch("scales / biases do not match the packed weight")
    out = torch.empty((n, k), dtype=torch.float32, device=wq.device)
    with torch.cuda.device(wq.device):
        _lib.check(_lib.load().lq_groupwise_dequantize(_lib.ptr(wq.contiguous()), _lib.ptr(scales.contiguous()),
                                                       _lib.ptr(biases.contiguous()), n, k, group_size, bits,
                                                       _lib.ptr(out), _lib.stream_ptr(wq.device)))
    return out


def quantized_matmul(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                     transpose: bool = True, group_size: int = 64, bits: int = 8, bias: torch.Tensor | None = None,
                     relu: bool = False) -> torch.Tensor:
    """``x @ w_hat.T`` with the weight decoded inside the kernel
    (lucid/quantization/_qgemm.py:228-320); ``bias`` / ``relu`` fold the caller's epilogue into
    the same launch.  float32 or bfloat16 activations; the result has the activation's dtype."""
    if not transpose:
        raise NotImplementedError("quantized_matmul(transpose=False): the packed weight is stored (out, in); "
                                  "use dequantize() and a float matmul")
    _lib.require_cuda(x, "activation")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.DtypeMismatch(f"activation must be float32 or bfloat16, got {x.dtype}")
    n = wq.shape[0]
    k = wq.shape[1] * 32 // bits
    _check(bits, group_size, k)
    if x.shape[-1] != k:
        raise _lib.ShapeMismatch(f"activation has {x.shape[-1]} features, the weight {k}")
    x2 = x.reshape(-1, k).contiguous()
    m = x2.shape[0]
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    b = None if bias is None else bias.to(torch.float32).contiguous()
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().lq_groupwise_matmul(
            _lib.ptr(x2), _lib.code_of(x2.dtype), m, k, _lib.ptr(wq.contiguous()), _lib.ptr(scales.contiguous()),
            _lib.ptr(biases.contiguous()), n, k, group_size, bits, None if b is None else _lib.ptr(b), int(relu),
            _lib.ptr(out), n, _lib.stream_ptr(x.device)))
    return out.reshape(*x.shape[:-1], n)
