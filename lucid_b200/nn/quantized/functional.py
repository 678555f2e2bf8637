"""Integer contraction entry points (tensor-level wrappers over the C ABI).

``gemm_s8`` / ``conv2d_nhwc_s8`` compute exact int32 accumulators on the
tcgen05 tensor cores and apply the fused epilogue documented in
``include/lucid_b200.h``.  They are what the quantized modules call in place of
the reference's dequantize -> float GEMM -> fake-quantize sequence
(lucid/nn/quantized/linear.py:199-215, lucid/nn/quantized/conv.py:168-184).
"""

from __future__ import annotations

import ctypes as C

import torch

from ... import _lib

_OUT_CODE = {torch.int32: _lib.S32, torch.float32: _lib.F32, torch.bfloat16: _lib.BF16,
             torch.int8: _lib.S8, torch.uint8: _lib.U8}


def _f32(t, dev, what):
    if t is None:
        return None
    if not isinstance(t, torch.Tensor):
        t = torch.tensor(float(t), dtype=torch.float32, device=dev)
    if t.device != dev:
        t = t.to(dev)
    if t.dtype != torch.float32:
        t = t.to(torch.float32)
    return t.contiguous()


def _need(t, count, what):
    if t is not None and t.numel() != count:
        raise _lib.ShapeMismatch(f"{what} has {t.numel()} entries, expected {count}")


def _check_out(out, rows, cols, dev, what):
    """`out=` of the contraction wrappers: the kernel writes rows x cols elements at the row
    stride of `out`, so anything smaller, of another dtype or on another device is refused."""
    if not isinstance(out, torch.Tensor) or not out.is_cuda or out.device != dev:
        raise _lib.DeviceMismatch(f"{what}: out= must be a CUDA tensor on {dev}")
    if out.dtype not in _OUT_CODE:
        raise _lib.DtypeMismatch(f"{what}: unsupported output dtype {out.dtype}")
    if out.dim() != 2 or out.shape[0] != rows or out.shape[1] != cols:
        raise _lib.ShapeMismatch(f"{what}: out= is {tuple(out.shape)}, expected {(rows, cols)}")
    if out.stride(1) != 1 or out.stride(0) < cols:
        raise _lib.ShapeMismatch(f"{what}: out= must have unit column stride and a row stride >= {cols}")


def _epilogue(dev, out_dtype, act, a_scale, a_zp, b_rowsum, b_scale, bias, out_scale, out_zp,
              qmin, qmax, keep, m=None, n=None):
    """Marshal the epilogue descriptor.  `m` / `n` (rows of the activation operand, rows of the
    weight operand) bound every per-row / per-channel vector the kernel will index."""
    if out_dtype not in _OUT_CODE:
        raise _lib.DtypeMismatch(f"unsupported GEMM output dtype {out_dtype}")
    a_scale = _f32(a_scale, dev, "a_scale")
    a_zp = _f32(a_zp, dev, "a_zp")
    b_scale = _f32(b_scale, dev, "b_scale")
    bias = _f32(bias, dev, "bias")
    out_scale = _f32(out_scale, dev, "out_scale")
    out_zp = _f32(out_zp, dev, "out_zp")
    if b_rowsum is not None:
        b_rowsum = b_rowsum.to(device=dev, dtype=torch.int32).contiguous()
    keep.extend([a_scale, a_zp, b_rowsum, b_scale, bias, out_scale, out_zp])
    if m is not None and a_scale is not None and a_scale.numel() not in (1, m):
        raise _lib.ShapeMismatch(f"a_scale has {a_scale.numel()} entries, expected 1 or {m}")
    if n is not None:
        _need(b_scale, n, "b_scale"), _need(bias, n, "bias"), _need(b_rowsum, n, "b_rowsum")
    _need(a_zp, 1, "a_zp"), _need(out_scale, 1, "out_scale"), _need(out_zp, 1, "out_zp")
    e = _lib.Epilogue()
    e.out_dtype = _OUT_CODE[out_dtype]
    e.act = act
    e.a_scale_mode = _lib.PER_ROW if (a_scale is not None and a_scale.numel() > 1) else _lib.PER_TENSOR
    e.qmin, e.qmax = int(qmin), int(qmax)
    e.a_scale = _lib.ptr(a_scale)
    e.a_zp = _lib.ptr(a_zp)
    e.b_rowsum = _lib.ptr(b_rowsum)
    e.b_scale = _lib.ptr(b_scale)
    e.bias = _lib.ptr(bias)
    e.out_scale = _lib.ptr(out_scale)
    e.out_zp = _lib.ptr(out_zp)
    return e


def rowsum_s8(b: torch.Tensor) -> torch.Tensor:
    """``sum_k b[n, k]`` as int32: the zero-point correction vector."""
    _lib.require_cuda(b, "weight codes")
    if b.dtype != torch.int8:
        raise _lib.DtypeMismatch("weight codes must be int8")
    b2 = b.contiguous().reshape(b.shape[0], -1)
    out = torch.empty(b2.shape[0], dtype=torch.int32, device=b.device)
    with torch.cuda.device(b.device):
        _lib.check(_lib.load().lq_rowsum_s8(_lib.ptr(b2), b2.shape[0], b2.shape[1], _lib.ptr(out),
                                            _lib.stream_ptr(b.device)))
    return out


def gemm_s8(a, b, *, out_dtype=torch.int32, a_scale=None, a_zp=None, b_rowsum=None, b_scale=None,
            bias=None, act=_lib.ACT_NONE, out_scale=None, out_zp=None, qmin=0, qmax=0, out=None):
    """``epilogue(a @ b.T)`` for 8-bit codes ``a (M, K)`` (int8 or uint8) and
    ``b (N, K)`` (int8).  ``a_scale`` scalar (per tensor) or ``M`` values (per
    token)."""
    _lib.require_cuda(a, "activation codes")
    _lib.require_cuda(b, "weight codes")
    if a.dtype not in (torch.int8, torch.uint8) or b.dtype != torch.int8:
        raise _lib.DtypeMismatch("gemm_s8 takes int8/uint8 activations and int8 weights")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise _lib.ShapeMismatch(f"gemm_s8 shapes {tuple(a.shape)} x {tuple(b.shape)}^T")
    a = a.contiguous()
    b = b.contiguous()
    m, k = a.shape
    n = b.shape[0]
    n_out = n // 2 if act == _lib.ACT_SILU_GATE else n
    dev = a.device
    if out is None:
        out = torch.empty((m, n_out), dtype=out_dtype, device=dev)
    else:
        _check_out(out, m, n_out, dev, "gemm_s8")
    keep: list = []
    e = _epilogue(dev, out.dtype, act, a_scale, a_zp, b_rowsum, b_scale, bias, out_scale, out_zp,
                  qmin, qmax, keep, m, n)
    with torch.cuda.device(dev):
        ws = _lib.gemm_workspace(dev)
        _lib.check(_lib.load().lq_gemm_s8_ws(
            _lib.ptr(a), int(a.dtype == torch.int8), _lib.ptr(b), m, n, k, C.byref(e),
            _lib.ptr(out), out.stride(0), _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)),
            _lib.stream_ptr(dev)))
    return out


def gemm_s8_bcast(a, b, dst_ptrs, dst_shape, col0, *, out_dtype=torch.bfloat16, a_scale=None, a_zp=None,
                  b_rowsum=None, b_scale=None, bias=None, act=_lib.ACT_NONE, out_scale=None,
                  out_zp=None, qmin=0, qmax=0, signal=None):
    """`gemm_s8` whose epilogue stores every tile into several `(M, ld)` buffers at column
    offset `col0`: `dst_ptrs` are raw device addresses (this GPU's buffer first, then the same
    buffer on its peers, e.g. `_SymmetricMemory.buffer_ptrs`) or ONE int, the buffer's NVSwitch
    multicast address (`_SymmetricMemory.multicast_ptr`); `dst_shape = (M, ld)`.
    `signal = (flag_addresses, counter_tensor)`: when the last tile is stored the kernel bumps
    this rank's step counter and publishes it to the given flag words (this rank's word on every
    rank); consumers wait with `peer_wait`.  Without `signal` the caller synchronises the ranks
    before the buffers are read."""
    _lib.require_cuda(a, "activation codes")
    _lib.require_cuda(b, "weight codes")
    if a.dtype not in (torch.int8, torch.uint8) or b.dtype != torch.int8:
        raise _lib.DtypeMismatch("gemm_s8_bcast takes int8/uint8 activations and int8 weights")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise _lib.ShapeMismatch(f"gemm_s8_bcast shapes {tuple(a.shape)} x {tuple(b.shape)}^T")
    a = a.contiguous()
    b = b.contiguous()
    m, k = a.shape
    n = b.shape[0]
    n_out = n // 2 if act == _lib.ACT_SILU_GATE else n
    if dst_shape[0] < m or dst_shape[1] < col0 + n_out:
        raise _lib.ShapeMismatch(f"destination {tuple(dst_shape)} too small for rows {m}, columns "
                                 f"[{col0}, {col0 + n_out})")
    dev = a.device
    keep: list = []
    e = _epilogue(dev, out_dtype, act, a_scale, a_zp, b_rowsum, b_scale, bias, out_scale, out_zp,
                  qmin, qmax, keep, m, n)
    multicast = isinstance(dst_ptrs, int)  # an NVSwitch multicast address: one store reaches every rank
    plist = [dst_ptrs] if multicast else [int(p) for p in dst_ptrs]
    ptrs = (C.c_void_p * len(plist))(*plist)
    if signal is not None:
        flag_addrs, counter = signal
        flags = (C.c_void_p * len(flag_addrs))(*[int(p) for p in flag_addrs])
        n_flags, counter_ptr = len(flag_addrs), _lib.ptr(counter)
    else:
        flags, n_flags, counter_ptr = None, 0, None
    with torch.cuda.device(dev):
        ws = _lib.gemm_workspace(dev)
        _lib.check(_lib.load().lq_gemm_s8_sharded(
            _lib.ptr(a), int(a.dtype == torch.int8), _lib.ptr(b), m, n, k, C.byref(e), ptrs,
            -1 if multicast else len(plist), int(dst_shape[1]), int(col0), flags, n_flags, counter_ptr,
            _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)))


def peer_signal(flag_addrs, counter: torch.Tensor) -> None:
    """Publish this rank's next step count to its flag word on every rank (stream-ordered after
    the kernels that stored into the peers' buffers)."""
    dev = counter.device
    flags = (C.c_void_p * len(flag_addrs))(*[int(p) for p in flag_addrs])
    with torch.cuda.device(dev):
        _lib.check(_lib.load().lq_peer_signal(flags, len(flag_addrs), _lib.ptr(counter), _lib.stream_ptr(dev)))


def peer_wait(flags: torch.Tensor, epoch: torch.Tensor, timeout_cycles: int = 0) -> None:
    """Stream-ordered, bounded wait until every producer's flag word in `flags` reached this
    rank's next step count (`epoch` is bumped); a timeout lands in the device status word."""
    dev = flags.device
    with torch.cuda.device(dev):
        _lib.check(_lib.load().lq_peer_wait(_lib.ptr(flags), flags.numel(), _lib.ptr(epoch), int(timeout_cycles),
                                            _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)))


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def conv_out_size(size: int, k: int, stride: int, pad: int, dil: int) -> int:
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def conv2d_nhwc_s8(x, w_krsc, *, pad=0, stride=1, dilation=1, groups=1, out_hw=None, out_dtype=torch.int32,
                   a_scale=None, a_zp=None, b_rowsum=None, b_scale=None, bias=None, act=_lib.ACT_NONE,
                   out_scale=None, out_zp=None, qmin=0, qmax=0):
    """NHWC implicit-GEMM convolution on codes: ``x (N, H, W, C)`` int8/uint8, ``w_krsc (K, R, S,
    C / groups)`` int8.  ``pad`` is the padding before the first row / column (int or pair);
    ``out_hw`` overrides the output extent (an asymmetric "same" padding is the leading padding
    plus a larger output).  Out-of-image taps read code 0, so a non-zero activation zero point
    (``a_zp`` with ``b_rowsum``) is accepted only for geometries that read no such tap.
    Returns ``(N, P, Q, K)``."""
    _lib.require_cuda(x, "activation codes")
    _lib.require_cuda(w_krsc, "weight codes")
    if x.dtype not in (torch.int8, torch.uint8) or w_krsc.dtype != torch.int8:
        raise _lib.DtypeMismatch("conv2d_nhwc_s8 takes int8/uint8 activations and int8 weights")
    if x.dim() != 4 or w_krsc.dim() != 4 or groups < 1 or x.shape[3] != w_krsc.shape[3] * groups:
        raise _lib.ShapeMismatch(f"conv2d_nhwc_s8 shapes {tuple(x.shape)} * {tuple(w_krsc.shape)}, groups {groups}")
    x = x.contiguous()
    w_krsc = w_krsc.contiguous()
    n, h, w, c = x.shape
    k, r, s, _ = w_krsc.shape
    (ph, pw), (sh, sw), (dh, dw) = _pair(pad), _pair(stride), _pair(dilation)
    if out_hw is None:
        p, q = conv_out_size(h, r, sh, ph, dh), conv_out_size(w, s, sw, pw, dw)
    else:
        p, q = int(out_hw[0]), int(out_hw[1])
    if p < 1 or q < 1:
        raise _lib.ShapeMismatch(f"conv2d_nhwc_s8: empty output ({p}, {q})")
    dev = x.device
    out = torch.empty((n, p, q, k), dtype=out_dtype, device=dev)
    keep: list = []
    e = _epilogue(dev, out_dtype, act, a_scale, a_zp, b_rowsum, b_scale, bias, out_scale, out_zp,
                  qmin, qmax, keep, None, k)
    g = _lib.ConvGeometry(N=n, H=h, W=w, C=c, K=k, R=r, S=s, P=p, Q=q, stride_h=sh, stride_w=sw, pad_h=ph,
                          pad_w=pw, dil_h=dh, dil_w=dw, groups=groups)
    with torch.cuda.device(dev):
        ws = _lib.gemm_workspace(dev)
        _lib.check(_lib.load().lq_conv2d_nhwc_s8_ex(
            _lib.ptr(x), int(x.dtype == torch.int8), _lib.ptr(w_krsc), C.byref(g), C.byref(e), _lib.ptr(out),
            _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)))
    return out
