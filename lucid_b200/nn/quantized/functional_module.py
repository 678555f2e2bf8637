"""Quantizable element-wise merges (lucid/nn/quantized/functional_module.py:26-260):
``FloatFunctional`` marks a residual add / mul / cat so ``prepare`` can observe its output,
``QFunctional`` snaps the result to the calibrated grid.

Each merge is one kernel (``lq_qmerge``): operands that carry 8-bit codes are read as codes
(one byte per element) and decoded in registers, the op, the ReLU and the encode follow in the
reference's float32 order, and the result leaves as codes plus the fake-quantized float tensor
the reference returns."""

from __future__ import annotations

import ctypes as C

import torch

from ... import _lib
from ...quantization import QDtype, quint8
from ._utils import QCodes, activation_qparams, codes_of, tag


class FloatFunctional(torch.nn.Module):
    """Float merges whose result feeds the attached observer (identity before ``prepare``)."""

    def _obs(self, x):
        app = getattr(self, "activation_post_process", None)
        if app is not None:
            app(x.detach().to(torch.float32).contiguous())
        return x

    def add(self, x, y):
        return self._obs(x + y)

    def mul(self, x, y):
        return self._obs(x * y)

    def add_relu(self, x, y):
        return self._obs(torch.relu(x + y))

    def cat(self, tensors, dim: int = 0):
        return self._obs(torch.cat(list(tensors), dim=dim))

    def add_scalar(self, x, scalar: float):
        return self._obs(x + scalar)

    def mul_scalar(self, x, scalar: float):
        return self._obs(x * scalar)


def _operand(t):
    """(pointer tensor, dtype code, scale, zero_point, layout) of a merge operand: its codes
    when it carries 8-bit ones, else its float values."""
    qc = codes_of(t)
    if qc is not None and qc.codes.dtype in (torch.int8, torch.uint8) and qc.scale.dim() == 0:
        c = qc.codes.contiguous()
        return c, _lib.code_of(c.dtype), qc.scale, qc.zero_point, qc.layout
    _lib.require_cuda(t, "merge operand")
    v = t.detach()
    if v.dtype not in (torch.float32, torch.bfloat16):
        v = v.to(torch.float32)
    return v.contiguous(), _lib.code_of(v.dtype), None, None, "rowmajor"


def _launch_qmerge(op, xa, xd, xs, xz, ya, yd, ys, yz, scalar, s, z, qdtype, codes, out):
    dev = xa.device
    with torch.cuda.device(dev):
        _lib.check(_lib.load().lq_qmerge(
            op, _lib.ptr(xa), xd, _lib.ptr(xs), _lib.ptr(xz), _lib.ptr(ya), yd, _lib.ptr(ys), _lib.ptr(yz),
            C.c_float(scalar), xa.numel(), _lib.ptr(s), _lib.ptr(z), qdtype.quant_min, qdtype.quant_max,
            _lib.ptr(codes), _lib.code_of(codes.dtype) if codes is not None else _lib.S8, _lib.ptr(out),
            _lib.stream_ptr(dev)))


def _ver(t):
    return (t.data_ptr(), t._version)


class _TableCache:
    """Tables of a merge site, rebuilt when a grid it was made for changes: 256 bytes for a
    unary op on codes (scalar operand, requantization), 64 KB for a binary op on two code
    tensors.  The entries are produced by the exact kernel itself, so streaming through the
    table equals running that kernel on the tensors."""

    def __init__(self):
        self._key, self._tab = None, None

    def get(self, key, make):
        if key != self._key:
            self._key, self._tab = key, make()
        return self._tab


def _all_bytes(dtype, dev):
    raw = torch.arange(256, device=dev, dtype=torch.int32).to(torch.uint8)
    return raw.view(torch.int8) if dtype == torch.int8 else raw


def qmerge(op: int, x, y, scale, zero_point, qdtype: QDtype = quint8, cache: _TableCache | None = None):
    """``fake_quantize(op(x, y))`` on the grid ``(scale, zero_point, qdtype)``; ``y`` is a tensor
    or a Python scalar.  Returns the float tensor tagged with its codes."""
    xa, xd, xs, xz, layout = _operand(x)
    scalar = 0.0
    if isinstance(y, torch.Tensor):
        ya, yd, ys, yz, ylayout = _operand(y)
        if layout != ylayout:  # one operand carries NHWC codes, the other does not: use values
            xa, xd, xs, xz, layout = _operand(x.detach().view_as(x))
            ya, yd, ys, yz, _ = _operand(y.detach().view_as(y))
        if ya.shape != xa.shape:
            raise _lib.ShapeMismatch(f"merge operands differ in shape: {tuple(xa.shape)} vs {tuple(ya.shape)}")
    else:
        ya, yd, ys, yz = None, _lib.F32, None, None
        scalar = 0.0 if y is None else float(y)
    dev = xa.device
    store = torch.int8 if qdtype.signed else torch.uint8
    eight_bit = qdtype.bits <= 8
    codes = torch.empty(xa.shape, dtype=store, device=dev) if eight_bit else None
    out = torch.empty(xa.shape, dtype=torch.float32, device=dev)
    s = scale.to(device=dev, dtype=torch.float32)
    z = zero_point.to(device=dev, dtype=torch.float32)
    x_coded = xs is not None and xa.dtype in (torch.int8, torch.uint8)
    y_coded = ya is not None and ys is not None and ya.dtype in (torch.int8, torch.uint8)
    if cache is not None and codes is not None and x_coded and (y_coded or ya is None) and xa.numel() >= 1 << 16:
        # functions of one or two bytes: stream the codes through a table
        key = (op, xa.dtype, _ver(xs), _ver(xz), _ver(s), _ver(z), qdtype.name, scalar,
               (ya.dtype, _ver(ys), _ver(yz)) if y_coded else None)
        if y_coded:
            def make():
                bx, by = _all_bytes(xa.dtype, dev), _all_bytes(ya.dtype, dev)
                tab = torch.empty(65536, dtype=store, device=dev)
                _launch_qmerge(op, bx.repeat_interleave(256).contiguous(), xd, xs, xz, by.repeat(256).contiguous(),
                               yd, ys, yz, 0.0, s, z, qdtype, tab, None)
                return tab
            tab = cache.get(key, make)
            with torch.cuda.device(dev):
                _lib.check(_lib.load().lq_lut2_u8(_lib.ptr(xa), _lib.ptr(ya), xa.numel(), _lib.ptr(tab),
                                                  _lib.ptr(codes), _lib.ptr(out), _lib.ptr(s), _lib.ptr(z),
                                                  int(qdtype.signed), _lib.stream_ptr(dev)))
        else:
            def make():
                tab = torch.empty(256, dtype=store, device=dev)
                _launch_qmerge(op, _all_bytes(xa.dtype, dev), xd, xs, xz, None, _lib.F32, None, None, scalar, s, z,
                               qdtype, tab, None)
                return tab
            tab = cache.get(key, make)
            from ...quantization import dequantize

            with torch.cuda.device(dev):
                _lib.check(_lib.load().lq_lut_u8(_lib.ptr(xa), xa.numel(), _lib.ptr(tab), _lib.ptr(codes),
                                                 _lib.stream_ptr(dev)))
            out = dequantize(codes, s, z)
    else:
        _launch_qmerge(op, xa, xd, xs, xz, ya, yd, ys, yz, scalar, s, z, qdtype, codes, out)
    if layout == "nhwc":  # codes are NHWC; the float carrier is the logical NCHW view of them
        out = out.permute(0, 3, 1, 2)
    elif layout == "nlc":  # 1-D convolutions: codes (N, L, C), carrier (N, C, L)
        out = out.permute(0, 2, 1)
    if codes is None:
        return out
    return tag(out, QCodes(codes, s, z, layout))


class QFunctional(torch.nn.Module):
    """Merges snapped to one calibrated grid (functional_module.py:127-260)."""

    def __init__(self, scale, zero_point, qdtype: QDtype = quint8) -> None:
        super().__init__()
        self.register_buffer("scale", torch.as_tensor(scale, dtype=torch.float32))
        self.register_buffer("zero_point", torch.as_tensor(zero_point, dtype=torch.float32))
        self.qdtype = qdtype
        self._tables = _TableCache()

    def _merge(self, op, x, y):
        return qmerge(op, x, y, self.scale, self.zero_point, self.qdtype, self._tables)

    def add(self, x, y):
        return self._merge(_lib.MERGE_ADD, x, y)

    def mul(self, x, y):
        return self._merge(_lib.MERGE_MUL, x, y)

    def add_relu(self, x, y):
        return self._merge(_lib.MERGE_ADD_RELU, x, y)

    def add_scalar(self, x, scalar: float):
        return self._merge(_lib.MERGE_ADD, x, float(scalar))

    def mul_scalar(self, x, scalar: float):
        return self._merge(_lib.MERGE_MUL, x, float(scalar))

    def cat(self, tensors, dim: int = 0):
        """Every piece is requantized to the common grid, then the pieces are joined."""
        parts = [self._merge(_lib.MERGE_COPY, t, None) for t in tensors]
        out = torch.cat(parts, dim=dim)
        metas = [codes_of(p) for p in parts]
        if all(m is not None and m.layout == "rowmajor" for m in metas):
            return tag(out, QCodes(torch.cat([m.codes for m in metas], dim=dim), metas[0].scale,
                                   metas[0].zero_point))
        return out

    def extra_repr(self) -> str:
        return f"qdtype={self.qdtype.name}"

    @classmethod
    def from_float(cls, mod) -> "QFunctional":
        scale, zero_point, qdtype = activation_qparams(mod)
        return cls(scale, zero_point, qdtype)
