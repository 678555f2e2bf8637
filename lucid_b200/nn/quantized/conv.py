"""Quantized Conv2d as an NHWC implicit GEMM on integer codes
(lucid/nn/quantized/conv.py:66-229, 388-542; ConvReLU2d:
lucid/nn/quantized/intrinsic.py:241-341).

Constructor, buffers (``weight_int8 (Cout, Cin/g, kh, kw)`` ...), ``from_float``
and ``extra_repr`` follow the reference; activations enter and leave as logical
NCHW float tensors like Lucid's, physically channels-last, and carry their NHWC
codes so a stack of quantized convolutions moves one byte per element between
layers.  The reference pads the *float* activation with 0.0; a float 0.0 is the
code ``zero_point``, so out-of-image taps read code 0 only when the input zero
point is 0 (symmetric or post-ReLU grids) -- otherwise the codes are padded
explicitly with ``zero_point`` and the correction term handles it.
"""

from __future__ import annotations

import warnings

import torch
import torch.nn.functional as F

from ... import _lib, backends
from ...quantization import QDtype, dequantize, fake_quantize, quint8
from . import functional as QF
from ._utils import QCodes, activation_qparams, codes_of, quantize_weight, tag
from .linear import _WeightCache, encode_activation


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv2d(torch.nn.Module):
    _RELU = False

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0,
                 dilation=1, groups: int = 1, bias: bool = True) -> None:
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation = _pair(stride), _pair(padding), _pair(dilation)
        self.groups = groups
        self.padding_str: str | None = None
        self.padding_mode = "zeros"
        self.weight_ch_axis = 0
        self.out_qdtype: QDtype = quint8
        shape = (out_channels, in_channels // groups, *self.kernel_size)
        self.register_buffer("weight_int8", torch.zeros(shape, dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_channels))
        self.register_buffer("weight_zero_point", torch.zeros(out_channels))
        if bias:
            self.register_buffer("bias", torch.zeros(out_channels))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self._cache = _WeightCache()
        # An untagged input is encoded on the affine quint8 grid of its live range; its zero point
        # is 0 exactly when the range has no negative part.  Set to False (e.g. by a caller that
        # knows the layer follows a ReLU) to skip the one-scalar read-back of that zero point.
        self._input_may_be_negative = True

    def _activation(self, y):
        return F.relu(y) if self._RELU else y

    def _geometry(self, h: int, w: int):
        """((pad_top, pad_left), (P, Q)) for an input of h x w, following the reference's
        ``_resolve_pad`` (lucid/nn/quantized/conv.py:119-144; "same": pad_lo = total // 2, the
        larger half after the last row / column)."""
        kh, kw = self.kernel_size
        (sh, sw), (dh, dw) = self.stride, self.dilation
        if self.padding_str == "valid":
            lo, hi = (0, 0), (0, 0)
        elif self.padding_str == "same":
            def pair(size, k, st, dl):
                out = (size + st - 1) // st
                total = max(0, (out - 1) * st + (k - 1) * dl + 1 - size)
                return total // 2, total - total // 2
            (lh, hh), (lw, hw) = pair(h, kh, sh, dh), pair(w, kw, sw, dw)
            lo, hi = (lh, lw), (hh, hw)
        else:
            lo, hi = self.padding, self.padding
        p = (h + lo[0] + hi[0] - dh * (kh - 1) - 1) // sh + 1
        q = (w + lo[1] + hi[1] - dw * (kw - 1) - 1) // sw + 1
        return lo, hi, (p, q)

    def _int8_ok(self):
        def probe():
            return bool((self.weight_zero_point == 0).all().item())
        sym = self._cache.get(self.weight_int8, "wz0:%d" % self.weight_zero_point._version, probe)
        ok = (sym and self.padding_mode == "zeros" and (self.in_channels // self.groups) % 16 == 0 and
              max(self.stride) <= 8 and self.out_qdtype.bits == 8 and self.weight_ch_axis == 0)
        if not ok and not getattr(self, "_warned", False):
            warnings.warn(f"{type(self).__name__}: configuration outside the implicit-GEMM path "
                          "(affine weights, non-zero padding mode, channels per group not a multiple "
                          "of 16, stride above 8 or a non-8-bit grid); running the dequantize-to-float route",
                          stacklevel=3)
            self._warned = True
        return ok

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x, "input")
        _lib.check_device_status_lazily(x.device)
        if backends.quantized.use_int8() and self._int8_ok():
            return self._forward_int8(x)
        return self._forward_float(x)

    def forward_codes(self, a_nhwc: torch.Tensor, a_scale, zp_is_zero: bool = True, a_zp=None):
        """NHWC codes in -> NHWC codes out on this module's output grid.  One kernel per group;
        a non-zero input zero point costs one extra copy (the padded frame)."""
        w = self.weight_int8
        w_krsc = self._cache.get(w, "krsc", lambda: w.permute(0, 2, 3, 1).contiguous())
        n, h, wd, c = a_nhwc.shape
        lo, hi, out_hw = self._geometry(h, wd)
        unsigned = not self.out_qdtype.signed
        common = dict(out_dtype=torch.uint8 if unsigned else torch.int8, b_scale=self.weight_scale,
                      bias=self.bias, act=_lib.ACT_RELU if self._RELU else _lib.ACT_NONE,
                      out_scale=self.scale, out_zp=self.zero_point,
                      qmin=self.out_qdtype.quant_min, qmax=self.out_qdtype.quant_max,
                      stride=self.stride, dilation=self.dilation, groups=self.groups)
        if zp_is_zero:
            return QF.conv2d_nhwc_s8(a_nhwc, w_krsc, pad=lo, out_hw=out_hw, a_scale=a_scale, **common)
        # Non-zero input zero point: the reference pads the float activation with 0.0, whose code
        # is the zero point, so lay the codes into a frame filled with that code; then every tap
        # holds a real code and the kernel's zero-point correction term is exact.
        if any(lo) or any(hi):
            frame = torch.empty((n, h + lo[0] + hi[0], wd + lo[1] + hi[1], c), dtype=a_nhwc.dtype,
                                device=a_nhwc.device)
            frame.copy_(a_zp.to(a_nhwc.dtype).reshape(1, 1, 1, 1).expand_as(frame))
            frame[:, lo[0]:lo[0] + h, lo[1]:lo[1] + wd, :] = a_nhwc
            a_nhwc = frame
        rowsum = self._cache.get(w, "rowsum", lambda: QF.rowsum_s8(w_krsc))
        return QF.conv2d_nhwc_s8(a_nhwc, w_krsc, pad=0, out_hw=out_hw, a_scale=a_scale, a_zp=a_zp,
                                 b_rowsum=rowsum, **common)

    def _forward_int8(self, x):
        qc = codes_of(x)
        if qc is not None and qc.layout == "nhwc":
            a, s, z = qc.codes, qc.scale, qc.zero_point
        elif qc is not None and qc.codes.dim() == 4 and qc.codes.dtype in (torch.int8, torch.uint8):
            a, s, z = qc.codes.permute(0, 2, 3, 1).contiguous(), qc.scale, qc.zero_point  # NCHW codes: re-lay, exact
        else:
            a, s, z = encode_activation(x.permute(0, 2, 3, 1))
        if qc is not None and qc.zp_is_zero is not None:
            zp0 = qc.zp_is_zero
        elif qc is None and not self._input_may_be_negative:
            zp0 = True
        else:
            zp0 = bool((z == 0).item())
        codes = self.forward_codes(a, s, zp0, z)
        y = dequantize(codes, self.scale, self.zero_point).permute(0, 3, 1, 2)
        out_zp0 = self._cache.get(self.weight_int8, "ozp0:%d" % self.zero_point._version,
                                  lambda: bool((self.zero_point == 0).item()))
        return tag(y, QCodes(codes, self.scale, self.zero_point, "nhwc", out_zp0))

    def _forward_float(self, x):
        w = dequantize(self.weight_int8, self.weight_scale, self.weight_zero_point,
                       ch_axis=self.weight_ch_axis)
        lo, hi, _ = self._geometry(x.shape[2], x.shape[3])
        x = x.to(torch.float32)
        mode = "constant" if self.padding_mode == "zeros" else self.padding_mode
        with _lib.ieee_float32():
            if mode != "constant" or lo != hi:
                xp = F.pad(x, (lo[1], hi[1], lo[0], hi[0]), mode=mode)
                y = F.conv2d(xp, w, self.bias, self.stride, 0, self.dilation, self.groups)
            else:
                y = F.conv2d(x, w, self.bias, self.stride, lo, self.dilation, self.groups)
        y = self._activation(y).contiguous()
        return fake_quantize(y, self.scale, self.zero_point, self.out_qdtype.quant_min,
                             self.out_qdtype.quant_max)

    @classmethod
    def from_float(cls, mod: torch.nn.Module) -> "Conv2d":
        inner = mod[0] if isinstance(mod, torch.nn.Sequential) else mod
        padding = inner.padding if not isinstance(inner.padding, str) else 0
        qmod = cls(inner.in_channels, inner.out_channels, inner.kernel_size, inner.stride, padding,
                   inner.dilation, inner.groups, bias=inner.bias is not None)
        if not hasattr(inner, "qconfig") and hasattr(mod, "qconfig"):
            inner.qconfig = mod.qconfig
        codes, w_scale, w_zp, ch_axis = quantize_weight(inner)
        qmod.weight_int8, qmod.weight_scale, qmod.weight_zero_point = codes, w_scale, w_zp
        qmod.weight_ch_axis = ch_axis
        qmod.padding_str = inner.padding if isinstance(inner.padding, str) else \
            getattr(inner, "_padding_str", None)
        qmod.padding_mode = getattr(inner, "padding_mode", "zeros")
        if inner.bias is not None:
            qmod.bias = inner.bias.detach().to(torch.float32)
        src = mod if hasattr(mod, "activation_post_process") else inner
        a_scale, a_zp, a_qdtype = activation_qparams(src)
        qmod.scale, qmod.zero_point, qmod.out_qdtype = a_scale, a_zp, a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride}, qdtype={self.out_qdtype.name}")


class ConvReLU2d(Conv2d):
    """Quantized Conv2d with the ReLU fused ahead of the output grid."""

    _RELU = True


class Conv1d(Conv2d):
    """Quantized Conv1d (lucid/nn/quantized/conv.py:232-385) on the same implicit GEMM: an
    ``(N, C, L)`` signal is an ``(N, C, 1, L)`` image and the ``(Cout, Cin/g, k)`` kernel a
    ``1 x k`` one.  Buffers keep the reference's shapes in ``state_dict`` (the weight is stored
    3-D); inside the module it carries the unit height."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0,
                 dilation=1, groups: int = 1, bias: bool = True) -> None:
        def one(v):
            return int(v[0]) if isinstance(v, (tuple, list)) else int(v)
        super().__init__(in_channels, out_channels, (1, one(kernel_size)), (1, one(stride)), (0, one(padding)),
                         (1, one(dilation)), groups, bias)
        self._register_state_dict_hook(self._squeeze_weight)
        self._register_load_state_dict_pre_hook(self._unsqueeze_weight)

    @staticmethod
    def _squeeze_weight(module, state, prefix, _meta):
        key = prefix + "weight_int8"
        if key in state and state[key].dim() == 4:
            state[key] = state[key].squeeze(2)
        return state

    def _unsqueeze_weight(self, state, prefix, *_):
        key = prefix + "weight_int8"
        if key in state and state[key].dim() == 3:
            state[key] = state[key].unsqueeze(2)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 3:
            raise _lib.ShapeMismatch(f"{type(self).__name__} expects (N, C, L), got {tuple(x.shape)}")
        # codes ride along as (N, L, C) ("nlc") between 1-D layers, or arrive (N, C, L) from a stub
        qc = codes_of(x)
        x4 = x.unsqueeze(2)
        if qc is not None and qc.codes.dim() == 3 and qc.codes.dtype in (torch.int8, torch.uint8):
            nlc = qc.codes if qc.layout == "nlc" else qc.codes.permute(0, 2, 1).contiguous()
            x4 = tag(x4, QCodes(nlc.unsqueeze(1), qc.scale, qc.zero_point, "nhwc", qc.zp_is_zero))
        y4 = super().forward(x4)
        y = y4.squeeze(2)
        q4 = codes_of(y4)
        if q4 is not None and q4.layout == "nhwc":
            y = tag(y, QCodes(q4.codes.squeeze(1), q4.scale, q4.zero_point, "nlc", q4.zp_is_zero))
        return y

    @classmethod
    def from_float(cls, mod: torch.nn.Module) -> "Conv1d":
        inner = mod[0] if isinstance(mod, torch.nn.Sequential) else mod
        padding = inner.padding if not isinstance(inner.padding, str) else 0
        qmod = cls(inner.in_channels, inner.out_channels, inner.kernel_size, inner.stride, padding,
                   inner.dilation, inner.groups, bias=inner.bias is not None)
        if not hasattr(inner, "qconfig") and hasattr(mod, "qconfig"):
            inner.qconfig = mod.qconfig
        codes, w_scale, w_zp, ch_axis = quantize_weight(inner)
        qmod.weight_int8, qmod.weight_scale, qmod.weight_zero_point = codes.unsqueeze(2), w_scale, w_zp
        qmod.weight_ch_axis = ch_axis
        qmod.padding_str = inner.padding if isinstance(inner.padding, str) else \
            getattr(inner, "_padding_str", None)
        qmod.padding_mode = getattr(inner, "padding_mode", "zeros")
        if inner.bias is not None:
            qmod.bias = inner.bias.detach().to(torch.float32)
        src = mod if hasattr(mod, "activation_post_process") else inner
        a_scale, a_zp, a_qdtype = activation_qparams(src)
        qmod.scale, qmod.zero_point, qmod.out_qdtype = a_scale, a_zp, a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size[1:]}, "
                f"stride={self.stride[1:]}, qdtype={self.out_qdtype.name}")


class ConvReLU1d(Conv1d):
    """Quantized Conv1d with the ReLU fused ahead of the output grid
    (lucid/nn/quantized/intrinsic.py)."""

    _RELU = True


class Conv3d(torch.nn.Module):
    """Quantized Conv3d (lucid/nn/quantized/conv.py:545-700): the reference's sequence --
    dequantize the weight, float convolution, activation, fake-quantize onto the output grid --
    around the library's float kernel with TF32 off.  (The implicit-GEMM kernel walks two spatial
    axes; volumes take this route.)"""

    _RELU = False

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0,
                 dilation=1, groups: int = 1, bias: bool = True) -> None:
        super().__init__()

        def triple(v):
            return (v, v, v) if isinstance(v, int) else tuple(v)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = triple(kernel_size)
        self.stride, self.padding, self.dilation = triple(stride), triple(padding), triple(dilation)
        self.groups = groups
        self.padding_str: str | None = None
        self.padding_mode = "zeros"
        self.weight_ch_axis = 0
        self.out_qdtype: QDtype = quint8
        self.register_buffer("weight_int8", torch.zeros((out_channels, in_channels // groups, *self.kernel_size),
                                                        dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_channels))
        self.register_buffer("weight_zero_point", torch.zeros(out_channels))
        if bias:
            self.register_buffer("bias", torch.zeros(out_channels))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x, "input")
        w = dequantize(self.weight_int8, self.weight_scale, self.weight_zero_point, ch_axis=self.weight_ch_axis)
        x = x.to(torch.float32)
        pad = self.padding_str if self.padding_str is not None else self.padding
        with _lib.ieee_float32():
            if self.padding_mode != "zeros" and not isinstance(pad, str):
                rev = [p for d in reversed(pad) for p in (d, d)]
                y = F.conv3d(F.pad(x, rev, mode=self.padding_mode), w, self.bias, self.stride, 0, self.dilation,
                             self.groups)
            else:
                y = F.conv3d(x, w, self.bias, self.stride, pad, self.dilation, self.groups)
        y = (F.relu(y) if self._RELU else y).contiguous()
        return fake_quantize(y, self.scale, self.zero_point, self.out_qdtype.quant_min, self.out_qdtype.quant_max)

    @classmethod
    def from_float(cls, mod: torch.nn.Module) -> "Conv3d":
        inner = mod[0] if isinstance(mod, torch.nn.Sequential) else mod
        padding = inner.padding if not isinstance(inner.padding, str) else 0
        qmod = cls(inner.in_channels, inner.out_channels, inner.kernel_size, inner.stride, padding,
                   inner.dilation, inner.groups, bias=inner.bias is not None)
        if not hasattr(inner, "qconfig") and hasattr(mod, "qconfig"):
            inner.qconfig = mod.qconfig
        codes, w_scale, w_zp, ch_axis = quantize_weight(inner)
        qmod.weight_int8, qmod.weight_scale, qmod.weight_zero_point = codes, w_scale, w_zp
        qmod.weight_ch_axis = ch_axis
        qmod.padding_str = inner.padding if isinstance(inner.padding, str) else None
        qmod.padding_mode = getattr(inner, "padding_mode", "zeros")
        if inner.bias is not None:
            qmod.bias = inner.bias.detach().to(torch.float32)
        src = mod if hasattr(mod, "activation_post_process") else inner
        a_scale, a_zp, a_qdtype = activation_qparams(src)
        qmod.scale, qmod.zero_point, qmod.out_qdtype = a_scale, a_zp, a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride}, qdtype={self.out_qdtype.name}")


class ConvReLU3d(Conv3d):
    _RELU = True
