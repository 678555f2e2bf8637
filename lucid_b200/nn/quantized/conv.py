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

    def _activation(self, y):
        return F.relu(y) if self._RELU else y

    def _resolved_padding(self):
        if self.padding_str == "valid":
            return (0, 0)
        if self.padding_str == "same":
            kh, kw = self.kernel_size
            if kh % 2 == 1 and kw % 2 == 1 and self.stride == (1, 1) and self.dilation == (1, 1):
                return (kh // 2, kw // 2)
            return None  # asymmetric "same": float route
        return self.padding

    def _int8_ok(self):
        def probe():
            return bool((self.weight_zero_point == 0).all().item())
        sym = self._cache.get(self.weight_int8, "wz0:%d" % self.weight_zero_point._version, probe)
        pad = self._resolved_padding()
        ok = (sym and self.groups == 1 and self.dilation == (1, 1) and self.stride == (1, 1) and
              self.padding_mode == "zeros" and pad is not None and pad[0] == pad[1] and
              self.in_channels % 16 == 0 and self.out_qdtype.bits == 8 and self.weight_ch_axis == 0)
        if not ok and not getattr(self, "_warned", False):
            warnings.warn(f"{type(self).__name__}: geometry outside the implicit-GEMM path; "
                          "running the dequantize-to-float route", stacklevel=3)
            self._warned = True
        return ok

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x, "input")
        if backends.quantized.use_int8() and self._int8_ok():
            return self._forward_int8(x)
        return self._forward_float(x)

    def forward_codes(self, a_nhwc: torch.Tensor, a_scale, zp_is_zero: bool = True, a_zp=None):
        """NHWC codes in -> NHWC codes out on this module's output grid."""
        w = self.weight_int8
        w_krsc = self._cache.get(w, "krsc", lambda: w.permute(0, 2, 3, 1).contiguous())
        pad = self._resolved_padding()[0]
        unsigned = not self.out_qdtype.signed
        common = dict(out_dtype=torch.uint8 if unsigned else torch.int8, b_scale=self.weight_scale,
                      bias=self.bias, act=_lib.ACT_RELU if self._RELU else _lib.ACT_NONE,
                      out_scale=self.scale, out_zp=self.zero_point,
                      qmin=self.out_qdtype.quant_min, qmax=self.out_qdtype.quant_max)
        if zp_is_zero:
            return QF.conv2d_nhwc_s8(a_nhwc, w_krsc, pad=pad, a_scale=a_scale, **common)
        # non-zero input zero point: lay the codes into a frame filled with the code of 0.0,
        # then the plain zero-point correction is exact (every tap holds a real code)
        n, h, wd, c = a_nhwc.shape
        if pad:
            frame = torch.empty((n, h + 2 * pad, wd + 2 * pad, c), dtype=a_nhwc.dtype, device=a_nhwc.device)
            frame.copy_(a_zp.to(a_nhwc.dtype).reshape(1, 1, 1, 1).expand_as(frame))
            frame[:, pad:pad + h, pad:pad + wd, :] = a_nhwc
            a_nhwc = frame
        kh, kw = self.kernel_size
        p, q = a_nhwc.shape[1] - kh + 1, a_nhwc.shape[2] - kw + 1
        rowsum = self._cache.get(w, "rowsum", lambda: QF.rowsum_s8(w_krsc))
        if kh == 1 and kw == 1:
            out = QF.gemm_s8(a_nhwc.reshape(-1, c), w_krsc.reshape(self.out_channels, -1),
                             a_scale=a_scale, a_zp=a_zp, b_rowsum=rowsum, **common)
            return out.reshape(n, p, q, self.out_channels)
        # im2col-free needs zero point 0; fold the correction on the accumulator instead
        acc = QF.conv2d_nhwc_s8(a_nhwc, w_krsc, pad=0, out_dtype=torch.int32)
        acc = acc - (a_zp.to(torch.int32) * rowsum).reshape(1, 1, 1, -1)
        y = acc.to(torch.float32) * (a_scale * self.weight_scale).reshape(1, 1, 1, -1)
        if self.bias is not None:
            y = y + self.bias.reshape(1, 1, 1, -1)
        y = self._activation(y)
        from ...quantization import quantize_to
        return quantize_to(y, self.scale, self.zero_point, self.out_qdtype.quant_min,
                           self.out_qdtype.quant_max, common["out_dtype"])

    def _forward_int8(self, x):
        qc = codes_of(x)
        if qc is not None and qc.layout == "nhwc":
            a, s, z = qc.codes, qc.scale, qc.zero_point
        else:
            a, s, z = encode_activation(x.permute(0, 2, 3, 1))
        zp0 = bool((z == 0).item()) if qc is None or qc.zp_is_zero is None else qc.zp_is_zero
        codes = self.forward_codes(a, s, zp0, z)
        y = dequantize(codes, self.scale, self.zero_point).permute(0, 3, 1, 2)
        out_zp0 = self._cache.get(self.weight_int8, "ozp0:%d" % self.zero_point._version,
                                  lambda: bool((self.zero_point == 0).item()))
        return tag(y, QCodes(codes, self.scale, self.zero_point, "nhwc", out_zp0))

    def _forward_float(self, x):
        w = dequantize(self.weight_int8, self.weight_scale, self.weight_zero_point,
                       ch_axis=self.weight_ch_axis)
        pad = self._resolved_padding()
        x = x.to(torch.float32)
        if pad is None:
            y = F.conv2d(x, w, self.bias, self.stride, "same", self.dilation, self.groups)
        elif self.padding_mode != "zeros":
            mode = {"reflect": "reflect", "replicate": "replicate", "circular": "circular"}[self.padding_mode]
            xp = F.pad(x, (pad[1], pad[1], pad[0], pad[0]), mode=mode)
            y = F.conv2d(xp, w, self.bias, self.stride, 0, self.dilation, self.groups)
        else:
            y = F.conv2d(x, w, self.bias, self.stride, pad, self.dilation, self.groups)
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
