"""Quantized transposed convolutions (lucid/nn/quantized/conv_transpose.py:45-260).

``ConvTranspose2d`` with symmetric weights and channels per group a multiple of 16 runs on the
integer convolution kernel: a transposed convolution is the forward convolution of the input
zero-inserted by the stride with the flipped kernel, so the input codes are laid at stride distance
into a frame filled with the code of 0.0 and the strided-convolution kernel does the rest
(contraction, zero-point correction, bias, requantisation in one launch).  Everything else
(1-D / 3-D, affine weights, padding beyond the kernel's reach) runs the reference's own sequence
on the device -- dequantize the weight (per output channel, axis 1 of the ``(in, out / groups,
*k)`` layout), the library's float transposed convolution, fake-quantize to the calibrated grid;
the decoded weight is cached until the code buffer changes."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ... import _lib, backends
from ...quantization import (PerChannelMinMaxObserver, QDtype, dequantize, fake_quantize,
                             per_channel_symmetric, qint8, quantize, quint8)
from . import functional as QF
from ._utils import QCodes, activation_qparams, codes_of, tag
from .linear import encode_activation


class _QuantizedConvTransposeNd(torch.nn.Module):
    _ND = 2
    _FN = staticmethod(F.conv_transpose2d)

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0,
                 output_padding=0, dilation=1, groups: int = 1, bias: bool = True) -> None:
        super().__init__()
        nd = self._ND

        def tup(v):
            return tuple(v) if isinstance(v, (tuple, list)) else (v,) * nd

        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = tup(kernel_size), tup(stride), tup(padding)
        self.output_padding, self.dilation, self.groups = tup(output_padding), tup(dilation), groups
        self.out_qdtype: QDtype = quint8
        self.weight_ch_axis = 1
        n_out = out_channels // groups
        self.register_buffer("weight_int8", torch.zeros((in_channels, n_out) + self.kernel_size, dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(n_out))
        self.register_buffer("weight_zero_point", torch.zeros(n_out))
        if bias:
            self.register_buffer("bias", torch.zeros(out_channels))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self._decoded = (None, None)
        self._krsc = (None, None, None, None)
        self._sym = (None, False)

    def _weight(self):
        w = self.weight_int8
        key = (w.data_ptr(), w._version, self.weight_scale._version, self.weight_zero_point._version)
        if self._decoded[0] != key:
            self._decoded = (key, dequantize(w, self.weight_scale, self.weight_zero_point,
                                             ch_axis=self.weight_ch_axis))
        return self._decoded[1]

    def _int8_ok(self) -> bool:
        """Integer route: 2-D, symmetric weights, channels per group a multiple of 16, an 8-bit
        output grid and padding no larger than the kernel's reach (so the up-sampled frame only
        has to be padded, never cropped)."""
        if self._ND != 2 or not backends.quantized.use_int8():
            return False
        key = ("wz0", self.weight_zero_point.data_ptr(), self.weight_zero_point._version)
        if self._sym[0] != key:
            self._sym = (key, bool((self.weight_zero_point == 0).all().item()))
        reach = [d * (k - 1) - p for d, k, p in zip(self.dilation, self.kernel_size, self.padding)]
        return (self._sym[1] and (self.in_channels // self.groups) % 16 == 0 and min(reach) >= 0 and
                self.out_qdtype.bits == 8)

    def _weight_krsc(self):
        """The equivalent forward-convolution filters as (Cout, kh, kw, Cin / groups) codes: the
        kernel flipped in both spatial directions with its channel axes swapped per group, plus
        their row sums and the per-filter scale."""
        w = self.weight_int8
        key = (w.data_ptr(), w._version, self.weight_scale._version)
        if self._krsc[0] != key:
            g, cin_g, cout_g = self.groups, self.in_channels // self.groups, self.out_channels // self.groups
            kh, kw = self.kernel_size
            wk = w.reshape(g, cin_g, cout_g, kh, kw).flip(3, 4).permute(0, 2, 3, 4, 1)
            wk = wk.reshape(self.out_channels, kh, kw, cin_g).contiguous()
            self._krsc = (key, wk, QF.rowsum_s8(wk), self.weight_scale.repeat(g).contiguous())
        return self._krsc[1:]

    def _forward_int8(self, x):
        """conv_transpose(x, W) = conv(x zero-inserted by the stride and padded by
        dilation * (k - 1) - padding, W flipped): the integer kernel of the quantized Conv2d runs on
        a frame of codes filled with the input's zero point (the code of the value 0.0), into which
        the input codes are laid at stride distance; every tap then holds a real code and the
        kernel's zero-point correction is exact."""
        qc = codes_of(x)
        if qc is not None and qc.layout == "nhwc":
            a, s, z = qc.codes, qc.scale, qc.zero_point
        else:
            a, s, z = encode_activation(x.permute(0, 2, 3, 1))
        n, h, w_in, c = a.shape
        (sh, sw), (dh, dw), (kh, kw) = self.stride, self.dilation, self.kernel_size
        rh, rw = dh * (kh - 1) - self.padding[0], dw * (kw - 1) - self.padding[1]
        fh = (h - 1) * sh + 1 + 2 * rh + self.output_padding[0]
        fw = (w_in - 1) * sw + 1 + 2 * rw + self.output_padding[1]
        frame = torch.empty((n, fh, fw, c), dtype=a.dtype, device=a.device)
        frame.copy_(z.to(a.dtype).reshape(1, 1, 1, 1).expand_as(frame))
        frame[:, rh:rh + (h - 1) * sh + 1:sh, rw:rw + (w_in - 1) * sw + 1:sw, :] = a
        wk, rowsum, wscale = self._weight_krsc()
        unsigned = not self.out_qdtype.signed
        codes = QF.conv2d_nhwc_s8(frame, wk, pad=0, dilation=self.dilation, groups=self.groups,
                                  out_hw=(fh - dh * (kh - 1), fw - dw * (kw - 1)),
                                  out_dtype=torch.uint8 if unsigned else torch.int8, a_scale=s, a_zp=z,
                                  b_rowsum=rowsum, b_scale=wscale, bias=self.bias, out_scale=self.scale,
                                  out_zp=self.zero_point, qmin=self.out_qdtype.quant_min,
                                  qmax=self.out_qdtype.quant_max)
        y = dequantize(codes, self.scale, self.zero_point).permute(0, 3, 1, 2)
        return tag(y, QCodes(codes, self.scale, self.zero_point, "nhwc"))

    def forward(self, x):
        _lib.require_cuda(x, "input")
        if self._int8_ok():
            return self._forward_int8(x)
        with _lib.ieee_float32():
            y = self._FN(x.to(torch.float32), self._weight(), self.bias, self.stride, self.padding,
                         self.output_padding, self.groups, self.dilation)
        return fake_quantize(y.contiguous(), self.scale, self.zero_point, self.out_qdtype.quant_min,
                             self.out_qdtype.quant_max)

    @classmethod
    def from_float(cls, mod):
        if isinstance(mod.padding, str):
            raise NotImplementedError("quantized conv_transpose: string padding is not supported yet")
        q = cls(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride, mod.padding,
                mod.output_padding, mod.dilation, mod.groups, bias=mod.bias is not None)
        wobs = PerChannelMinMaxObserver(ch_axis=1, qscheme=per_channel_symmetric, qdtype=qint8)
        w = mod.weight.detach()
        wobs(w)
        w_scale, w_zp = wobs.calculate_qparams()
        q.weight_int8 = quantize(w, w_scale, w_zp, qint8, ch_axis=1)
        q.weight_scale, q.weight_zero_point = w_scale, w_zp
        if mod.bias is not None:
            q.bias = mod.bias.detach().to(torch.float32)
        q.scale, q.zero_point, q.out_qdtype = activation_qparams(mod)
        return q

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride}, qdtype={self.out_qdtype.name}")


class ConvTranspose1d(_QuantizedConvTransposeNd):
    _ND = 1
    _FN = staticmethod(F.conv_transpose1d)


class ConvTranspose2d(_QuantizedConvTransposeNd):
    _ND = 2
    _FN = staticmethod(F.conv_transpose2d)


class ConvTranspose3d(_QuantizedConvTransposeNd):
    _ND = 3
    _FN = staticmethod(F.conv_transpose3d)
