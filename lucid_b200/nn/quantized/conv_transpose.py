"""Quantized transposed convolutions (lucid/nn/quantized/conv_transpose.py:45-260).

These run the reference's own sequence on the device -- dequantize the weight (per output
channel, axis 1 of the ``(in, out / groups, *k)`` layout), the float transposed convolution,
fake-quantize to the calibrated grid -- with this package's decode / fake-quantize kernels
around the library's float contraction; there is no integer transposed-convolution kernel.
The decoded weight is cached until the code buffer changes."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ... import _lib
from ...quantization import (PerChannelMinMaxObserver, QDtype, dequantize, fake_quantize,
                             per_channel_symmetric, qint8, quantize, quint8)
from ._utils import activation_qparams


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

    def _weight(self):
        w = self.weight_int8
        key = (w.data_ptr(), w._version, self.weight_scale._version, self.weight_zero_point._version)
        if self._decoded[0] != key:
            self._decoded = (key, dequantize(w, self.weight_scale, self.weight_zero_point,
                                             ch_axis=self.weight_ch_axis))
        return self._decoded[1]

    def forward(self, x):
        _lib.require_cuda(x, "input")
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
