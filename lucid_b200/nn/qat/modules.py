"""``nn.qat.Linear`` / ``Conv2d`` (lucid/nn/qat/linear.py:140-178, conv.py): the float layer with
its weight fake-quantized per output channel and its output fake-quantized per tensor.  The
contraction itself is the float library op (training path); the fake-quantize forward and its
straight-through backward are this package's kernels."""

from __future__ import annotations

import torch
import torch.nn.functional as F


class Linear(torch.nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, qconfig=None, **kw) -> None:
        super().__init__(in_features, out_features, bias, **kw)
        if qconfig is None:
            raise ValueError("qat.Linear requires a qconfig")
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()
        self.activation_post_process = qconfig.activation()

    def forward(self, x):
        w_q = self.weight_fake_quant(self.weight)
        return self.activation_post_process(F.linear(x, w_q, self.bias))

    @classmethod
    def from_float(cls, mod) -> "Linear":
        qat = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, qconfig=mod.qconfig,
                  device=mod.weight.device, dtype=mod.weight.dtype)
        qat.weight = mod.weight
        if mod.bias is not None:
            qat.bias = mod.bias
        return qat


class Conv2d(torch.nn.Conv2d):
    def __init__(self, *args, qconfig=None, **kw) -> None:
        super().__init__(*args, **kw)
        if qconfig is None:
            raise ValueError("qat.Conv2d requires a qconfig")
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()
        self.activation_post_process = qconfig.activation()

    def forward(self, x):
        w_q = self.weight_fake_quant(self.weight)
        return self.activation_post_process(self._conv_forward(x, w_q, self.bias))

    @classmethod
    def from_float(cls, mod) -> "Conv2d":
        qat = cls(mod.in_channels, mod.out_channels, mod.kernel_size, stride=mod.stride, padding=mod.padding,
                  dilation=mod.dilation, groups=mod.groups, bias=mod.bias is not None,
                  padding_mode=mod.padding_mode, qconfig=mod.qconfig, device=mod.weight.device,
                  dtype=mod.weight.dtype)
        qat.weight = mod.weight
        if mod.bias is not None:
            qat.bias = mod.bias
        return qat
