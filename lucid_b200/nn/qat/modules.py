"""``nn.qat`` layers (lucid/nn/qat/linear.py:23-260, conv.py:46-800): the float layer with its
weight fake-quantized per output channel and its output fake-quantized per tensor; the fused
``*ReLU`` forms apply the ReLU before the output fake-quantize, so the grid the layer trains
against covers the post-ReLU range only.  The contraction itself is the float library op
(training path); the fake-quantize forward and its straight-through backward are this package's
kernels.  ``convert`` turns each into the inference layer of the same name under
``nn.quantized``."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _inner_of(mod):
    """A fused float container (``nni.LinearReLU`` / ``nni.ConvReLU*d``) hands over its first
    member with the container's qconfig (lucid/nn/qat/conv.py:469-473)."""
    if isinstance(mod, torch.nn.Sequential):
        inner = mod[0]
        inner.qconfig = mod.qconfig
        return inner
    return mod


class Linear(torch.nn.Linear):
    _RELU = False

    def __init__(self, in_features: int, out_features: int, bias: bool = True, qconfig=None, **kw) -> None:
        super().__init__(in_features, out_features, bias, **kw)
        if qconfig is None:
            raise ValueError(f"qat.{type(self).__name__} requires a qconfig")
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()
        self.activation_post_process = qconfig.activation()

    def forward(self, x):
        w_q = self.weight_fake_quant(self.weight)
        y = F.linear(x, w_q, self.bias)
        return self.activation_post_process(F.relu(y) if self._RELU else y)

    @classmethod
    def from_float(cls, mod) -> "Linear":
        mod = _inner_of(mod)
        qat = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, qconfig=mod.qconfig,
                  device=mod.weight.device, dtype=mod.weight.dtype)
        qat.weight = mod.weight
        if mod.bias is not None:
            qat.bias = mod.bias
        return qat


class LinearReLU(Linear):
    _RELU = True


class _ConvMixin:
    """Shared by the three ranks: construction with a qconfig, the fake-quantized forward and
    ``from_float``.  The concrete classes put it in front of ``torch.nn.Conv{1,2,3}d``."""

    _RELU = False

    def __init__(self, *args, qconfig=None, **kw) -> None:
        super().__init__(*args, **kw)
        if qconfig is None:
            raise ValueError(f"qat.{type(self).__name__} requires a qconfig")
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()
        self.activation_post_process = qconfig.activation()

    def forward(self, x):
        w_q = self.weight_fake_quant(self.weight)
        y = self._conv_forward(x, w_q, self.bias)
        return self.activation_post_process(F.relu(y) if self._RELU else y)

    @classmethod
    def from_float(cls, mod):
        mod = _inner_of(mod)
        qat = cls(mod.in_channels, mod.out_channels, mod.kernel_size, stride=mod.stride, padding=mod.padding,
                  dilation=mod.dilation, groups=mod.groups, bias=mod.bias is not None,
                  padding_mode=mod.padding_mode, qconfig=mod.qconfig, device=mod.weight.device,
                  dtype=mod.weight.dtype)
        qat.weight = mod.weight
        if mod.bias is not None:
            qat.bias = mod.bias
        return qat


class Conv1d(_ConvMixin, torch.nn.Conv1d):
    pass


class Conv2d(_ConvMixin, torch.nn.Conv2d):
    pass


class Conv3d(_ConvMixin, torch.nn.Conv3d):
    pass


class ConvReLU1d(Conv1d):
    _RELU = True


class ConvReLU2d(Conv2d):
    _RELU = True


class ConvReLU3d(Conv3d):
    _RELU = True


class Embedding(torch.nn.Embedding):
    """Lookup in the fake-quantized table (lucid/nn/qat/sparse.py:21-132): one
    ``weight_fake_quant`` and no output fake-quantizer, as the rows are read back unchanged."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx=None, *, qconfig=None, **kw) -> None:
        super().__init__(num_embeddings, embedding_dim, padding_idx, **kw)
        if qconfig is None:
            raise ValueError("qat.Embedding requires a qconfig")
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()

    def forward(self, x):
        return F.embedding(x, self.weight_fake_quant(self.weight), self.padding_idx)

    @classmethod
    def from_float(cls, mod) -> "Embedding":
        qat = cls(mod.num_embeddings, mod.embedding_dim, mod.padding_idx, qconfig=mod.qconfig,
                  device=mod.weight.device, dtype=mod.weight.dtype)
        qat.weight = mod.weight
        return qat
