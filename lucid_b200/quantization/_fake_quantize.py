"""``FakeQuantize``: an observer plus the straight-through fake-quantize it parameterises
(lucid/quantization/_fake_quantize.py:29-225).  Every step runs on the device: the range
reduction, the qparams kernel and the fake-quantize kernel (whose saved mask is the STE
gradient gate); nothing is read back."""

from __future__ import annotations

import functools

import torch

from ._functional import fake_quantize
from .observer import MovingAverageMinMaxObserver


class FakeQuantize(torch.nn.Module):
    def __init__(self, observer=MovingAverageMinMaxObserver, **observer_kwargs) -> None:
        super().__init__()
        self.activation_post_process = observer(**observer_kwargs)
        self.qdtype = self.activation_post_process.qdtype
        self.qscheme = self.activation_post_process.qscheme
        self.ch_axis = self.activation_post_process.ch_axis
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self._observer_enabled = True
        self._fake_quant_enabled = True

    def forward(self, x):
        if self._observer_enabled:
            self.activation_post_process(x.detach())
            self.scale, self.zero_point = self.activation_post_process.calculate_qparams()
        if self._fake_quant_enabled:
            dev = x.device
            return fake_quantize(x, self.scale.to(dev), self.zero_point.to(dev), self.qdtype.quant_min,
                                 self.qdtype.quant_max, self.ch_axis)
        return x

    def enable_observer(self, enabled: bool = True) -> "FakeQuantize":
        self._observer_enabled = enabled
        return self

    def disable_observer(self) -> "FakeQuantize":
        return self.enable_observer(False)

    def enable_fake_quant(self, enabled: bool = True) -> "FakeQuantize":
        self._fake_quant_enabled = enabled
        return self

    def disable_fake_quant(self) -> "FakeQuantize":
        return self.enable_fake_quant(False)

    def calculate_qparams(self):
        return self.scale, self.zero_point

    @classmethod
    def with_args(cls, **kwargs):
        return functools.partial(cls, **kwargs)
