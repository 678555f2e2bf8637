"""Boundary stubs (lucid/nn/quantized/modules.py:186-350): float -> grid at the
model's entry, grid -> float at its exit."""

from __future__ import annotations

import torch

from ...quantization import QDtype, dequantize, quantize_to, quint8
from ...quantization._quantize import DeQuantStub, QuantStub, QuantWrapper  # noqa: F401  (the reference exports them here)
from ._utils import QCodes, activation_qparams, codes_of, tag


class Quantize(torch.nn.Module):
    """Snap a float activation onto a fixed grid; the result is the
    fake-quantized float tensor (as in the reference) carrying its codes."""

    def __init__(self, scale=1.0, zero_point=0.0, qdtype: QDtype = quint8, nhwc: bool | None = None):
        super().__init__()
        self.register_buffer("scale", torch.as_tensor(scale, dtype=torch.float32))
        self.register_buffer("zero_point", torch.as_tensor(zero_point, dtype=torch.float32))
        self.qdtype = qdtype
        self.nhwc = nhwc
        self._zp0 = None  # (key of the zero-point buffer, "it is zero"): read back once, not per call

    def _zp_is_zero(self) -> bool:
        z = self.zero_point
        key = (z.data_ptr(), z._version)
        if self._zp0 is None or self._zp0[0] != key:
            self._zp0 = (key, bool((z == 0).all().item()))
        return self._zp0[1]

    def forward(self, x):
        # image batches (4-D) carry their codes channels-last, the layout the convolution reads
        nhwc = self.nhwc if self.nhwc is not None else x.dim() == 4
        src = x.permute(0, 2, 3, 1) if nhwc else x
        store = torch.int8 if self.qdtype.signed else torch.uint8
        codes = quantize_to(src, self.scale, self.zero_point, self.qdtype.quant_min,
                            self.qdtype.quant_max, store)
        y = dequantize(codes, self.scale, self.zero_point)
        if nhwc:
            y = y.permute(0, 3, 1, 2)
        return tag(y, QCodes(codes, self.scale, self.zero_point, "nhwc" if nhwc else "rowmajor", self._zp_is_zero()))

    @classmethod
    def from_float(cls, mod):
        s, z, qd = activation_qparams(mod)
        return cls(s, z, qd)


class DeQuantize(torch.nn.Module):
    """Identity on the float carrier (drops the codes)."""

    def forward(self, x):
        return x.view_as(x) if codes_of(x) is not None else x

    @classmethod
    def from_float(cls, mod):
        return cls()
