"""Quantized activations (lucid/nn/quantized/activation.py:22-486): the float activation followed
by a fake-quantize to the calibrated output grid.

When the input carries 8-bit codes the whole module is a function of one byte: the 256 values
``encode(act(decode(c)))`` are evaluated once per input grid and the tensor streams through that
table (``lq_lut_u8``: one byte read, one byte written per element).  Float inputs run the float
activation and the fake-quantize kernel."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ... import _lib
from ...quantization import QDtype, dequantize, fake_quantize, quantize_to, quint8
from ._utils import QCodes, activation_qparams, codes_of, tag


class _QuantizedActivation(torch.nn.Module):
    def __init__(self, scale, zero_point, qdtype: QDtype = quint8) -> None:
        super().__init__()
        self.register_buffer("scale", torch.as_tensor(scale, dtype=torch.float32))
        self.register_buffer("zero_point", torch.as_tensor(zero_point, dtype=torch.float32))
        self.qdtype = qdtype
        self._tables: dict = {}

    def _act(self, x):
        raise NotImplementedError

    def _configure(self, mod) -> None:
        """Copy activation-specific parameters from the float module."""

    def _table(self, qc: QCodes) -> torch.Tensor:
        """256-byte map from an input code (as a raw byte) to the output code (as a raw byte)."""
        key = (qc.codes.dtype, qc.scale.data_ptr(), qc.scale._version, qc.zero_point.data_ptr(),
               qc.zero_point._version, self.scale._version, self.zero_point._version)
        tab = self._tables.get(key)
        if tab is None:
            dev = qc.codes.device
            raw = torch.arange(256, device=dev, dtype=torch.int32).to(torch.uint8)
            codes_in = raw.view(torch.int8) if qc.codes.dtype == torch.int8 else raw
            x = dequantize(codes_in.contiguous(), qc.scale, qc.zero_point)
            store = torch.int8 if self.qdtype.signed else torch.uint8
            tab = quantize_to(self._act(x).contiguous(), self.scale, self.zero_point,
                              self.qdtype.quant_min, self.qdtype.quant_max, store).view(torch.uint8)
            self._tables = {key: tab}
        return tab

    def forward(self, x):
        _lib.require_cuda(x, "input")
        qc = codes_of(x)
        if (qc is not None and qc.codes.dtype in (torch.int8, torch.uint8) and qc.scale.dim() == 0
                and self.qdtype.bits <= 8):
            src = qc.codes.contiguous()
            out = torch.empty_like(src, dtype=torch.int8 if self.qdtype.signed else torch.uint8)
            with torch.cuda.device(src.device):
                _lib.check(_lib.load().lq_lut_u8(_lib.ptr(src), src.numel(), _lib.ptr(self._table(qc)),
                                                 _lib.ptr(out), _lib.stream_ptr(src.device)))
            y = dequantize(out, self.scale, self.zero_point)
            if qc.layout == "nhwc":
                y = y.permute(0, 3, 1, 2)
            elif qc.layout == "nlc":
                y = y.permute(0, 2, 1)
            return tag(y, QCodes(out, self.scale, self.zero_point, qc.layout))
        return fake_quantize(self._act(x.to(torch.float32)).contiguous(), self.scale, self.zero_point,
                             self.qdtype.quant_min, self.qdtype.quant_max)

    def extra_repr(self) -> str:
        return f"qdtype={self.qdtype.name}"

    @classmethod
    def from_float(cls, mod):
        scale, zero_point, qdtype = activation_qparams(mod)
        obj = cls(scale, zero_point, qdtype)
        obj._configure(mod)
        return obj


class Sigmoid(_QuantizedActivation):
    def _act(self, x):
        return torch.sigmoid(x)


class Hardswish(_QuantizedActivation):
    def _act(self, x):
        return F.hardswish(x)


class Hardsigmoid(_QuantizedActivation):
    def _act(self, x):
        return F.hardsigmoid(x)


class Tanh(_QuantizedActivation):
    def _act(self, x):
        return torch.tanh(x)


class ELU(_QuantizedActivation):
    alpha: float = 1.0

    def _configure(self, mod) -> None:
        self.alpha = float(getattr(mod, "alpha", 1.0))

    def _act(self, x):
        return F.elu(x, self.alpha)


class LeakyReLU(_QuantizedActivation):
    negative_slope: float = 0.01

    def _configure(self, mod) -> None:
        self.negative_slope = float(getattr(mod, "negative_slope", 0.01))

    def _act(self, x):
        return F.leaky_relu(x, self.negative_slope)


class ReLU(torch.nn.ReLU):
    """``nn.ReLU`` that keeps the codes of its input alive.  On floats it is the plain ReLU (the
    reference's converted model keeps ``nn.ReLU`` as it is); when the input carries integer codes,
    the rectified tensor carries ``max(code, zero_point)`` on the same grid -- exactly the codes
    of the rectified values -- so that a quantized layer behind an unfused (possibly in-place)
    ReLU consumes codes instead of re-encoding floats.  ``convert`` swaps every ``nn.ReLU`` of
    the model for this class; it has no state and no observer."""

    def forward(self, x):
        qc = codes_of(x) if isinstance(x, torch.Tensor) and x.is_cuda else None
        y = F.relu(x, inplace=self.inplace)
        if qc is None or qc.scale.dim() != 0:
            return y
        floor = qc.zero_point.to(qc.codes.dtype)
        codes = torch.maximum(qc.codes, floor)
        return tag(y, QCodes(codes, qc.scale, qc.zero_point, qc.layout, qc.zp_is_zero))

    @classmethod
    def from_float(cls, mod):
        return cls(inplace=mod.inplace)
