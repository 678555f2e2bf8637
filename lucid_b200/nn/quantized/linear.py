"""Quantized Linear with a real integer contraction
(lucid/nn/quantized/linear.py:34-243; LinearReLU: lucid/nn/quantized/intrinsic.py:40-138).

Same constructor, buffers (``weight_int8``, ``weight_scale``, ``weight_zero_point``,
``bias``, ``scale``, ``zero_point``), ``from_float`` and ``extra_repr`` as the
reference.  ``forward`` computes

    y = fake_quantize(act(x_hat @ dequantize(W).T + b))

where the reference runs a float GEMM; here the contraction is s8 x s8 -> s32 on
the tensor cores and dequantisation, bias, activation and the output
requantisation are the GEMM's epilogue.  The float result returned is
``(codes - zero_point) * scale`` -- bit-identical to what ``fake_quantize``
returns for the same codes -- and carries the codes so the next quantized
module does not re-encode them.
"""

from __future__ import annotations

import warnings

import torch
import torch.nn.functional as F

from ... import _lib, backends
from ...quantization import QDtype, dequantize, fake_quantize, quantize_dynamic_per_tensor, quint8
from . import functional as QF
from ._utils import QCodes, activation_qparams, codes_of, quantize_weight, tag


def encode_activation(x: torch.Tensor):
    """Codes of an activation whose grid is not known: per-tensor affine quint8
    from the live range, exactly the encode dynamic.Linear performs
    (lucid/nn/quantized/dynamic/linear.py:87-92)."""
    return quantize_dynamic_per_tensor(x, quint8)


class _WeightCache:
    """Derived, non-persistent views of ``weight_int8`` (row sums; re-laid-out
    copies), rebuilt when the buffer is replaced or modified in place."""

    def __init__(self):
        self._key = None
        self._vals = {}

    def get(self, w: torch.Tensor, name: str, make):
        key = (w.data_ptr(), w._version, tuple(w.shape))
        if key != self._key:
            self._key, self._vals = key, {}
        if name not in self._vals:
            self._vals[name] = make()
        return self._vals[name]


class Linear(torch.nn.Module):
    _RELU = False

    def __init__(self, in_features: int, out_features: int, bias: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight_ch_axis = 0
        self.out_qdtype: QDtype = quint8
        self.register_buffer("weight_int8", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features))
        self.register_buffer("weight_zero_point", torch.zeros(out_features))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self._cache = _WeightCache()

    # -- hooks ---------------------------------------------------------------
    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return F.relu(y) if self._RELU else y

    def _int8_ok(self) -> bool:
        """The integer path needs symmetric weights (zero point 0), the weight
        axis on the rows and an 8-bit output grid."""
        def probe():
            return bool((self.weight_zero_point == 0).all().item())
        sym = self._cache.get(self.weight_int8, "wz0:%d" % self.weight_zero_point._version, probe)
        ok = sym and self.weight_ch_axis == 0 and self.out_qdtype.bits == 8 and \
            self.in_features % 16 == 0
        if not ok and not getattr(self, "_warned", False):
            warnings.warn(f"{type(self).__name__}: configuration outside the integer path "
                          "(affine weights, non-8-bit output or in_features % 16 != 0); "
                          "running the dequantize-to-float route", stacklevel=3)
            self._warned = True
        return ok

    # -- forward -----------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x, "input")
        _lib.check_device_status_lazily(x.device)
        if backends.quantized.use_int8() and self._int8_ok():
            return self._forward_int8(x)
        return self._forward_float(x)

    def forward_codes(self, a: torch.Tensor, a_scale, a_zp) -> torch.Tensor:
        """Codes in, codes out: ``a`` is ``(M, in_features)`` int8/uint8 on the grid
        ``(a_scale, a_zp)``; returns ``(M, out_features)`` codes on this module's
        output grid.  One kernel."""
        w = self.weight_int8
        rowsum = self._cache.get(w, "rowsum", lambda: QF.rowsum_s8(w))
        unsigned = not self.out_qdtype.signed
        return QF.gemm_s8(
            a, w, out_dtype=torch.uint8 if unsigned else torch.int8, a_scale=a_scale, a_zp=a_zp,
            b_rowsum=rowsum, b_scale=self.weight_scale, bias=self.bias,
            act=_lib.ACT_RELU if self._RELU else _lib.ACT_NONE, out_scale=self.scale,
            out_zp=self.zero_point, qmin=self.out_qdtype.quant_min, qmax=self.out_qdtype.quant_max)

    def _forward_int8(self, x):
        lead = x.shape[:-1]
        qc = codes_of(x)
        if qc is not None and qc.layout == "rowmajor":
            a, s, z = qc.codes, qc.scale, qc.zero_point
        else:
            a, s, z = encode_activation(x.to(torch.float32) if x.dtype not in
                                        (torch.float32, torch.bfloat16) else x)
        codes = self.forward_codes(a.reshape(-1, self.in_features), s, z)
        y = dequantize(codes, self.scale, self.zero_point)
        y = y.reshape(*lead, self.out_features)
        return tag(y, QCodes(codes.reshape(*lead, self.out_features), self.scale, self.zero_point))

    def _forward_float(self, x):
        """The reference's own sequence, on device (engine ``"reference"``)."""
        w = dequantize(self.weight_int8, self.weight_scale, self.weight_zero_point,
                       ch_axis=self.weight_ch_axis)
        with _lib.ieee_float32():
            y = self._activation(F.linear(x.to(torch.float32), w, self.bias))
        return fake_quantize(y, self.scale, self.zero_point, self.out_qdtype.quant_min,
                             self.out_qdtype.quant_max)

    # -- construction ------------------------------------------------------------
    @classmethod
    def from_float(cls, mod: torch.nn.Module) -> "Linear":
        """Quantize a calibrated float ``Linear`` (needs ``activation_post_process``)."""
        inner = mod[0] if isinstance(mod, torch.nn.Sequential) else mod
        qmod = cls(inner.in_features, inner.out_features, bias=inner.bias is not None)
        if not hasattr(inner, "qconfig") and hasattr(mod, "qconfig"):
            inner.qconfig = mod.qconfig
        codes, w_scale, w_zp, ch_axis = quantize_weight(inner)
        qmod.weight_int8, qmod.weight_scale, qmod.weight_zero_point = codes, w_scale, w_zp
        qmod.weight_ch_axis = ch_axis
        if inner.bias is not None:
            qmod.bias = inner.bias.detach().to(torch.float32)
        src = mod if hasattr(mod, "activation_post_process") else inner
        a_scale, a_zp, a_qdtype = activation_qparams(src)
        qmod.scale, qmod.zero_point, qmod.out_qdtype = a_scale, a_zp, a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"qdtype={self.out_qdtype.name}")


class LinearReLU(Linear):
    """Quantized Linear with the ReLU fused ahead of the output grid."""

    _RELU = True
