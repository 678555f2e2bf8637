"""Dynamically quantized Linear layers.

``Linear`` mirrors lucid/nn/quantized/dynamic/linear.py:36-124: int8 per-row
symmetric weight, per-forward per-tensor affine quint8 activation grid, float
output, no output requantisation.  The reference fake-quantizes the input and
runs a float GEMM; here the activation is encoded once (range reduction ->
qparams -> u8 codes, all on device, no host sync) and the contraction is the
integer GEMM whose epilogue applies ``s_x * s_w[n]``, the zero-point correction
and the bias.

``PerTokenLinear`` and ``GatedMLP`` are the per-token W8A8 compositions the
transformer configs use; the reference has no single module for them, they are
built from the same primitives (per-row observer -> symmetric qparams ->
quantize(ch_axis=0) -> linear).
"""

from __future__ import annotations

import warnings

import torch
import torch.nn.functional as F

from .... import _lib, backends
from ....quantization import (PerChannelMinMaxObserver, QDtype, calculate_qparams, dequantize, fake_quantize,
                              minmax, per_channel_symmetric, per_tensor_affine, qint8, quantize,
                              quantize_dynamic_per_tensor, quantize_per_token, quint8)
from .. import functional as QF
from ..linear import _WeightCache


def _encode_weight(weight: torch.Tensor, dtype: QDtype):
    obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=dtype)
    obs(weight)
    scale, zero_point = obs.calculate_qparams()
    return quantize(weight, scale, zero_point, dtype, ch_axis=0), scale, zero_point


class Linear(torch.nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight_ch_axis = 0
        self.act_qdtype: QDtype = quint8
        self.register_buffer("weight_int8", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features))
        self.register_buffer("weight_zero_point", torch.zeros(out_features))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None
        self._cache = _WeightCache()

    def _int8_ok(self) -> bool:
        """The integer path needs symmetric weights (zero point 0) on the row axis and
        ``in_features % 16 == 0``; anything else takes the reference's float sequence."""
        def probe():
            return bool((self.weight_zero_point == 0).all().item())
        sym = self._cache.get(self.weight_int8, "wz0:%d" % self.weight_zero_point._version, probe)
        ok = sym and self.weight_ch_axis == 0 and self.in_features % 16 == 0
        if not ok and not getattr(self, "_warned", False):
            warnings.warn("dynamic.Linear: configuration outside the integer path (affine weights or "
                          "in_features % 16 != 0); running the dequantize-to-float route", stacklevel=3)
            self._warned = True
        return ok

    def _forward_float(self, x: torch.Tensor) -> torch.Tensor:
        """The reference's own sequence (lucid/nn/quantized/dynamic/linear.py:84-99) on device:
        fake-quantize the input on its live affine grid, dequantize the weight, float GEMM."""
        x32 = x.to(torch.float32)
        mn, mx = minmax(x32.reshape(-1))
        s, z = calculate_qparams(mn, mx, per_tensor_affine, self.act_qdtype)
        xq = fake_quantize(x32.contiguous(), s, z, self.act_qdtype.quant_min, self.act_qdtype.quant_max)
        w = dequantize(self.weight_int8, self.weight_scale, self.weight_zero_point, ch_axis=self.weight_ch_axis)
        with _lib.ieee_float32():
            return F.linear(xq, w, self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x, "input")
        _lib.check_device_status_lazily(x.device)
        if not (backends.quantized.use_int8() and self._int8_ok()):
            return self._forward_float(x)
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        a, x_scale, x_zp = quantize_dynamic_per_tensor(x2, self.act_qdtype)
        w = self.weight_int8
        rowsum = self._cache.get(w, "rowsum", lambda: QF.rowsum_s8(w))
        out_dtype = x.dtype if x.dtype in (torch.float32, torch.bfloat16) else torch.float32
        y = QF.gemm_s8(a, w, out_dtype=out_dtype, a_scale=x_scale, a_zp=x_zp, b_rowsum=rowsum,
                       b_scale=self.weight_scale, bias=self.bias)
        return y.reshape(*lead, self.out_features)

    @classmethod
    def from_float(cls, mod: torch.nn.Module, dtype: QDtype = qint8) -> "Linear":
        qmod = cls(mod.in_features, mod.out_features, bias=mod.bias is not None)
        codes, scale, zp = _encode_weight(mod.weight.detach(), dtype)
        qmod.weight_int8, qmod.weight_scale, qmod.weight_zero_point = codes, scale, zp
        if mod.bias is not None:
            qmod.bias = mod.bias.detach().to(torch.float32)
        return qmod

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, dynamic=True"


class PerTokenLinear(torch.nn.Module):
    """W8A8 linear with per-token symmetric int8 activations; bf16/f32 in and out.

    Two kernels per call: fused per-token encode (one HBM pass) and the GEMM
    whose epilogue applies ``s_token[m] * s_w[n]`` (+ bias)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight_int8", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features))
        self.register_buffer("weight_zero_point", torch.zeros(out_features))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None

    def forward_codes(self, a: torch.Tensor, a_scale: torch.Tensor, out_dtype=torch.bfloat16):
        return QF.gemm_s8(a, self.weight_int8, out_dtype=out_dtype, a_scale=a_scale,
                          b_scale=self.weight_scale, bias=self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        a, s = quantize_per_token(x.reshape(-1, self.in_features), qint8)
        return self.forward_codes(a, s, x.dtype).reshape(*lead, self.out_features)

    @classmethod
    def from_float(cls, mod: torch.nn.Module, dtype: QDtype = qint8) -> "PerTokenLinear":
        qmod = cls(mod.in_features, mod.out_features, bias=mod.bias is not None)
        codes, scale, zp = _encode_weight(mod.weight.detach().to(torch.float32), dtype)
        qmod.weight_int8, qmod.weight_scale, qmod.weight_zero_point = codes, scale, zp
        if mod.bias is not None:
            qmod.bias = mod.bias.detach().to(torch.float32)
        return qmod


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[gate; up] interleaved in blocks of ``block`` rows, the layout the gated
    GEMM epilogue pairs inside one CTA tile."""
    n = gate.shape[0]
    if n % block != 0 or gate.shape != up.shape:
        raise _lib.ShapeMismatch(f"gate/up need equal shapes and rows % {block} == 0")
    g = gate.reshape(n // block, block, *gate.shape[1:])
    u = up.reshape(n // block, block, *up.shape[1:])
    return torch.stack((g, u), dim=1).reshape(2 * n, *gate.shape[1:]).contiguous()


class GatedMLP(torch.nn.Module):
    """``down(silu(gate(x)) * up(x))`` with int8 weights and per-token int8
    activations: encode x -> one GEMM for gate and up with the SiLU-gate epilogue ->
    encode h -> down GEMM."""

    def __init__(self, d_model: int, d_ff: int) -> None:
        super().__init__()
        self.d_model, self.d_ff = d_model, d_ff
        self.register_buffer("gate_up_int8", torch.zeros((2 * d_ff, d_model), dtype=torch.int8))
        self.register_buffer("gate_up_scale", torch.ones(2 * d_ff))
        self.register_buffer("down_int8", torch.zeros((d_model, d_ff), dtype=torch.int8))
        self.register_buffer("down_scale", torch.ones(d_model))

    @classmethod
    def from_float(cls, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                   dtype: QDtype = qint8) -> "GatedMLP":
        d_ff, d_model = gate.shape
        m = cls(d_model, d_ff)
        gq, gs, _ = _encode_weight(gate.to(torch.float32), dtype)
        uq, us, _ = _encode_weight(up.to(torch.float32), dtype)
        dq, ds, _ = _encode_weight(down.to(torch.float32), dtype)
        m.gate_up_int8 = interleave_gate_up(gq, uq)
        m.gate_up_scale = interleave_gate_up(gs, us)
        m.down_int8, m.down_scale = dq, ds
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        a, s = quantize_per_token(x.reshape(-1, self.d_model), qint8)
        h = QF.gemm_s8(a, self.gate_up_int8, out_dtype=x.dtype, a_scale=s,
                       b_scale=self.gate_up_scale, act=_lib.ACT_SILU_GATE)
        hq, hs = quantize_per_token(h, qint8)
        y = QF.gemm_s8(hq, self.down_int8, out_dtype=x.dtype, a_scale=hs, b_scale=self.down_scale)
        return y.reshape(*lead, self.d_model)
