"""Weight-only Linear on group-wise 4 / 8-bit codes (lucid/nn/quantized/mlx_linear.py:21-255).
The reference runs it on Metal through MLX; the class keeps its name, constructor, buffers
(``packed_weight`` int32-tagged, ``scales``, ``biases``, ``bias``) and ``from_float``, and runs
the fused decode matmul of this library."""

from __future__ import annotations

import torch

from ... import _lib
from ...quantization import _qgemm


class QuantizedLinearMLX(torch.nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, bits: int = 8,
                 group_size: int = 64, relu: bool = False) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.bits, self.group_size, self.relu = bits, group_size, relu
        self.register_buffer("packed_weight", torch.zeros((out_features, in_features * bits // 32), dtype=torch.int32))
        self.register_buffer("scales", torch.zeros((out_features, in_features // group_size)))
        self.register_buffer("biases", torch.zeros((out_features, in_features // group_size)))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _lib.require_cuda(x, "input")
        xin = x if x.dtype in (torch.float32, torch.bfloat16) else x.to(torch.float32)
        return _qgemm.quantized_matmul(xin, self.packed_weight, self.scales, self.biases, transpose=True,
                                       group_size=self.group_size, bits=self.bits, bias=self.bias, relu=self.relu)

    @classmethod
    def from_float(cls, mod: torch.nn.Module, bits: int = 8, group_size: int = 64, relu: bool = False):
        m = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, bits=bits, group_size=group_size,
                relu=relu)
        packed, scales, biases = _qgemm.quantize(mod.weight.detach(), group_size=group_size, bits=bits)
        m.packed_weight, m.scales, m.biases = packed, scales, biases
        if mod.bias is not None:
            m.bias = mod.bias.detach().to(torch.float32)
        return m

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"group_size={self.group_size}, relu={self.relu}, backend=b200")
