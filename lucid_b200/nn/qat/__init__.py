"""Quantization-aware-training layers (lucid/nn/qat/__init__.py): float layers whose weight and
output pass through a ``FakeQuantize``; ``convert`` turns them into the int8 inference layers."""

from .modules import (  # noqa: F401
    Conv1d,
    Conv2d,
    Conv3d,
    ConvReLU1d,
    ConvReLU2d,
    ConvReLU3d,
    Embedding,
    Linear,
    LinearReLU,
)
