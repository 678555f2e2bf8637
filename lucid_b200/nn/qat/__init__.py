"""Quantization-aware-training layers (lucid/nn/qat/__init__.py): float layers whose weight and
output pass through a ``FakeQuantize``; ``convert`` turns them into the int8 inference layers."""

from .modules import Conv2d, Linear  # noqa: F401
