"""Quantized inference modules of the hot path
(lucid/nn/quantized/__init__.py:45-73): Linear, LinearReLU, Conv2d, ConvReLU2d,
the dynamic Linear family and the boundary stubs."""

from . import dynamic, functional  # noqa: F401
from .conv import Conv2d, ConvReLU2d  # noqa: F401
from .linear import Linear, LinearReLU  # noqa: F401
from .modules import DeQuantize, Quantize  # noqa: F401
from .sharded import ColumnShardedLinear  # noqa: F401
