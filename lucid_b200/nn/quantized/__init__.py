"""Quantized inference modules of the hot path
(lucid/nn/quantized/__init__.py:45-73): Linear, LinearReLU, Conv2d, ConvReLU2d,
the dynamic Linear family, the boundary stubs, the element-wise merges and the activations."""

from . import dynamic, functional  # noqa: F401
from .activation import ELU, Hardsigmoid, Hardswish, LeakyReLU, ReLU, Sigmoid, Tanh  # noqa: F401
from .conv import Conv1d, Conv2d, Conv3d, ConvReLU1d, ConvReLU2d, ConvReLU3d  # noqa: F401
from .conv_transpose import ConvTranspose1d, ConvTranspose2d, ConvTranspose3d  # noqa: F401
from .functional_module import FloatFunctional, QFunctional  # noqa: F401
from .linear import Linear, LinearReLU  # noqa: F401
from .mlx_linear import QuantizedLinearMLX  # noqa: F401
from .modules import DeQuantize, DeQuantStub, Quantize, QuantStub, QuantWrapper  # noqa: F401
from .sharded import ColumnShardedLinear  # noqa: F401
from .sparse import Embedding, EmbeddingBag  # noqa: F401
