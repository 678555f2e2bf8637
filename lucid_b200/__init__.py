"""lucid_b200 -- B200-native implementation of Lucid's quantized-inference hot
path: ``lucid.quantization`` affine int8 quantize / dequantize / fake-quantize
with their calibration, and the quantized Linear / Conv2d contraction as a true
s8 x s8 -> s32 tensor-core GEMM with a fused epilogue.

    import lucid_b200 as lucid
    import lucid_b200.quantization as Q
    q = Q.quantize(x_cuda, 0.05, 0.0, Q.qint8)

Tensors are torch CUDA tensors.  There is no CPU path: a missing CUDA extension
or a CPU tensor raises.
"""

from . import backends, nn, quantization  # noqa: F401
from ._device import device  # noqa: F401
from ._pipeline import HostPipeline  # noqa: F401
from ._lib import (DeviceMismatch, DtypeMismatch, EngineUnavailable, LucidError,  # noqa: F401
                   ShapeMismatch, is_available)

__version__ = "0.1.0"
