"""B200-native drop-in for the hot part of ``lucid.quantization``
(lucid/quantization/__init__.py:58-65): schemes, grids, qparams, the three
affine primitives and the calibration observers."""

from ._functional import (dequantize, fake_quantize, quantize, quantize_dynamic_per_tensor,  # noqa: F401
                          quantize_per_token, quantize_to)
from ._qparams import QParams, calculate_qparams  # noqa: F401
from ._qscheme import (QDtype, QScheme, per_channel_affine, per_channel_symmetric,  # noqa: F401
                       per_tensor_affine, per_tensor_symmetric, qint4, qint8, qint32, quint8)
from .observer import (FixedQParamsObserver, HistogramObserver, MinMaxObserver,  # noqa: F401
                       MovingAverageMinMaxObserver, MovingAveragePerChannelMinMaxObserver,
                       NoopObserver, ObserverBase, PerChannelMinMaxObserver, PlaceholderObserver,
                       histc, minmax)
from ._quantize import DeQuantStub, QuantStub, QuantWrapper, convert, prepare, quantize_dynamic  # noqa: F401,E402
from ._fake_quantize import FakeQuantize  # noqa: F401,E402
from ._quantize import prepare_qat  # noqa: F401,E402
from ._quantize_fx import convert_fx, prepare_fx  # noqa: F401,E402
from .fuse_modules import fuse_conv_bn_eval, fuse_modules, fuse_modules_qat  # noqa: F401,E402
from .qconfig import (  # noqa: F401,E402
    QConfig,
    QConfigMapping,
    get_default_qat_qconfig,
    get_default_qat_qconfig_mapping,
    get_default_qconfig,
    get_default_qconfig_mapping,
)
