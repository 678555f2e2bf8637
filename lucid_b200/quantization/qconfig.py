"""``QConfig``: the (activation, weight) observer recipe
(lucid/quantization/qconfig.py:35-192)."""

from __future__ import annotations

from typing import Callable, NamedTuple

from ._qscheme import per_channel_symmetric, per_tensor_affine, qint8, quint8
from .observer import HistogramObserver, MovingAverageMinMaxObserver, PerChannelMinMaxObserver


class QConfig(NamedTuple):
    """Two zero-argument factories: one observer per insertion site."""

    activation: Callable[..., object]
    weight: Callable[..., object]


def get_default_qconfig() -> QConfig:
    """Per-tensor affine quint8 activations calibrated by the histogram observer,
    per-output-channel symmetric qint8 weights (lucid/quantization/qconfig.py:180-192)."""
    return QConfig(
        activation=HistogramObserver.with_args(qscheme=per_tensor_affine, qdtype=quint8),
        weight=PerChannelMinMaxObserver.with_args(ch_axis=0, qscheme=per_channel_symmetric,
                                                  qdtype=qint8),
    )


def get_default_qat_qconfig() -> QConfig:
    """The same grids as :func:`get_default_qconfig`, each observer wrapped in a
    ``FakeQuantize``; activations follow a moving-average min / max
    (lucid/quantization/qconfig.py:195-260)."""
    from ._fake_quantize import FakeQuantize

    return QConfig(
        activation=FakeQuantize.with_args(observer=MovingAverageMinMaxObserver, qscheme=per_tensor_affine,
                                          qdtype=quint8),
        weight=FakeQuantize.with_args(observer=PerChannelMinMaxObserver, ch_axis=0,
                                      qscheme=per_channel_symmetric, qdtype=qint8),
    )
