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


class QConfigMapping:
    """Which ``QConfig`` applies where (lucid/quantization/qconfig.py:261-425): a per-name entry
    (the module's dotted path) wins over a per-type entry (exact class, not ``isinstance``),
    which wins over the global fallback; an entry of ``None`` leaves the module in float.
    Setters return ``self`` so they chain."""

    def __init__(self) -> None:
        self._global: QConfig | None = None
        self._object_type: dict[type, QConfig | None] = {}
        self._module_name: dict[str, QConfig | None] = {}

    def set_global(self, qconfig: QConfig | None) -> "QConfigMapping":
        self._global = qconfig
        return self

    def set_object_type(self, module_type: type, qconfig: QConfig | None) -> "QConfigMapping":
        self._object_type[module_type] = qconfig
        return self

    def set_module_name(self, name: str, qconfig: QConfig | None) -> "QConfigMapping":
        self._module_name[name] = qconfig
        return self

    def get_qconfig(self, module_type: type, module_name: str) -> QConfig | None:
        if module_name in self._module_name:
            return self._module_name[module_name]
        if module_type in self._object_type:
            return self._object_type[module_type]
        return self._global


def get_default_qconfig_mapping() -> QConfigMapping:
    """Global tier = the default static-PTQ config (lucid/quantization/qconfig.py:428-463)."""
    return QConfigMapping().set_global(get_default_qconfig())


def get_default_qat_qconfig_mapping() -> QConfigMapping:
    """Global tier = the default QAT config (lucid/quantization/qconfig.py:471-503)."""
    return QConfigMapping().set_global(get_default_qat_qconfig())
