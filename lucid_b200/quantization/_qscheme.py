"""Quantization grids and schemes: the metadata half of the path.

Same public names and values as the reference (lucid/quantization/_qscheme.py:25-245);
``storage`` names a torch dtype here.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class QScheme(enum.Enum):
    """Granularity x symmetry of the affine map (lucid/quantization/_qscheme.py:25-128)."""

    PER_TENSOR_AFFINE = "per_tensor_affine"
    PER_TENSOR_SYMMETRIC = "per_tensor_symmetric"
    PER_CHANNEL_AFFINE = "per_channel_affine"
    PER_CHANNEL_SYMMETRIC = "per_channel_symmetric"

    @property
    def is_per_channel(self) -> bool:
        return self in (QScheme.PER_CHANNEL_AFFINE, QScheme.PER_CHANNEL_SYMMETRIC)

    @property
    def is_symmetric(self) -> bool:
        return self in (QScheme.PER_TENSOR_SYMMETRIC, QScheme.PER_CHANNEL_SYMMETRIC)

    def __repr__(self) -> str:
        return f"lucid.quantization.{self.value}"


per_tensor_affine = QScheme.PER_TENSOR_AFFINE
per_tensor_symmetric = QScheme.PER_TENSOR_SYMMETRIC
per_channel_affine = QScheme.PER_CHANNEL_AFFINE
per_channel_symmetric = QScheme.PER_CHANNEL_SYMMETRIC


@dataclass(frozen=True)
class QDtype:
    """Integer grid descriptor (lucid/quantization/_qscheme.py:131-239).

    ``quint8`` codes are carried in ``int16`` because the reference engine has
    no unsigned 8-bit dtype; the kernels keep them as u8 internally."""

    name: str
    bits: int
    signed: bool
    quant_min: int
    quant_max: int
    storage: str

    @property
    def torch_storage(self) -> torch.dtype:
        return getattr(torch, self.storage)

    def __repr__(self) -> str:
        return f"lucid.quantization.{self.name}"


qint8 = QDtype("qint8", 8, True, -128, 127, "int8")
quint8 = QDtype("quint8", 8, False, 0, 255, "int16")
qint32 = QDtype("qint32", 32, True, -(2**31), 2**31 - 1, "int32")
qint4 = QDtype("qint4", 4, True, -8, 7, "int8")
