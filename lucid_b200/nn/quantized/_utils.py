"""Shared helpers of the quantized modules (lucid/nn/quantized/_utils.py:27-113)."""

from __future__ import annotations

import warnings
from dataclasses import dataclass

import torch

from ...quantization import (PerChannelMinMaxObserver, QDtype, per_channel_symmetric, qint8,
                             quantize)


@dataclass
class QCodes:
    """Integer codes riding along a fake-quantized float tensor, so that the
    next quantized module can consume them without re-encoding."""

    codes: torch.Tensor       # int8 or uint8, same shape as the float tensor (NHWC for conv)
    scale: torch.Tensor       # 0-d f32
    zero_point: torch.Tensor  # 0-d f32
    layout: str = "rowmajor"  # "rowmajor" | "nhwc" | "nlc" (1-D convolutions: (N, L, C))
    zp_is_zero: bool | None = None  # known on the host without a sync, when not None
    # identity of the float tensor at tag time (set by `tag`): an in-place op on the tensor
    # (relu_(), `y += identity`, nn.ReLU(inplace=True)) keeps the Python attribute but bumps
    # the version counter, and the codes no longer describe the values
    version: int = -1
    data_ptr: int = 0


def tag(t: torch.Tensor, qc: QCodes) -> torch.Tensor:
    qc.version, qc.data_ptr = t._version, t.data_ptr()
    t._lq_codes = qc
    return t


def codes_of(t: torch.Tensor):
    """The codes riding on ``t``, or None when there are none or ``t`` was modified in place
    since it was tagged (the consumer then re-encodes the float values, as the reference,
    which only ever sees the float tensor, does)."""
    qc = getattr(t, "_lq_codes", None)
    if qc is None:
        return None
    if qc.version != t._version or qc.data_ptr != t.data_ptr():
        try:
            del t._lq_codes
        except AttributeError:
            pass
        return None
    return qc


def quantize_weight(mod) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """(codes, scale, zero_point, ch_axis) of a float module's weight.

    A module with a ``qconfig`` uses its weight observer factory; otherwise the
    default per-output-channel symmetric qint8 observer."""
    weight = mod.weight.detach()
    wfq = getattr(mod, "weight_fake_quant", None)
    if wfq is not None:  # a QAT layer: refresh its weight observer on the trained weight
        wfq(weight)
        scale, zero_point = wfq.calculate_qparams()
        wobs = wfq
    else:
        qconfig = getattr(mod, "qconfig", None)
        wobs = qconfig.weight() if qconfig is not None and hasattr(qconfig, "weight") else \
            PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=qint8)
        wobs(weight)
        scale, zero_point = wobs.calculate_qparams()
    ch_axis = wobs.ch_axis
    scale, zero_point = scale.to(weight.device), zero_point.to(weight.device)
    codes = quantize(weight, scale, zero_point, wobs.qdtype, ch_axis=ch_axis)
    return codes, scale, zero_point, (ch_axis if ch_axis is not None else 0)


def activation_qparams(mod) -> tuple[torch.Tensor, torch.Tensor, QDtype]:
    """Output (scale, zero_point, qdtype) from the module's calibrated observer."""
    obs = mod.activation_post_process
    min_val = getattr(obs, "min_val", None)
    if min_val is not None and bool(torch.isinf(min_val).any().item()):
        warnings.warn(
            f"Quantizing {type(mod).__name__} whose activation observer never saw data -- "
            "calibrate the prepared model before converting, or the quantized output "
            "collapses to a near-zero grid.", stacklevel=3)
    scale, zero_point = obs.calculate_qparams()
    dev = mod.weight.device if hasattr(mod, "weight") else scale.device
    return scale.to(dev), zero_point.to(dev), obs.qdtype
