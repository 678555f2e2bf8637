"""Graph-mode entry points ``prepare_fx`` / ``convert_fx``
(lucid/quantization/_quantize_fx.py:21-149): the eager workflow with the boundaries placed
automatically -- the model is wrapped in a ``QuantWrapper`` (input quantized, output
dequantized) and handed to ``prepare``; ``convert_fx`` is ``convert``.  The reference's point of
the graph mode is that the converted model traces through its compiler; the counterpart here is
that the converted model's launches are stream-ordered and allocation-stable, so a forward can
be captured into a CUDA graph."""

from __future__ import annotations

import torch

from ._quantize import QuantWrapper, convert, prepare


def prepare_fx(model: torch.nn.Module, qconfig_mapping=None, example_inputs=None, inplace: bool = False):
    """``prepare(QuantWrapper(model), qconfig_mapping)``; ``example_inputs`` is accepted for
    signature compatibility and unused, as in the reference."""
    return prepare(QuantWrapper(model), qconfig_mapping, inplace=inplace)


def convert_fx(model: torch.nn.Module, inplace: bool = False):
    return convert(model, inplace=inplace)
