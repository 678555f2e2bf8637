"""Dynamically quantized modules (lucid/nn/quantized/dynamic/__init__.py)."""

from .linear import GatedMLP, Linear, PerTokenLinear, interleave_gate_up  # noqa: F401
from .rnn import LSTM  # noqa: F401
