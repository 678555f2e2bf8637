"""``lucid.nn`` surface of the hot path: only the quantized inference modules."""

from . import quantized  # noqa: F401
