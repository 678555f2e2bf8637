"""Fused float containers of the quantization workflow.  ``ConvReLU1d/2d/3d`` / ``LinearReLU`` are
torch's own intrinsic containers (a ``Sequential`` of the two layers); the trainable
Conv + BatchNorm fusions live in :mod:`lucid_b200.nn.intrinsic.qat`."""

from torch.ao.nn.intrinsic import ConvReLU1d, ConvReLU2d, ConvReLU3d, LinearReLU  # noqa: F401

from . import qat  # noqa: F401
