"""Device parsing with the CUDA route added (lucid/_device.py:21-63,
lucid/_dispatch.py:255-263 accept only "cpu" and "metal")."""

from __future__ import annotations

import torch

_VALID_TYPES = {"cuda", "cpu", "metal"}


def device(spec="cuda") -> torch.device:
    """``device("cuda")`` / ``device("cuda:1")`` -> torch.device.  ``"metal"``
    is recognised and rejected: there is no Metal device here."""
    if isinstance(spec, torch.device):
        return spec
    kind = str(spec).split(":")[0]
    if kind not in _VALID_TYPES:
        raise ValueError(f"unknown device type {kind!r}; expected one of {sorted(_VALID_TYPES)}")
    if kind == "metal":
        raise RuntimeError("device 'metal' is not available on this platform; use 'cuda'")
    return torch.device(spec)
