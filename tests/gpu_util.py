"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

import lucid_b200.quantization as Q


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()


def qd_of(qmin, qmax):
    if qmin >= 0:
        return Q.QDtype("u8grid", 8, False, qmin, qmax, "int16")
    return Q.QDtype("s8grid", 8, True, qmin, qmax, "int8")


def rel_max(a, b):
    """max |a - b| / max |b| : the norm-wise metric used for float outputs."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
