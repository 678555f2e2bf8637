"""The allocation-free range reduction, called straight through the C ABI.

`lq_minmax_noalloc` serves callers that cannot allocate device memory at the call
site (arena owners, latency-critical threads, foreign-language hosts binding only
the C header): its scratch is a fixed array inside the library.  This file runs
last so that a failure here cannot hide other tests; the checks are written to
pass both in a fresh process and after every other GPU test has used the device.
"""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_minmax(lib, _lib, x):
    """The existing entry point (caller-supplied workspace)."""
    dev = x.device
    mn = torch.empty((), dtype=torch.float32, device=dev)
    mx = torch.empty((), dtype=torch.float32, device=dev)
    ws = torch.zeros(int(lib.lq_minmax_workspace_bytes()), dtype=torch.uint8, device=dev)
    rc = lib.lq_minmax(_lib.ptr(x), _lib.code_of(x.dtype), 1, x.numel(), _lib.PER_TENSOR,
                       _lib.ptr(mn), _lib.ptr(mx), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    assert rc == 0, _lib.last_error()
    return mn, mx


@pytest.mark.parametrize("n,dtype", [(1, torch.float32), (4099, torch.float32),
                                     (1 << 24, torch.float32), (3_000_001, torch.bfloat16)])
def test_noalloc_matches_workspace_entry_point_twice(n, dtype):
    from lucid_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(n)
    xs = [torch.randn(n, device=dev, generator=g).to(dtype) * s for s in (1.0, 7.5)]
    # outputs are allocated before the calls under test; the calls themselves take no workspace
    outs = [(torch.full((), 123.0, device=dev), torch.full((), -123.0, device=dev)) for _ in xs]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    for x, (mn, mx) in zip(xs, outs):  # two calls in a row share the built-in scratch
        rc = lib.lq_minmax_noalloc(_lib.ptr(x), _lib.code_of(x.dtype), x.numel(), _lib.ptr(mn),
                                   _lib.ptr(mx), _lib.stream_ptr(dev))
        assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    for x, (mn, mx) in zip(xs, outs):
        rmn, rmx = _ref_minmax(lib, _lib, x)
        # min / max are exact in any order: the two entry points agree bit for bit
        assert mn.item() == rmn.item() and mx.item() == rmx.item()
        xf = x.float()
        assert mn.item() == xf.min().item() and mx.item() == xf.max().item()


def test_noalloc_rejects_oversize_and_bad_arguments():
    from lucid_b200 import _lib

    lib = _lib.load()
    limit = int(lib.lq_minmax_noalloc_max_elems())
    assert limit == 1 << 30
    one = C.c_void_p(256)
    assert lib.lq_minmax_noalloc(one, _lib.F32, limit + 1, one, one, None) == 1
    assert "exceed" in _lib.last_error() and "lq_minmax" in _lib.last_error()
    assert lib.lq_minmax_noalloc(one, _lib.F32, 0, one, one, None) == 1
    assert lib.lq_minmax_noalloc(None, _lib.F32, 16, one, one, None) == 3
    assert lib.lq_minmax_noalloc(one, _lib.S8, 16, one, one, None) == 2
