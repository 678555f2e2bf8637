"""The bounded-wait path of the integer GEMM, exercised in its harmless form: a test-only build
of the kernel (`liblucid_b200_testing.so`, compiled with -DLQ_TESTING; the product library has
no such hook) whose TMA producer issues no loads and whose waits give up after about a
millisecond.  The MMA warp's first wait runs out, every role leaves its loop, the kernel frees
its tensor memory, writes LQ_ERR_TIMEOUT to the status word and RETURNS -- nothing traps or
spins forever -- and the context stays usable: a normal GEMM right after is bit-exact."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import lucid_oracle as O

pytestmark = pytest.mark.gpu

from gpu_util import dev, host  # noqa: E402
from lucid_b200 import _lib  # noqa: E402
from lucid_b200.nn.quantized import functional as QF  # noqa: E402


def test_wait_expiry_reports_timeout_and_context_survives():
    assert os.path.exists(_lib.TEST_LIB_PATH), "build the test-only library: python -m lucid_b200.csrc.build"
    tlib = C.CDLL(_lib.TEST_LIB_PATH)
    fn = tlib.lq_test_gemm_wait_expiry
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_longlong,
                   C.c_void_p, C.c_void_p]
    rng = np.random.default_rng(0)
    m, n, k = 384, 512, 1024
    a = rng.integers(-128, 128, (m, k)).astype(np.int8)
    b = rng.integers(-128, 128, (n, k)).astype(np.int8)
    a_d, b_d = dev(a), dev(b)
    out = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    budget = 2_000_000  # SM clock cycles: about a millisecond
    t0 = torch.cuda.Event(True)
    t1 = torch.cuda.Event(True)
    t0.record()
    rc = fn(a_d.data_ptr(), b_d.data_ptr(), m, n, k, out.data_ptr(), budget, status.data_ptr(), C.c_void_p(stream))
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()  # the kernel returned by itself
    assert int(status.item()) == _lib.ERR_TIMEOUT
    assert t0.elapsed_time(t1) < 500.0  # milliseconds: a bounded wait, not the one-second default
    # the product path right after: exact
    acc = QF.gemm_s8(a_d, b_d, out_dtype=torch.int32)
    torch.cuda.synchronize()
    assert np.array_equal(host(acc), O.int_gemm_exact(a, b))
    _lib.check_device_status(torch.device("cuda", torch.cuda.current_device()))


def test_peer_wait_gives_up_and_reports():
    """The consumer-side wait of the sharded exchange on a flag nobody sets: the one-warp kernel
    returns after its budget and leaves LQ_ERR_TIMEOUT in the status word."""
    lib = _lib.load()
    d = torch.device("cuda", torch.cuda.current_device())
    flags = torch.zeros(4, dtype=torch.int32, device=d)
    epoch = torch.zeros(1, dtype=torch.int32, device=d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    st = _lib.stream_ptr(d)
    _lib.check(lib.lq_peer_wait(_lib.ptr(flags), 4, _lib.ptr(epoch), 2_000_000, _lib.ptr(status), st))
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.ERR_TIMEOUT and int(epoch.item()) == 1
    # signalled flags: the wait passes and bumps the epoch
    status.zero_()
    counter = torch.zeros(1, dtype=torch.int32, device=d)
    ptrs = (C.c_void_p * 4)(*[flags.data_ptr() + 4 * i for i in range(4)])
    for _ in range(2):  # two signals: the producers' count reaches 2 = the consumer's next epoch
        _lib.check(lib.lq_peer_signal(ptrs, 4, _lib.ptr(counter), st))
    _lib.check(lib.lq_peer_wait(_lib.ptr(flags), 4, _lib.ptr(epoch), 2_000_000, _lib.ptr(status), st))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(epoch.item()) == 2 and flags.tolist() == [2, 2, 2, 2]
