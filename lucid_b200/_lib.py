"""ctypes binding of ``liblucid_b200.so`` (the C ABI in ``include/lucid_b200.h``).

This is the thin shim that sits where the reference registers its
``engine.quantized`` ops (lucid/_C/bindings/bind_quantized.cpp:18-30): raw
device pointers in, status code out.  There is no CPU fallback: a missing
library or a non-CUDA tensor raises.
"""

from __future__ import annotations

import contextlib
import ctypes as C
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "liblucid_b200.so")
TEST_LIB_PATH = os.path.join(_HERE, "csrc", "liblucid_b200_testing.so")

# dtype / mode codes of include/lucid_b200.h
F32, BF16, S8, U8, S16, S32 = 0, 1, 2, 3, 4, 5
PER_TENSOR, PER_ROW, PER_COL = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_SILU_GATE = 0, 1, 2
MERGE_ADD, MERGE_MUL, MERGE_ADD_RELU, MERGE_COPY = 0, 1, 2, 3
ERR_TIMEOUT = 8

_TORCH_CODE = {
    torch.float32: F32, torch.bfloat16: BF16, torch.int8: S8, torch.uint8: U8,
    torch.int16: S16, torch.int32: S32,
}


# ---- error taxonomy, named after the reference's (lucid/_C/core/Error.h:63-495)
class LucidError(RuntimeError):
    pass


class ShapeMismatch(LucidError):
    pass


class DtypeMismatch(LucidError):
    pass


class DeviceMismatch(LucidError):
    pass


class EngineUnavailable(LucidError):
    pass


_STATUS_EXC = {1: ShapeMismatch, 2: DtypeMismatch, 3: DeviceMismatch, 4: ShapeMismatch,
               5: NotImplementedError, 6: LucidError, 7: LucidError, 8: TimeoutError}


class ConvGeometry(C.Structure):
    """``lq_conv_geometry_t``."""

    _fields_ = [(n, C.c_size_t) for n in
                ("N", "H", "W", "C", "K", "R", "S", "P", "Q", "stride_h", "stride_w", "pad_h", "pad_w",
                 "dil_h", "dil_w", "groups")]


class Epilogue(C.Structure):
    _fields_ = [
        ("out_dtype", C.c_int32), ("act", C.c_int32), ("a_scale_mode", C.c_int32),
        ("qmin", C.c_int32), ("qmax", C.c_int32), ("reserved", C.c_int32),
        ("a_scale", C.c_void_p), ("a_zp", C.c_void_p), ("b_rowsum", C.c_void_p),
        ("b_scale", C.c_void_p), ("bias", C.c_void_p), ("out_scale", C.c_void_p),
        ("out_zp", C.c_void_p),
    ]


_SIGNATURES = {
    "lq_version": (C.c_int, []),
    "lq_last_error": (C.c_int, [C.c_char_p, C.c_size_t]),
    "lq_reload_env": (None, []),
    "lq_minmax_workspace_bytes": (C.c_size_t, []),
    "lq_stream_timeouts": (C.c_int, [C.POINTER(C.c_uint)]),
    "lq_gemm_workspace_bytes": (C.c_size_t, []),
    "lq_gemm_s8_ws": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                C.POINTER(Epilogue), C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p,
                                C.c_void_p]),
    "lq_gemm_s8_sharded": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                     C.POINTER(Epilogue), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_size_t,
                                     C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p, C.c_size_t,
                                     C.c_void_p, C.c_void_p]),
    "lq_peer_signal": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p]),
    "lq_peer_wait": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p]),
    "lq_absmax_rows_bcast": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t,
                                       C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_void_p]),
    "lq_quantize_per_token_bcast": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_int, C.c_int,
                                              C.c_float, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int,
                                              C.c_void_p, C.c_size_t, C.c_void_p]),
    "lq_conv2d_nhwc_s8_ex": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(ConvGeometry),
                                       C.POINTER(Epilogue), C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                       C.c_void_p]),
    "lq_minmax": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p,
                            C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lq_minmax_noalloc_max_elems": (C.c_size_t, []),
    "lq_minmax_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lq_histc_workspace_bytes": (C.c_size_t, []),
    "lq_histc_max_bins": (C.c_int, []),
    "lq_histc": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_double, C.c_double, C.c_int,
                           C.c_void_p, C.c_double, C.c_double, C.c_void_p, C.c_void_p, C.c_void_p,
                           C.c_void_p, C.c_size_t, C.c_void_p]),
    "lq_histogram_observe": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lq_calculate_qparams": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
                                       C.c_void_p]),
    "lq_quantize": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                              C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                              C.c_void_p]),
    "lq_quantize_dynamic": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_float, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lq_dequantize": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_void_p,
                                C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_void_p, C.c_int,
                                C.c_void_p]),
    "lq_fake_quantize": (C.c_int, [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                                   C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_void_p]),
    "lq_quantize_per_token": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_int,
                                        C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lq_qmerge": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                            C.c_void_p, C.c_void_p, C.c_float, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int,
                            C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "lq_lut2_u8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                             C.c_void_p, C.c_int, C.c_void_p]),
    "lq_lut_u8": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lq_groupwise_quantize": (C.c_int, [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p]),
    "lq_groupwise_dequantize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int,
                                          C.c_int, C.c_void_p, C.c_void_p]),
    "lq_groupwise_matmul": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                      C.c_void_p, C.c_size_t, C.c_void_p]),
    "lq_embedding_s8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int,
                                  C.c_size_t, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_longlong, C.c_void_p,
                                  C.c_int, C.c_void_p, C.c_void_p]),
    "lq_gemm_s8": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                             C.POINTER(Epilogue), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "lq_gemm_s8_bcast": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                   C.POINTER(Epilogue), C.POINTER(C.c_void_p), C.c_int, C.c_size_t,
                                   C.c_size_t, C.c_void_p, C.c_void_p]),
    "lq_quantize_rows_bcast": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p,
                                         C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_float, C.POINTER(C.c_void_p), C.c_int, C.c_size_t,
                                         C.c_size_t, C.c_void_p, C.c_void_p]),
    "lq_gemm_s8_multicast": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                       C.POINTER(Epilogue), C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                       C.c_void_p]),
    "lq_lstm_cell_f32": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                   C.c_size_t, C.c_size_t, C.c_void_p]),
    "lq_rowsum_s8": (C.c_int, [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]),
    "lq_conv2d_nhwc_s8": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p] + [C.c_size_t] * 9 +
                          [C.POINTER(Epilogue), C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def library_present() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    """Load the shared library (no GPU needed) and declare every signature."""
    global _lib
    if _lib is None:
        if not library_present():
            raise EngineUnavailable(
                f"{LIB_PATH} is missing: build it with `python -m lucid_b200.csrc.build` "
                "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def is_available() -> bool:
    """True when the kernels can run: library built and a CUDA device visible."""
    return library_present() and torch.cuda.is_available()


def last_error() -> str:
    buf = C.create_string_buffer(512)
    load().lq_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(rc: int) -> None:
    if rc != 0:
        raise _STATUS_EXC.get(rc, LucidError)(f"lucid_b200 [{rc}]: {last_error()}")


def code_of(dt: torch.dtype) -> int:
    try:
        return _TORCH_CODE[dt]
    except KeyError:
        raise DtypeMismatch(f"dtype {dt} is not supported by the B200 quantized engine") from None


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what} must be a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise DeviceMismatch(
            f"{what} lives on {t.device}; the B200 quantized engine only runs on CUDA tensors "
            "(no CPU fallback)")


@contextlib.contextmanager
def ieee_float32():
    """The float routes (engine "reference", layers outside the integer path, the weight-only
    LSTM) restate the reference's binary32 arithmetic: keep the library's convolutions and
    matrix products off TF32 (19-bit operands) while they run."""
    old_mm = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
            yield
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_mm


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# per-(device, stream) zero-initialised workspace for the per-tensor range reduction
_minmax_ws: dict = {}


def minmax_workspace(device: torch.device) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _minmax_ws.get(key)
    if ws is None:
        n = int(load().lq_minmax_workspace_bytes())
        ws = torch.zeros(n, dtype=torch.uint8, device=device)
        _minmax_ws[key] = ws
    return ws


_gemm_ws: dict = {}
_ws_tag = threading.local()


@contextlib.contextmanager
def workspace_tag(tag):
    """Contractions issued inside run on a workspace of their own when they are captured in a
    CUDA graph.  Launches that may run concurrently (branches of a graph, i.e. independent chains
    of a step forked over several streams) must not share the scratch: give each branch its tag."""
    prev = getattr(_ws_tag, "value", None)
    _ws_tag.value = tag
    try:
        yield
    finally:
        _ws_tag.value = prev


def gemm_workspace(device: torch.device) -> torch.Tensor:
    """Zero-initialised scratch of the integer contraction (stream-K partial tiles, exchange
    ticket) for the current (device, stream); the kernels leave it zeroed."""
    cap_key = (device.index, "capture", getattr(_ws_tag, "value", None))
    if torch.cuda.is_current_stream_capturing():
        # A capture runs on a stream of its own; allocating (and zero-filling) a workspace there
        # would put a 24 MB fill into every replay.  Captured launches use one workspace per
        # device and tag, created eagerly below, so run the step once before capturing it.
        ws = _gemm_ws.get(cap_key)
        if ws is None:
            raise LucidError("run the step once eagerly before capturing it in a CUDA graph "
                             "(the contraction's workspace is created on first use)")
        return ws
    if cap_key not in _gemm_ws:
        _gemm_ws[cap_key] = torch.zeros(int(load().lq_gemm_workspace_bytes()), dtype=torch.uint8, device=device)
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _gemm_ws.get(key)
    if ws is None:
        ws = torch.zeros(int(load().lq_gemm_workspace_bytes()), dtype=torch.uint8, device=device)
        _gemm_ws[key] = ws
    return ws


_hist_ws: dict = {}


def histc_workspace(device: torch.device) -> torch.Tensor:
    """Zero-initialised workspace of ``lq_histc`` for the current (device, stream)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _hist_ws.get(key)
    if ws is None:
        ws = torch.zeros(int(load().lq_histc_workspace_bytes()), dtype=torch.uint8, device=device)
        _hist_ws[key] = ws
    return ws


# per-device word the GEMM writes LQ_ERR_TIMEOUT into when a bounded wait ran out
_status_words: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    w = _status_words.get(device.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device.index] = w
    return w


def check_device_status(device: torch.device) -> None:
    """Synchronising check of what the kernels report from the device: the status word of the
    contraction / exchange kernels and the give-up count of the pipelined stream kernels.  Raises
    ``TimeoutError`` when a bounded device-side wait ran out since the last check (the outputs of
    that launch are incomplete; the scratch workspaces are re-zeroed here)."""
    w = _status_words.get(device.index)
    code = int(w.item()) if w is not None else 0
    n = C.c_uint(0)
    with torch.cuda.device(device):
        check(load().lq_stream_timeouts(C.byref(n)))
    if code != 0 or n.value != 0:
        if w is not None:
            w.zero_()
        for key, ws in _gemm_ws.items():
            if key[0] == device.index:
                ws.zero_()
        what = f"status {code}" if code else f"{n.value} pipelined stream launch(es) gave up"
        raise _STATUS_EXC.get(code or ERR_TIMEOUT, LucidError)(f"lucid_b200: device-side {what}")


_lazy_checks: dict = {}


def check_device_status_lazily(device: torch.device, every: int = 256) -> None:
    """Called by the module layer on every forward: every ``every``-th call per device reads
    the device status (one small synchronising copy), so that a timeout inside a long-running
    service surfaces within a bounded number of calls instead of never."""
    k = _lazy_checks.get(device.index, 0) + 1
    _lazy_checks[device.index] = k
    if k % every == 0 and not torch.cuda.is_current_stream_capturing():
        check_device_status(device)
