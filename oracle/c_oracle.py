"""ctypes loader for the plain-C oracle (TEST INFRASTRUCTURE ONLY).

Builds ``liblucid_oracle.so`` next to the source on first use when it is missing
(gcc only; see ``oracle/Makefile``)."""

from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "liblucid_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_DIR, "lucid_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _DIR, "-B", "liblucid_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _params(scale, zp, rows, cols):
    s = np.ascontiguousarray(np.asarray(scale, dtype=np.float32).reshape(-1))
    z = np.ascontiguousarray(np.broadcast_to(np.asarray(zp, dtype=np.float32).reshape(-1), s.shape))
    return s, z


def quantize(x, scale, zp, ch_mode, qmin, qmax, storage=np.int8):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    s, z = _params(scale, zp, rows, cols)
    out = np.empty((rows, cols), dtype=storage)
    fn = lib().lo_quantize_f32_s8 if storage == np.int8 else lib().lo_quantize_f32_s16
    fn(_p(x), C.c_size_t(rows), C.c_size_t(cols), _p(s), _p(z), C.c_int(ch_mode),
       C.c_int(qmin), C.c_int(qmax), _p(out))
    return out


def dequantize(q, scale, zp, ch_mode):
    q = np.ascontiguousarray(q)
    rows, cols = q.shape
    s, z = _params(scale, zp, rows, cols)
    out = np.empty((rows, cols), dtype=np.float32)
    fn = lib().lo_dequantize_s8_f32 if q.dtype == np.int8 else lib().lo_dequantize_s16_f32
    fn(_p(q), C.c_size_t(rows), C.c_size_t(cols), _p(s), _p(z), C.c_int(ch_mode), _p(out))
    return out


def fake_quantize(x, scale, zp, ch_mode, qmin, qmax):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    s, z = _params(scale, zp, rows, cols)
    out = np.empty((rows, cols), dtype=np.float32)
    lib().lo_fake_quantize_f32(_p(x), C.c_size_t(rows), C.c_size_t(cols), _p(s), _p(z),
                               C.c_int(ch_mode), C.c_int(qmin), C.c_int(qmax), _p(out))
    return out


def minmax_rows(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    mn = np.empty(rows, dtype=np.float32)
    mx = np.empty(rows, dtype=np.float32)
    lib().lo_minmax_rows_f32(_p(x), C.c_size_t(rows), C.c_size_t(cols), _p(mn), _p(mx))
    return mn, mx


def calculate_qparams(mn, mx, symmetric, signed, qmin, qmax, eps=1e-8):
    mn = np.ascontiguousarray(np.asarray(mn, dtype=np.float32).reshape(-1))
    mx = np.ascontiguousarray(np.asarray(mx, dtype=np.float32).reshape(-1))
    s = np.empty_like(mn)
    z = np.empty_like(mn)
    lib().lo_calculate_qparams(_p(mn), _p(mx), C.c_size_t(mn.size), C.c_int(int(symmetric)),
                               C.c_int(int(signed)), C.c_int(qmin), C.c_int(qmax),
                               C.c_float(eps), _p(s), _p(z))
    return s, z


def gemm_i8(a, w):
    a = np.ascontiguousarray(a)
    w = np.ascontiguousarray(w, dtype=np.int8)
    assert a.dtype in (np.int8, np.uint8)
    m, k = a.shape
    n = w.shape[0]
    acc = np.empty((m, n), dtype=np.int32)
    lib().lo_gemm_i8_i32(_p(a), C.c_int(int(a.dtype == np.int8)), _p(w), C.c_size_t(m),
                         C.c_size_t(n), C.c_size_t(k), _p(acc))
    return acc


def histc(x, bins, lo, hi):
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32).ravel())
    out = np.empty(bins, dtype=np.float32)
    lib().lo_histc_f32(_p(x), C.c_size_t(x.size), C.c_int(bins), C.c_double(lo), C.c_double(hi), _p(out))
    return out


def histogram_rebin(hist, old_min, old_max, new_min, new_max):
    hist = np.ascontiguousarray(hist, dtype=np.float32)
    out = np.empty_like(hist)
    lib().lo_hist_rebin_f32(_p(hist), C.c_int(hist.size), C.c_double(old_min), C.c_double(old_max),
                            C.c_double(new_min), C.c_double(new_max), _p(out))
    return out


def qfunctional(op, x, y, scale, zp, qmin, qmax):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.ascontiguousarray(np.broadcast_to(np.asarray(y, dtype=np.float32), x.shape))
    out = np.empty_like(x)
    lib().lo_qfunctional_f32(C.c_int({"add": 0, "mul": 1, "add_relu": 2}[op]), _p(x), _p(y), C.c_size_t(x.size),
                             C.c_float(scale), C.c_float(zp), C.c_int(qmin), C.c_int(qmax), _p(out))
    return out


def groupwise_quantize(w, group_size=64, bits=8):
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    packed = np.empty((n, k * bits // 32), dtype=np.uint32)
    scales = np.empty((n, k // group_size), dtype=np.float32)
    biases = np.empty((n, k // group_size), dtype=np.float32)
    lib().lo_groupwise_quantize(_p(w), C.c_size_t(n), C.c_size_t(k), C.c_int(group_size), C.c_int(bits),
                                _p(packed), _p(scales), _p(biases))
    return packed, scales, biases


def groupwise_dequantize(packed, scales, biases, group_size=64, bits=8):
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    biases = np.ascontiguousarray(biases, dtype=np.float32)
    n, k = packed.shape[0], packed.shape[1] * 32 // bits
    out = np.empty((n, k), dtype=np.float32)
    lib().lo_groupwise_dequantize(_p(packed), _p(scales), _p(biases), C.c_size_t(n), C.c_size_t(k),
                                  C.c_int(group_size), C.c_int(bits), _p(out))
    return out


def per_token_quantize(x, eps=1e-8):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), dtype=np.int8)
    s = np.empty(rows, dtype=np.float32)
    lib().lo_per_token_quantize_f32_s8(_p(x), C.c_size_t(rows), C.c_size_t(cols), C.c_float(eps), _p(q), _p(s))
    return q, s


def int_gemm(a, w):
    a, w = np.ascontiguousarray(a), np.ascontiguousarray(w, dtype=np.int8)
    (m, k), n = a.shape, w.shape[0]
    acc = np.empty((m, n), dtype=np.int32)
    lib().lo_gemm_i8_i32(_p(a), C.c_int(int(a.dtype == np.int8)), _p(w), C.c_size_t(m), C.c_size_t(n), C.c_size_t(k), _p(acc))
    return acc


def linear_epilogue(acc, a_scale, w_scale, bias=None, relu=False, out_bf16=False):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    m, n = acc.shape
    a_s = np.ascontiguousarray(np.broadcast_to(np.asarray(a_scale, dtype=np.float32).reshape(-1), (m,)))
    w_s = np.ascontiguousarray(w_scale, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    y = np.empty((m, n), dtype=np.float32)
    lib().lo_linear_epilogue_f32(_p(acc), C.c_size_t(m), C.c_size_t(n), _p(a_s), _p(w_s),
                                 None if b is None else _p(b), C.c_int(int(relu)), C.c_int(int(out_bf16)), _p(y))
    return y


def requantize(y, out_scale, out_zp, qmin, qmax):
    y = np.ascontiguousarray(y, dtype=np.float32)
    out = np.empty(y.shape, dtype=np.float32)
    lib().lo_requantize_f32(_p(y), C.c_size_t(y.size), C.c_float(out_scale), C.c_float(out_zp), C.c_int(qmin),
                            C.c_int(qmax), _p(out))
    return out
