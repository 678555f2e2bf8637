"""A NumPy stand-in for a handful of C-ABI entry points -- TEST INFRASTRUCTURE ONLY.

The package has no CPU path: without the CUDA library every call raises.  The CPU test suite
still wants to exercise the HOST logic around the kernels (what ``prepare_qat`` swaps, what
``convert`` builds from a trained module, which scale / zero point / row sum reaches which slot
of an epilogue).  ``install`` replaces, for the duration of one test, ``lucid_b200._lib.load`` by
an object that implements in NumPy, on host pointers, the entry points those paths touch:

* streams: ``lq_quantize``, ``lq_dequantize``, ``lq_fake_quantize``, ``lq_minmax``,
  ``lq_calculate_qparams``, ``lq_histogram_observe``, ``lq_quantize_dynamic``, the plain ``lq_embedding_s8`` gather;
* contractions: ``lq_rowsum_s8``, ``lq_gemm_s8_ws``, ``lq_conv2d_nhwc_s8_ex`` (the oracle's exact
  convolution), with the epilogue as ``include/lucid_b200.h`` states it;
* merges and byte tables: ``lq_qmerge``, ``lq_lut_u8``, ``lq_lut2_u8``;
* the recurrent cell ``lq_lstm_cell_f32``;
* the group-wise weight-only route: ``lq_groupwise_quantize`` / ``_dequantize`` / ``_matmul``.

It also lifts the device checks and sets the engine (``"reference"`` by default: layers run the
reference's float sequence; ``"auto"`` runs the integer routes through the stand-in).  The
arithmetic is the oracle's (same operation order).  Nothing here is importable from the package
and nothing in the package knows about it."""

from __future__ import annotations

import collections
import contextlib
import ctypes as C

import numpy as np
import torch

_NP = {0: np.float32, 2: np.int8, 3: np.uint8, 4: np.int16, 5: np.int32}


def _addr(p):
    if p is None:
        return None
    return p.value if isinstance(p, C.c_void_p) else int(p)


def _arr(p, code, n):
    a = _addr(p)
    if a is None or n == 0:
        return None
    dt = np.dtype(_NP[code])
    return np.frombuffer((C.c_char * (n * dt.itemsize)).from_address(a), dtype=dt)


def _f(v):
    return float(v.value) if isinstance(v, C.c_float) else float(v)


def _grid(sp, zp, sv, zv, rows, cols, mode):
    """(scale, zero_point) broadcastable over a (rows, cols) view: scalars passed by value, or
    one entry per tensor / row / column behind the pointers."""
    if _addr(sp) is None:
        return np.float32(_f(sv)), np.float32(_f(zv))
    n = 1 if mode == 0 else (rows if mode == 1 else cols)
    s, z = _arr(sp, 0, n), _arr(zp, 0, n)
    if mode == 0:
        return s[0], z[0]
    return (s[:, None], z[:, None]) if mode == 1 else (s[None, :], z[None, :])


class StandIn:
    """The operation order of lucid/quantization/_functional.py:175-182, 269-281, 299-331 and
    _qparams.py:197-215, on host memory.  ``calls`` counts the contractions that ran (a test can
    tell the integer route from the float one by it)."""

    def __init__(self) -> None:
        self.calls = collections.Counter()

    def lq_quantize(self, x, xcode, rows, cols, sp, zp, sv, zv, mode, qmin, qmax, out, ocode, stream):
        X = _arr(x, xcode, rows * cols).reshape(rows, cols)
        s, z = _grid(sp, zp, sv, zv, rows, cols, mode)
        q = np.clip(np.rint((X / s).astype(np.float32)) + z, qmin, qmax)
        _arr(out, ocode, rows * cols).reshape(rows, cols)[...] = q.astype(_NP[ocode])
        return 0

    def lq_dequantize(self, q, qcode, rows, cols, sp, zp, sv, zv, mode, out, ocode, stream):
        codes = _arr(q, qcode, rows * cols).reshape(rows, cols).astype(np.float32)
        s, z = _grid(sp, zp, sv, zv, rows, cols, mode)
        _arr(out, ocode, rows * cols).reshape(rows, cols)[...] = ((codes - z) * s).astype(np.float32)
        return 0

    def lq_fake_quantize(self, x, rows, cols, sp, zp, sv, zv, mode, qmin, qmax, out, mask, stream):
        X = _arr(x, 0, rows * cols).reshape(rows, cols)
        s, z = _grid(sp, zp, sv, zv, rows, cols, mode)
        t = np.rint((X / s).astype(np.float32)) + z
        _arr(out, 0, rows * cols).reshape(rows, cols)[...] = ((np.clip(t, qmin, qmax) - z) * s).astype(np.float32)
        if _addr(mask) is not None:
            _arr(mask, 0, rows * cols).reshape(rows, cols)[...] = ((t >= qmin) & (t <= qmax)).astype(np.float32)
        return 0

    def lq_minmax(self, x, code, rows, cols, mode, mn, mx, ws, ws_bytes, stream):
        X = _arr(x, code, rows * cols).reshape(rows, cols)
        if mode == 1:
            _arr(mn, 0, rows)[...] = X.min(axis=1)
            _arr(mx, 0, rows)[...] = X.max(axis=1)
        else:
            _arr(mn, 0, 1)[0] = X.min()
            _arr(mx, 0, 1)[0] = X.max()
        return 0

    def lq_histogram_observe(self, x, code, n, bins, min_val, max_val, hist, ws, ws_bytes, stream):
        """One HistogramObserver batch on the state behind the pointers (the oracle's step)."""
        from oracle import lucid_oracle as O

        mn, mx, h = _arr(min_val, 0, 1), _arr(max_val, 0, 1), _arr(hist, 0, bins)
        state = None if not np.isfinite(mn[0]) else (float(mn[0]), float(mx[0]), h.copy())
        mn[0], mx[0], h[...] = O.histogram_observe(_arr(x, code, n), state, bins)
        return 0

    def lq_histc_workspace_bytes(self):
        return 64

    def lq_minmax_workspace_bytes(self):
        return 64

    def lq_calculate_qparams(self, mn, mx, n, symmetric, is_signed, qmin, qmax, eps, scale, zp, stream):
        lo = np.minimum(_arr(mn, 0, n), np.float32(0))
        hi = np.maximum(_arr(mx, 0, n), np.float32(0))
        e = np.float32(_f(eps))
        if symmetric:
            m = np.maximum(np.abs(lo), np.abs(hi))
            _arr(scale, 0, n)[...] = np.maximum(m / np.float32((qmax - qmin) / 2.0), e)
            _arr(zp, 0, n)[...] = 0.0 if is_signed else float((qmax + qmin + 1) // 2)
        else:
            s = np.maximum(((hi - lo) / np.float32(qmax - qmin)).astype(np.float32), e)
            _arr(scale, 0, n)[...] = s
            _arr(zp, 0, n)[...] = np.clip(np.float32(qmin) - np.rint((lo / s).astype(np.float32)), qmin, qmax)
        return 0

    def lq_embedding_s8(self, w, w_scale, w_zp, rows, dim, idx, idx_bits, n, offsets, n_bags, include_last, mode,
                        padding_idx, out, ocode, status, stream):
        if _addr(offsets) is not None:
            raise NotImplementedError("the stand-in gathers rows only (no bags)")
        table = _arr(w, 2, rows * dim).reshape(rows, dim).astype(np.float32)
        s, z = _arr(w_scale, 0, rows), _arr(w_zp, 0, rows)
        index = np.frombuffer((C.c_char * (n * idx_bits // 8)).from_address(_addr(idx)),
                              dtype=np.int64 if idx_bits == 64 else np.int32)
        got = ((table[index] - z[index][:, None]) * s[index][:, None]).astype(np.float32)
        if padding_idx >= 0:
            got[index == padding_idx] = 0.0
        _arr(out, ocode, n * dim).reshape(n, dim)[...] = got
        return 0


    # ---- the integer Linear: row sums, dynamic encode, contraction + epilogue -----------------
    def lq_rowsum_s8(self, b, n, k, out, stream):
        _arr(out, 5, n)[...] = _arr(b, 2, n * k).reshape(n, k).astype(np.int32).sum(axis=1)
        return 0

    def lq_quantize_dynamic(self, x, code, rows, cols, symmetric, is_signed, qmin, qmax, eps, ws, ws_bytes, out,
                            ocode, out_scale, out_zp, out_minmax, stream):
        X = _arr(x, code, rows * cols)
        mm = _arr(out_minmax, 0, 2)
        mm[0], mm[1] = X.min(), X.max()
        self.lq_calculate_qparams(C.c_void_p(_addr(out_minmax)), C.c_void_p(_addr(out_minmax) + 4), 1, symmetric,
                                  is_signed, qmin, qmax, eps, out_scale, out_zp, None)
        s, z = _arr(out_scale, 0, 1)[0], _arr(out_zp, 0, 1)[0]
        _arr(out, ocode, rows * cols)[...] = np.clip(np.rint((X / s).astype(np.float32)) + z, qmin, qmax).astype(_NP[ocode])
        return 0

    @staticmethod
    def _epilogue(acc, e, m, n):
        """The epilogue of include/lucid_b200.h on exact accumulators ``acc (m, n)`` (int64):
        t = acc - a_zp * rowsum(b); S32: out = t; otherwise y = f32(t) * (a_scale * b_scale) + bias,
        optional ReLU, then float, or clip(rint(y / out_scale) + out_zp, qmin, qmax) for 8-bit."""
        if e.act not in (0, 1):
            raise NotImplementedError("the stand-in has no gated activation")
        if e.a_zp and e.b_rowsum:
            acc = acc - np.int64(_arr(e.a_zp, 0, 1)[0]) * _arr(e.b_rowsum, 5, n).astype(np.int64)[None, :]
        if e.out_dtype == 5:
            return acc.astype(np.int32)
        a_s = _arr(e.a_scale, 0, m if e.a_scale_mode == 1 else 1).reshape(-1, 1) if e.a_scale else np.float32(1)
        b_s = _arr(e.b_scale, 0, n).reshape(1, -1) if e.b_scale else np.float32(1)
        y = acc.astype(np.int32).astype(np.float32) * (a_s * b_s).astype(np.float32)
        if e.bias:
            y = (y + _arr(e.bias, 0, n).reshape(1, -1)).astype(np.float32)
        if e.act == 1:
            y = np.maximum(y, np.float32(0))
        if e.out_dtype in (2, 3):
            s, z = _arr(e.out_scale, 0, 1)[0], _arr(e.out_zp, 0, 1)[0]
            y = np.clip(np.rint((y / s).astype(np.float32)) + z, e.qmin, e.qmax)
        elif e.out_dtype != 0:
            raise NotImplementedError("the stand-in writes f32, s32 and 8-bit outputs")
        return y.astype(_NP[e.out_dtype])

    def lq_gemm_s8_ws(self, a, a_signed, b, m, n, k, e_ref, out, ldo, ws, ws_bytes, status, stream):
        e = e_ref._obj
        self.calls["gemm"] += 1
        A = _arr(a, 2 if a_signed else 3, m * k).reshape(m, k).astype(np.int64)
        B = _arr(b, 2, n * k).reshape(n, k).astype(np.int64)
        if ldo != n:
            raise NotImplementedError("the stand-in writes dense outputs")
        _arr(out, e.out_dtype, m * n).reshape(m, n)[...] = self._epilogue(A @ B.T, e, m, n)
        return 0

    def lq_conv2d_nhwc_s8_ex(self, x, a_signed, w, g_ref, e_ref, out, ws, ws_bytes, status, stream):
        """NHWC codes * KRSC codes; out-of-image taps read code 0; the output extent (P, Q) is the
        caller's (a larger one than the leading padding alone gives means trailing padding)."""
        from oracle import lucid_oracle as O

        g, e = g_ref._obj, e_ref._obj
        self.calls["conv"] += 1
        cg = g.C // g.groups
        X = _arr(x, 2 if a_signed else 3, g.N * g.H * g.W * g.C).reshape(g.N, g.H, g.W, g.C)
        Wt = _arr(w, 2, g.K * g.R * g.S * cg).reshape(g.K, g.R, g.S, cg)
        hi_h = max(0, (g.P - 1) * g.stride_h + g.dil_h * (g.R - 1) + 1 - g.H - g.pad_h)
        hi_w = max(0, (g.Q - 1) * g.stride_w + g.dil_w * (g.S - 1) + 1 - g.W - g.pad_w)
        acc = O.int_conv2d_nhwc_general(X, Wt, (g.stride_h, g.stride_w), (g.pad_h, g.pad_w), (hi_h, hi_w),
                                        (g.dil_h, g.dil_w), g.groups, zp=0)[:, :g.P, :g.Q, :]
        m = g.N * g.P * g.Q
        got = self._epilogue(np.ascontiguousarray(acc).reshape(m, g.K).astype(np.int64), e, m, g.K)
        _arr(out, e.out_dtype, m * g.K).reshape(m, g.K)[...] = got
        return 0

    # ---- element-wise merges and byte tables ---------------------------------------------------
    @staticmethod
    def _operand(p, code, sp, zp, n):
        v = _arr(p, code, n)
        if code in (2, 3, 4):  # codes: decoded as lq_dequantize would
            return ((v.astype(np.float32) - _arr(zp, 0, 1)[0]) * _arr(sp, 0, 1)[0]).astype(np.float32)
        if code != 0:
            raise NotImplementedError("the stand-in merges f32 values and integer codes")
        return v

    def lq_qmerge(self, op, x, xcode, xs, xz, y, ycode, ys, yz, y_scalar, n, out_scale, out_zp, qmin, qmax, out_codes,
                  ccode, out_f32, stream):
        self.calls["merge"] += 1
        a = self._operand(x, xcode, xs, xz, n)
        b = np.float32(_f(y_scalar)) if _addr(y) is None else self._operand(y, ycode, ys, yz, n)
        t = a if op == 3 else ((a * b) if op == 1 else (a + b)).astype(np.float32)
        if op == 2:
            t = np.maximum(t, np.float32(0))
        S, Z = _arr(out_scale, 0, 1)[0], _arr(out_zp, 0, 1)[0]
        q = np.clip(np.rint((t / S).astype(np.float32)) + Z, qmin, qmax)
        if _addr(out_codes) is not None:
            _arr(out_codes, ccode, n)[...] = q.astype(_NP[ccode])
        if _addr(out_f32) is not None:
            _arr(out_f32, 0, n)[...] = ((q - Z) * S).astype(np.float32)
        return 0

    def lq_lut_u8(self, codes, n, table, out, stream):
        self.calls["lut"] += 1
        _arr(out, 3, n)[...] = _arr(table, 3, 256)[_arr(codes, 3, n)]
        return 0

    def lq_lut2_u8(self, x, y, n, table, out_codes, out_f32, out_scale, out_zp, is_signed, stream):
        self.calls["lut2"] += 1
        got = _arr(table, 3, 65536)[_arr(x, 3, n).astype(np.int64) * 256 + _arr(y, 3, n)]
        if _addr(out_codes) is not None:
            _arr(out_codes, 3, n)[...] = got
        if _addr(out_f32) is not None:
            q = got.view(np.int8).astype(np.float32) if is_signed else got.astype(np.float32)
            _arr(out_f32, 0, n)[...] = ((q - _arr(out_zp, 0, 1)[0]) * _arr(out_scale, 0, 1)[0]).astype(np.float32)
        return 0

    # ---- group-wise weight-only codes (the oracle's restatement) ---------------------------------
    def lq_groupwise_quantize(self, w, n, k, group, bits, packed, scales, biases, stream):
        from oracle import lucid_oracle as O

        p, s, b = O.groupwise_quantize(_arr(w, 0, n * k).reshape(n, k), group, bits)
        _arr(packed, 5, n * k * bits // 32).view(np.uint32)[...] = p.reshape(-1)
        _arr(scales, 0, n * (k // group))[...] = s.reshape(-1)
        _arr(biases, 0, n * (k // group))[...] = b.reshape(-1)
        return 0

    def _gw(self, packed, scales, biases, n, k, group, bits):
        return (_arr(packed, 5, n * k * bits // 32).view(np.uint32).reshape(n, -1),
                _arr(scales, 0, n * (k // group)).reshape(n, -1), _arr(biases, 0, n * (k // group)).reshape(n, -1))

    def lq_groupwise_dequantize(self, packed, scales, biases, n, k, group, bits, out, stream):
        from oracle import lucid_oracle as O

        _arr(out, 0, n * k).reshape(n, k)[...] = O.groupwise_dequantize(*self._gw(packed, scales, biases, n, k, group, bits),
                                                                         group, bits)
        return 0

    def lq_groupwise_matmul(self, x, xcode, m, ldx, packed, scales, biases, n, k, group, bits, bias, relu, out, ldo, stream):
        from oracle import lucid_oracle as O

        if xcode != 0 or ldx != k or ldo != n:
            raise NotImplementedError("the stand-in multiplies dense f32 activations")
        self.calls["groupwise"] += 1
        y = O.groupwise_matmul_f64(_arr(x, 0, m * k).reshape(m, k), *self._gw(packed, scales, biases, n, k, group, bits),
                                   group, bits)
        if _addr(bias) is not None:
            y = y + _arr(bias, 0, n)[None, :]
        if relu:
            y = np.maximum(y, 0.0)
        _arr(out, 0, m * n).reshape(m, n)[...] = y.astype(np.float32)
        return 0

    def lq_lstm_cell_f32(self, gates, ldg, c_prev, h_out, ldh, c_out, batch, hidden, stream):
        """c = sigmoid(f) * c_prev + sigmoid(i) * tanh(g); h = sigmoid(o) * tanh(c); gate order i, f, g, o."""
        self.calls["lstm_cell"] += 1
        if ldg != 4 * hidden or ldh != hidden:
            raise NotImplementedError("the stand-in reads dense gates")
        g = _arr(gates, 0, batch * 4 * hidden).reshape(batch, 4, hidden).astype(np.float64)
        sig = lambda v: 1.0 / (1.0 + np.exp(-v))  # noqa: E731
        c = sig(g[:, 1]) * _arr(c_prev, 0, batch * hidden).reshape(batch, hidden) + sig(g[:, 0]) * np.tanh(g[:, 2])
        _arr(c_out, 0, batch * hidden).reshape(batch, hidden)[...] = c.astype(np.float32)
        _arr(h_out, 0, batch * hidden).reshape(batch, hidden)[...] = (sig(g[:, 3]) * np.tanh(c)).astype(np.float32)
        return 0

    def lq_gemm_workspace_bytes(self):
        return 64


def install(monkeypatch, engine: str = "reference", pose_as_cuda: bool = False) -> StandIn:
    """Stand the NumPy object in for the library until the end of the calling test.
    ``pose_as_cuda`` makes CPU tensors answer ``is_cuda`` with True, for the modules that only
    read carried codes off device tensors."""
    from lucid_b200 import _lib, backends

    fake = StandIn()

    @contextlib.contextmanager
    def plain_float32():
        yield

    monkeypatch.setattr(_lib, "load", lambda: fake)
    monkeypatch.setattr(_lib, "require_cuda", lambda t, what: None)
    monkeypatch.setattr(_lib, "stream_ptr", lambda device=None: None)
    monkeypatch.setattr(_lib, "check_device_status_lazily", lambda device, every=256: None)
    monkeypatch.setattr(_lib, "minmax_workspace", lambda device: torch.zeros(64, dtype=torch.uint8))
    monkeypatch.setattr(_lib, "status_word", lambda device: torch.zeros(1, dtype=torch.int32))
    monkeypatch.setattr(_lib, "histc_workspace", lambda device: torch.zeros(64, dtype=torch.uint8))
    monkeypatch.setattr(_lib, "ieee_float32", plain_float32)
    monkeypatch.setattr(torch.cuda, "device", lambda dev: contextlib.nullcontext())
    monkeypatch.setattr(_lib, "gemm_workspace", lambda device: torch.zeros(64, dtype=torch.uint8))
    monkeypatch.setattr(backends.quantized, "_engine", engine)
    if pose_as_cuda:
        monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    return fake
