/*
 * Plain-C restatement of the reference's quantization arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: this file is a checker for the CUDA kernels (and a
 * second, independent restatement that the NumPy oracle is cross-checked
 * against).  The shipped library never links or calls it.
 *
 * Build with IEEE semantics intact: no -ffast-math, -ffp-contract=off.
 * rintf() under the default rounding mode rounds ties to even, matching the
 * reference's CPU round (lucid/_C/backend/cpu/Vforce.cpp:136,
 * lucid/_C/ops/ufunc/Discrete.h:44); '/' is a true divide like vDSP_vdiv
 * (lucid/_C/backend/cpu/Vdsp.cpp:47-49).
 *
 * Parity pin: checked against the fixtures produced by executing the
 * reference's Python sources (tests/golden/reference_vectors.npz) and the
 * known answers in lucid/test/unit/quantization/test_functional.py.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

/* clip: v < lo ? lo : (v > hi ? hi : v)   lucid/_C/backend/cpu/CpuBackend.h:6863-6892 */
static inline float clipf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* quantize, lucid/quantization/_functional.py:180-182.
 * ch_mode 0: scalar scale/zp; 1: one per row (ch_axis=0); 2: one per column (last axis). */
static inline float code_of(float x, float s, float z, float qmin, float qmax) {
  float t = x / s;
  t = rintf(t);
  t = t + z;
  return clipf(t, qmin, qmax);
}

#define PARAM(arr, mode, r, c) ((mode) == 0 ? (arr)[0] : ((mode) == 1 ? (arr)[r] : (arr)[c]))

void lo_quantize_f32_s8(const float* x, size_t rows, size_t cols, const float* scale,
                        const float* zp, int ch_mode, int qmin, int qmax, int8_t* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      float s = PARAM(scale, ch_mode, r, c), z = PARAM(zp, ch_mode, r, c);
      out[r * cols + c] = (int8_t)code_of(x[r * cols + c], s, z, (float)qmin, (float)qmax);
    }
}

/* quint8 codes ride in int16 storage (lucid/quantization/_qscheme.py:243). */
void lo_quantize_f32_s16(const float* x, size_t rows, size_t cols, const float* scale,
                         const float* zp, int ch_mode, int qmin, int qmax, int16_t* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      float s = PARAM(scale, ch_mode, r, c), z = PARAM(zp, ch_mode, r, c);
      out[r * cols + c] = (int16_t)code_of(x[r * cols + c], s, z, (float)qmin, (float)qmax);
    }
}

/* dequantize, lucid/quantization/_functional.py:281: (f32(q) - z) * s */
void lo_dequantize_s8_f32(const int8_t* q, size_t rows, size_t cols, const float* scale,
                          const float* zp, int ch_mode, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      float s = PARAM(scale, ch_mode, r, c), z = PARAM(zp, ch_mode, r, c);
      float u = (float)q[r * cols + c];
      u = u - z;
      out[r * cols + c] = u * s;
    }
}

void lo_dequantize_s16_f32(const int16_t* q, size_t rows, size_t cols, const float* scale,
                           const float* zp, int ch_mode, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      float s = PARAM(scale, ch_mode, r, c), z = PARAM(zp, ch_mode, r, c);
      float u = (float)q[r * cols + c];
      u = u - z;
      out[r * cols + c] = u * s;
    }
}

/* fake_quantize forward, lucid/quantization/_functional.py:311-313 */
void lo_fake_quantize_f32(const float* x, size_t rows, size_t cols, const float* scale,
                          const float* zp, int ch_mode, int qmin, int qmax, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      float s = PARAM(scale, ch_mode, r, c), z = PARAM(zp, ch_mode, r, c);
      float q = code_of(x[r * cols + c], s, z, (float)qmin, (float)qmax);
      q = q - z;
      out[r * cols + c] = q * s;
    }
}

/* Per-row min/max (PerChannelMinMaxObserver with ch_axis=0,
 * lucid/quantization/observer.py:635-648); rows==1 gives the per-tensor case. */
void lo_minmax_rows_f32(const float* x, size_t rows, size_t cols, float* out_min, float* out_max) {
  for (size_t r = 0; r < rows; ++r) {
    float mn = INFINITY, mx = -INFINITY;
    for (size_t c = 0; c < cols; ++c) {
      float v = x[r * cols + c];
      mn = v < mn ? v : mn;
      mx = v > mx ? v : mx;
    }
    out_min[r] = mn;
    out_max[r] = mx;
  }
}

/* calculate_qparams, lucid/quantization/_qparams.py:197-215 */
void lo_calculate_qparams(const float* mn, const float* mx, size_t n, int symmetric, int is_signed,
                          int qmin, int qmax, float eps, float* scale, float* zp) {
  for (size_t i = 0; i < n; ++i) {
    float lo = mn[i] < 0.0f ? mn[i] : 0.0f;
    float hi = mx[i] > 0.0f ? mx[i] : 0.0f;
    if (symmetric) {
      float a = fabsf(lo), b = fabsf(hi);
      float m = a > b ? a : b;
      float half = (float)((double)(qmax - qmin) / 2.0);
      float s = m / half;
      scale[i] = s > eps ? s : eps;
      zp[i] = is_signed ? 0.0f : (float)((qmax + qmin + 1) / 2);
    } else {
      float s = (hi - lo) / (float)(qmax - qmin);
      s = s > eps ? s : eps;
      scale[i] = s;
      float t = rintf(lo / s);
      t = (float)qmin - t;
      zp[i] = clipf(t, (float)qmin, (float)qmax);
    }
  }
}

/* Exact integer contraction acc[m,n] = sum_k a[m,k] * w[n,k]; a is signed or
 * unsigned 8-bit, w signed 8-bit, both K-contiguous. */
void lo_gemm_i8_i32(const void* a, int a_signed, const int8_t* w, size_t M, size_t N, size_t K,
                    int32_t* acc) {
  const int8_t* as = (const int8_t*)a;
  const uint8_t* au = (const uint8_t*)a;
  for (size_t m = 0; m < M; ++m)
    for (size_t n = 0; n < N; ++n) {
      int32_t s = 0;
      for (size_t k = 0; k < K; ++k) {
        int32_t av = a_signed ? (int32_t)as[m * K + k] : (int32_t)au[m * K + k];
        s += av * (int32_t)w[n * K + k];
      }
      acc[m * N + n] = s;
    }
}
