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
#include <stdlib.h>

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

/* ---- histogram observer ----------------------------------------------------------------
 * histc: lucid/_C/ops/composite/Stats.cpp:47-91 over the counting loop of
 * lucid/_C/backend/cpu/CpuBackend.h:13276-13318 (binary64 arithmetic, values outside
 * [lo, hi] skipped, truncation, the top edge folded into the last bin; an empty range is taken
 * from the data, a constant tensor gets [v, v + 1]).  Counts leave as binary32, as the reference
 * casts them to the input dtype.  NaN elements are skipped. */
void lo_histc_f32(const float* x, size_t n, int bins, double lo, double hi, float* out) {
  if (lo == hi && n > 0) {
    double mn = x[0], mx = x[0];
    for (size_t i = 1; i < n; ++i) {
      if (x[i] < mn) mn = x[i];
      if (x[i] > mx) mx = x[i];
    }
    lo = mn, hi = mx;
    if (lo == hi) hi = lo + 1.0;
  }
  const double step = (hi - lo) / (double)bins;
  double* counts = (double*)calloc((size_t)bins, sizeof(double));
  for (size_t i = 0; i < n; ++i) {
    const double v = (double)x[i];
    if (v != v || v < lo || v > hi) continue;
    long long b = (long long)((v - lo) / step);
    if (b >= bins) b = bins - 1;
    counts[b] += 1.0;
  }
  for (int b = 0; b < bins; ++b) out[b] = (float)counts[b];
  free(counts);
}

/* HistogramObserver._rebin, lucid/quantization/observer.py:786-817: binary32 centres of the old
 * bins, their destination on the new grid (clipped, truncated), scatter-add in index order. */
void lo_hist_rebin_f32(const float* hist, int bins, double old_min, double old_max, double new_min,
                       double new_max, float* out) {
  const float old_width = (float)((old_max - old_min) / bins);
  const float new_width = (float)((new_max - new_min) / bins);
  const float omin = (float)old_min, nmin = (float)new_min, top = (float)(bins - 1);
  for (int b = 0; b < bins; ++b) out[b] = 0.0f;
  for (int i = 0; i < bins; ++i) {
    volatile float t = (float)i + 0.5f;
    volatile float u = t * old_width;
    volatile float centre = omin + u;
    volatile float num = centre - nmin;
    float raw = num / new_width;
    raw = raw < 0.0f ? 0.0f : (raw > top ? top : raw);
    const int dst = raw == raw ? (int)raw : 0;
    volatile float acc = out[dst] + hist[i];
    out[dst] = acc;
  }
}

/* QFunctional.add / mul / add_relu, lucid/nn/quantized/functional_module.py:230-246: the
 * binary32 merge, then fake_quantize (op 0 add, 1 mul, 2 relu(add)). */
void lo_qfunctional_f32(int op, const float* x, const float* y, size_t n, float scale, float zp, int qmin,
                        int qmax, float* out) {
  for (size_t i = 0; i < n; ++i) {
    volatile float t = op == 1 ? x[i] * y[i] : x[i] + y[i];
    if (op == 2 && !(t > 0.0f)) t = 0.0f;
    const float c = code_of(t, scale, zp, (float)qmin, (float)qmax);
    volatile float d = c - zp;
    out[i] = d * scale;
  }
}

/* ---- group-wise weight-only codes --------------------------------------------------------
 * Formulas the reference documents for its MLX route (lucid/quantization/_qgemm.py:84-97):
 * per group of `group` consecutive input positions, scale = (max - min) / (2^bits - 1),
 * bias = min, code = clip(rint((w - bias) / scale), 0, 2^bits - 1), codes packed
 * little-endian into 32-bit words; a constant group takes scale 1.  The engine that implements
 * them (MLX) is absent here: parity unpinned, like the NumPy form. */
void lo_groupwise_quantize(const float* w, size_t n, size_t k, int group, int bits, uint32_t* packed,
                           float* scales, float* biases) {
  const float top = (float)((1 << bits) - 1);
  const size_t per = (size_t)(32 / bits), groups = k / (size_t)group;
  for (size_t r = 0; r < n; ++r) {
    for (size_t g = 0; g < groups; ++g) {
      const float* wg = w + r * k + g * (size_t)group;
      float mn = wg[0], mx = wg[0];
      for (int i = 1; i < group; ++i) {
        mn = wg[i] < mn ? wg[i] : mn;
        mx = wg[i] > mx ? wg[i] : mx;
      }
      float s = (mx - mn) / top;
      if (!(s > 0.0f)) s = 1.0f;
      scales[r * groups + g] = s;
      biases[r * groups + g] = mn;
      for (int i = 0; i < group; ++i) {
        const size_t e = g * (size_t)group + (size_t)i;
        const float q = clipf(rintf((wg[i] - mn) / s), 0.0f, top);
        uint32_t* word = packed + r * (k / per) + e / per;
        if (e % per == 0) *word = 0u;
        *word |= (uint32_t)q << ((e % per) * (size_t)bits);
      }
    }
  }
}

void lo_groupwise_dequantize(const uint32_t* packed, const float* scales, const float* biases, size_t n, size_t k,
                             int group, int bits, float* out) {
  const size_t per = (size_t)(32 / bits), groups = k / (size_t)group;
  const uint32_t mask = (1u << bits) - 1u;
  for (size_t r = 0; r < n; ++r)
    for (size_t e = 0; e < k; ++e) {
      const uint32_t code = (packed[r * (k / per) + e / per] >> ((e % per) * (size_t)bits)) & mask;
      const size_t g = r * groups + e / (size_t)group;
      const float prod = (float)code * scales[g]; /* two roundings: product, then sum */
      out[r * k + e] = prod + biases[g];
    }
}

/* ---- the integer form of a quantized Linear, end to end --------------------------------
 * Per-token symmetric activation encode (the reference's primitives composed:
 * PerChannelMinMaxObserver(ch_axis=0) -> calculate_qparams -> quantize(ch_axis=0),
 * lucid/quantization/observer.py:635-648, _qparams.py:197-215, _functional.py:175-182),
 * exact int32 accumulation, then the epilogue in the kernels' operation order:
 *   y = f32(acc) * (a_scale[m] * w_scale[n]); y += bias[n]; optional ReLU;
 * then either the bfloat16 rounding of y (out_bf16, nearest even, lucid/_C/core/Half.h:37-48)
 * or its requantisation clip(rint(y / out_scale) + out_zp, qmin, qmax). */
void lo_per_token_quantize_f32_s8(const float* x, size_t rows, size_t cols, float eps, int8_t* q, float* scale) {
  for (size_t r = 0; r < rows; ++r) {
    float mn = 0.0f, mx = 0.0f; /* the range always contains 0 */
    for (size_t c = 0; c < cols; ++c) {
      const float v = x[r * cols + c];
      mn = v < mn ? v : mn;
      mx = v > mx ? v : mx;
    }
    const float a = fabsf(mn), b = fabsf(mx);
    float s = (a > b ? a : b) / 127.5f; /* (qmax - qmin) / 2 for the signed 8-bit grid */
    s = s > eps ? s : eps;
    scale[r] = s;
    for (size_t c = 0; c < cols; ++c) q[r * cols + c] = (int8_t)clipf(rintf(x[r * cols + c] / s), -128.0f, 127.0f);
  }
}

static inline float bf16_round_f32(float v) {
  union { float f; uint32_t u; } w;
  w.f = v;
  w.u = (uint32_t)((((uint64_t)w.u + 0x7FFFu + ((w.u >> 16) & 1u)) >> 16) << 16);
  return w.f;
}

void lo_linear_epilogue_f32(const int32_t* acc, size_t M, size_t N, const float* a_scale, const float* w_scale,
                            const float* bias, int relu, int out_bf16, float* y) {
  for (size_t m = 0; m < M; ++m)
    for (size_t n = 0; n < N; ++n) {
      const float sc = a_scale[m] * w_scale[n];
      float v = (float)acc[m * N + n] * sc;
      if (bias) v = v + bias[n];
      if (relu) v = v > 0.0f ? v : 0.0f;
      y[m * N + n] = out_bf16 ? bf16_round_f32(v) : v;
    }
}

void lo_requantize_f32(const float* y, size_t n, float out_scale, float out_zp, int qmin, int qmax, float* codes) {
  for (size_t i = 0; i < n; ++i) codes[i] = clipf(rintf(y[i] / out_scale) + out_zp, (float)qmin, (float)qmax);
}
