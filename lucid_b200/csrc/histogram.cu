// Equal-width histogram of a float stream: the device form of the reference's histc
// (lucid/_C/ops/composite/Stats.cpp:47-91 over the counting loop of
// lucid/_C/backend/cpu/CpuBackend.h:13276-13318), fused with what its histogram observer does
// around it (lucid/quantization/observer.py:786-838): the min / max of the same batch and the
// fold of the previous histogram, re-binned when the range widened.
//
// One pass over HBM.  Every CTA counts into a shared-memory histogram with shared atomics, adds
// its non-empty bins to 64-bit counters in the workspace, and the CTA that takes the last ticket
// converts the counters, folds the previous histogram and re-arms the workspace.
//
// Bin index, bit for bit the reference's  trunc((double(v) - lo) / ((hi - lo) / bins)):
// the quotient is first approximated by a multiplication with the rounded reciprocal of the
// step (relative error < 2^-51); adding 2^33 with round-toward-zero leaves trunc(q * 2^19) in
// the low mantissa word, so the bin is its top 13 bits and the low 19 bits are the fraction.  A
// fraction of all zeros or all ones is the only case in which the approximation can sit on the
// other side of a bin edge from the true quotient; those elements take the IEEE division.
#include <math.h>

#include "common.cuh"

namespace lq {
namespace {

constexpr int kHistThreads = 256;
constexpr int kHistCtasPerSm = 4;
constexpr int kHistMaxCtas = kNumSMs * kHistCtasPerSm;
constexpr int kHistMaxBins = 4096;
constexpr int kFracBits = 19;
constexpr unsigned int kFracMask = (1u << kFracBits) - 1u;

struct HistWorkspace {
  unsigned int ticket;
  unsigned int pad[3];
  float pmin[kHistMaxCtas];
  float pmax[kHistMaxCtas];
  unsigned long long counts[kHistMaxBins];
};

enum PrevMode : int { kPrevNone = 0, kPrevAdd = 1, kPrevRebin = 2 };

struct HistArgs {
  double lo, step, rstep;  // rstep == 0 sends every element through the division
  float flo, fhi;          // v in [lo, hi]  <=>  flo <= v <= fhi  for every float v
  int bins;
  int prev_mode;
  const float* prev;
  float old_min, old_width, new_min, new_width;  // re-binning, in binary32 as the reference
  float* out;
  float* out_min;
  float* out_max;
};

__device__ __noinline__ unsigned int bin_by_division(double d, double step, unsigned int last) {
  const double q = __ddiv_rn(d, step);
  return q >= (double)last ? last : (unsigned int)(long long)q;
}

struct Counter {
  unsigned int* sh;
  double lo, step, rstep;
  float flo, fhi;
  unsigned int last;
  float mn, mx;

  __device__ __forceinline__ void add(float v) {
    mn = fminf(mn, v), mx = fmaxf(mx, v);
    if (v >= flo && v <= fhi) {  // false for NaN
      const double d = __dsub_rn((double)v, lo);
      unsigned int b;
      if (d == 0.0) {
        b = 0u;  // the batch minimum, or the zeros of a rectified tensor: no arithmetic needed
      } else {
        const double q = __dmul_rn(d, rstep);
        const unsigned int w = (unsigned int)__double2loint(__dadd_rz(q, 0x1p33));
        const unsigned int fr = w & kFracMask;
        b = w >> kFracBits;
        if (fr == 0u || fr == kFracMask) b = bin_by_division(d, step, last);
      }
      atomicAdd(sh + (b < last ? b : last), 1u);
    }
  }
};

template <typename In>
__device__ __forceinline__ void count_vec(uint4 u, Counter& c);
template <>
__device__ __forceinline__ void count_vec<float>(uint4 u, Counter& c) {
  c.add(__uint_as_float(u.x)), c.add(__uint_as_float(u.y));
  c.add(__uint_as_float(u.z)), c.add(__uint_as_float(u.w));
}
template <>
__device__ __forceinline__ void count_vec<__nv_bfloat16>(uint4 u, Counter& c) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) c.add(bf16_bits_to_f32(w[j] & 0xffffu)), c.add(bf16_bits_to_f32(w[j] >> 16));
}
template <typename In>
__device__ __forceinline__ float load1(const In* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) {
  return bf16_bits_to_f32(*reinterpret_cast<const unsigned short*>(p));
}

__device__ __forceinline__ void block_minmax_h(float& mn, float& mx) {
  __shared__ float smn[kHistThreads / 32], smx[kHistThreads / 32];
  mn = warp_min(mn), mx = warp_max(mx);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) smn[w] = mn, smx[w] = mx;
  __syncthreads();
  if (w == 0) {
    mn = l < kHistThreads / 32 ? smn[l] : INFINITY;
    mx = l < kHistThreads / 32 ? smx[l] : -INFINITY;
    mn = warp_min(mn), mx = warp_max(mx);
  }
  __syncthreads();
}

// Fold of the previous histogram by the last CTA.  `smem` holds 3 * bins words.
__device__ void finish_histogram(const HistArgs& a, HistWorkspace* ws, unsigned int* smem) {
  const int bins = a.bins;
  float* s_prev = reinterpret_cast<float*>(smem);
  int* s_dst = reinterpret_cast<int*>(smem) + bins;
  float* s_acc = reinterpret_cast<float*>(smem) + 2 * bins;
  // The previous histogram may be the output buffer: read all of it first.
  if (a.prev_mode != kPrevNone)
    for (int j = threadIdx.x; j < bins; j += kHistThreads) s_prev[j] = a.prev[j];
  __syncthreads();
  for (int j = threadIdx.x; j < bins; j += kHistThreads) {
    const unsigned long long c = __ldcg(&ws->counts[j]);
    ws->counts[j] = 0ull;  // leave the workspace zeroed for the next call
    float h = __ull2float_rn(c);  // the reference counts in binary64, then casts to binary32
    if (a.prev_mode == kPrevAdd) h = __fadd_rn(h, s_prev[j]);
    a.out[j] = h;
  }
  if (a.prev_mode != kPrevRebin) return;

  // Destination bin of every old bin centre (observer.py:800-815), all in binary32.
  const float top = (float)(bins - 1);
  for (int j = threadIdx.x; j < bins; j += kHistThreads) {
    const float centre = __fadd_rn(a.old_min, __fmul_rn(__fadd_rn((float)j, 0.5f), a.old_width));
    float raw = __fdiv_rn(__fsub_rn(centre, a.new_min), a.new_width);
    raw = raw < 0.0f ? 0.0f : (raw > top ? top : raw);
    s_dst[j] = raw == raw ? (int)raw : 0;
    s_acc[j] = 0.0f;
  }
  __syncthreads();
  // The scatter adds old bins in index order.  Destinations never decrease with the index, so
  // each output bin receives one contiguous run: the thread at the head of a run sums it in
  // order.  (If an inconsistent range ever broke the ordering, one thread replays the scatter.)
  int disorder = 0;
  for (int j = threadIdx.x + 1; j < bins; j += kHistThreads) disorder |= s_dst[j] < s_dst[j - 1];
  if (__syncthreads_or(disorder)) {
    if (threadIdx.x == 0)
      for (int j = 0; j < bins; ++j) s_acc[s_dst[j]] = __fadd_rn(s_acc[s_dst[j]], s_prev[j]);
  } else {
    for (int j = threadIdx.x; j < bins; j += kHistThreads) {
      if (j != 0 && s_dst[j - 1] == s_dst[j]) continue;
      const int d = s_dst[j];
      float acc = 0.0f;
      for (int k = j; k < bins && s_dst[k] == d; ++k) acc = __fadd_rn(acc, s_prev[k]);
      s_acc[d] = acc;
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < bins; j += kHistThreads) a.out[j] = __fadd_rn(a.out[j], s_acc[j]);
}

template <typename In>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
histc_kernel(const In* __restrict__ x, size_t n, bool vec_ok, HistArgs a, HistWorkspace* ws) {
  extern __shared__ __align__(16) unsigned int smem[];
  for (int j = threadIdx.x; j < a.bins; j += kHistThreads) smem[j] = 0u;
  __syncthreads();

  Counter c{smem, a.lo, a.step, a.rstep, a.flo, a.fhi, (unsigned int)(a.bins - 1), INFINITY, -INFINITY};
  constexpr int E = 16 / sizeof(In);
  const size_t nvec = vec_ok ? n / E : 0;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const size_t first = (size_t)blockIdx.x * kHistThreads + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * kHistThreads;
  size_t i = first;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 v0 = ld_stream_u4(xv + i), v1 = ld_stream_u4(xv + i + stride);
    const uint4 v2 = ld_stream_u4(xv + i + 2 * stride), v3 = ld_stream_u4(xv + i + 3 * stride);
    count_vec<In>(v0, c), count_vec<In>(v1, c), count_vec<In>(v2, c), count_vec<In>(v3, c);
  }
  for (; i < nvec; i += stride) count_vec<In>(ld_stream_u4(xv + i), c);
  for (size_t e = nvec * E + first; e < n; e += stride) c.add(load1<In>(x + e));

  float mn = c.mn, mx = c.mx;
  block_minmax_h(mn, mx);  // also orders the shared atomics before the flush
  for (int j = threadIdx.x; j < a.bins; j += kHistThreads) {
    const unsigned int v = smem[j];
    if (v) atomicAdd(&ws->counts[j], (unsigned long long)v);
  }
  __shared__ bool is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    ws->pmin[blockIdx.x] = mn;
    ws->pmax[blockIdx.x] = mx;
    __threadfence();
    is_last = atomicAdd(&ws->ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  mn = INFINITY, mx = -INFINITY;
  for (unsigned int k = threadIdx.x; k < gridDim.x; k += kHistThreads) {
    mn = fminf(mn, __ldcg(&ws->pmin[k]));
    mx = fmaxf(mx, __ldcg(&ws->pmax[k]));
  }
  block_minmax_h(mn, mx);
  if (threadIdx.x == 0) {
    if (a.out_min) *a.out_min = mn;
    if (a.out_max) *a.out_max = mx;
    ws->ticket = 0;
  }
  finish_histogram(a, ws, smem);
}

// Largest float <= d and smallest float >= d.
float float_at_most(double d) {
  float f = (float)d;
  return (double)f > d ? nextafterf(f, -INFINITY) : f;
}
float float_at_least(double d) {
  float f = (float)d;
  return (double)f < d ? nextafterf(f, INFINITY) : f;
}

}  // namespace
}  // namespace lq

using namespace lq;

extern "C" size_t lq_histc_workspace_bytes(void) { return sizeof(HistWorkspace); }
extern "C" int lq_histc_max_bins(void) { return kHistMaxBins; }

extern "C" int lq_histc(const void* x, int in_dtype, size_t n, double lo, double hi, int bins,
                        const float* prev_hist, double prev_lo, double prev_hi, float* hist_out,
                        float* out_min, float* out_max, void* workspace, size_t workspace_bytes,
                        void* stream) {
  if (!x || !hist_out) return fail(LQ_ERR_DEVICE, "lq_histc: null pointer");
  if (n == 0) return fail(LQ_ERR_SHAPE, "lq_histc: empty input");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_histc: in_dtype");
  if (bins < 1 || bins > kHistMaxBins)
    return fail(LQ_ERR_UNSUPPORTED, "lq_histc: bins must be in [1, " + std::to_string(kHistMaxBins) + "]");
  if (!(hi > lo) || !isfinite(lo) || !isfinite(hi))
    return fail(LQ_ERR_SHAPE, "lq_histc: the range must be finite with lo < hi (the caller derives an empty "
                              "range from the data, as the reference's histc does)");
  if (!workspace) return fail(LQ_ERR_DEVICE, "lq_histc: workspace");
  if (workspace_bytes < sizeof(HistWorkspace))
    return fail(LQ_ERR_WORKSPACE, "lq_histc: workspace smaller than lq_histc_workspace_bytes()");
  if (!aligned16(workspace)) return fail(LQ_ERR_ALIGNMENT, "lq_histc: workspace alignment");

  HistArgs a{};
  a.lo = lo;
  a.step = (hi - lo) / (double)bins;
  if (!(a.step > 0.0) || !isfinite(a.step))
    return fail(LQ_ERR_SHAPE, "lq_histc: (hi - lo) / bins is not a positive finite number");
  a.rstep = (a.step > 0x1p-900 && a.step < 0x1p900) ? 1.0 / a.step : 0.0;
  a.flo = float_at_least(lo);
  a.fhi = float_at_most(hi);
  a.bins = bins;
  a.prev = prev_hist;
  a.out = hist_out;
  a.out_min = out_min;
  a.out_max = out_max;
  if (!prev_hist) {
    a.prev_mode = kPrevNone;
  } else if (prev_lo == lo && prev_hi == hi) {
    a.prev_mode = kPrevAdd;
  } else {
    a.prev_mode = kPrevRebin;
    a.old_min = (float)prev_lo;
    a.old_width = (float)((prev_hi - prev_lo) / (double)bins);
    a.new_min = (float)lo;
    a.new_width = (float)a.step;
  }

  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  const bool vec_ok = aligned16(x);
  // four 16-byte vectors per thread and iteration; grid capped at the resident CTA count
  const size_t per_cta = (size_t)kHistThreads * 4 * (16 / esz);
  size_t want = (n + per_cta - 1) / per_cta;
  const int grid = (int)(want < 1 ? 1 : (want > (size_t)kHistMaxCtas ? (size_t)kHistMaxCtas : want));
  const size_t smem = (size_t)bins * 3 * sizeof(unsigned int);
  if (smem > 40 * 1024) {  // static shared memory included, this passes the 48 KB default
    LQ_CUDA(cudaFuncSetAttribute(histc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LQ_CUDA(cudaFuncSetAttribute(histc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  cudaStream_t st = (cudaStream_t)stream;
  auto* ws = (HistWorkspace*)workspace;
  if (in_dtype == LQ_F32)
    histc_kernel<float><<<grid, kHistThreads, smem, st>>>((const float*)x, n, vec_ok, a, ws);
  else
    histc_kernel<__nv_bfloat16><<<grid, kHistThreads, smem, st>>>((const __nv_bfloat16*)x, n, vec_ok, a, ws);
  return check_cuda(cudaGetLastError(), "lq_histc launch");
}
