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
// Bin index, bit for bit the reference's  trunc((double(v) - lo) / ((hi - lo) / bins)), in three
// tiers.  Binary64 arithmetic at one element per lane would cap the kernel near 60 % of the HBM
// rate, so the common case stays in binary32:
//   1. q = RN32(RN32(v - lo) * RN32(1 / step)) is within 3.01 * 2^-24 * bins of the true quotient.
//      Adding M = 2^k + one unit in the last place (2^k >= 2 * bins) with round-toward-zero leaves
//      u = trunc(q * 2^f) + 1, f = 23 - k, in the mantissa: the bin and f fraction bits, and 2^-f
//      exceeds the error bound.  If u <= bins * 2^f and the fraction of u is neither 0 nor 1 (or
//      u == 1: a quotient in [0, 2^-f) is in bin 0 whatever its error) the element is inside the
//      range and its bin is u >> f, for certain: seven integer / float instructions with no
//      branch, which also reject NaN, infinities and everything outside [lo, hi].  The factor and
//      M carry a common power of two that brings the factor into [1, 2), so the product never
//      underflows to zero and a value just below lo keeps its sign.  (Needs lo representable in
//      binary32 -- an observed minimum always is -- and a step far from the exponent limits.)
//   2. Otherwise the same test in binary64 with the rounded reciprocal (error < 2^-39 bins,
//      19 fraction bits).
//   3. Otherwise the IEEE division itself.
#include <math.h>
#include <stdlib.h>
#include <string.h>

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
  // tier 1 (see the head of the file): scaled factor, scaled M, bits of the scaled 2^k,
  // bins << f, f, and the fraction mask without its lowest bit
  float rstep32, magic32;
  unsigned int magic_bits, limit32, frac_bits32, frac_hi32;
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

// Tiers 2 and 3, for the elements tier 1 cannot place.  d = double(v) - lo >= 0.
// Low-precision data (bfloat16 activations, quantized grids) puts many elements exactly on bin
// edges, so the edge case must stay cheap: with n the integer the approximate quotient sits
// next to, t = fma(-n, step, d) has the sign of d - n * step exactly; t >= 0 proves the rounded
// quotient is at least n (rounding is monotonic and n is representable), and it is below n + 1.
// Only an element within 2^-39 bins BELOW an edge is left to the IEEE division.
__device__ __forceinline__ unsigned int bin_in_binary64(double d, double step, double rstep, unsigned int last) {
  const double q = __dmul_rn(d, rstep);
  const unsigned int w = (unsigned int)__double2loint(__dadd_rz(q, 0x1p33));
  const unsigned int fr = w & kFracMask;
  unsigned int b = w >> kFracBits;
  if (fr == 0u || fr == kFracMask) {
    const unsigned int n = fr == 0u ? b : b + 1u;
    if (rstep != 0.0 && __fma_rn(-(double)n, step, d) >= 0.0)
      b = n;
    else
      b = bin_by_division(d, step, last);
  }
  return b < last ? b : last;
}

__device__ __forceinline__ float min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

struct Binner {
  unsigned int* sh;
  double lo, step, rstep;
  float flo, fhi, rstep32, magic32;
  unsigned int magic_bits, limit, frac_bits, frac_hi;
  unsigned int last;

  // Tier 1: true when the element is certainly inside the range; `bin` is then its bin.
  __device__ __forceinline__ bool certain(float v, unsigned int& bin) const {
    const float s = __fadd_rz(__fmul_rn(__fsub_rn(v, flo), rstep32), magic32);
    const unsigned int u = __float_as_uint(s) - magic_bits;
    bin = u >> frac_bits;
    return u <= limit && ((u & frac_hi) != 0u || u == 1u);
  }
  // The same test as straight-line code for the counting loop: returns the word to count into
  // (the bin, or the spare word) and sets `bit` in `open` when the element is not certain.
  __device__ __forceinline__ unsigned int classify(float v, unsigned int& open, unsigned int bit) const {
    const float s = __fadd_rz(__fmul_rn(__fsub_rn(v, flo), rstep32), magic32);
    unsigned int idx;
    asm("{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b32 u, t;\n\t"
        "sub.u32 u, %2, %3;\n\t"
        "and.b32 t, u, %4;\n\t"
        "setp.ne.u32 p, t, 0;\n\t"
        "setp.eq.or.u32 p, u, 1, p;\n\t"
        "setp.le.and.u32 p, u, %5, p;\n\t"
        "shr.u32 t, u, %6;\n\t"
        "selp.u32 %0, t, %7, p;\n\t"
        "@!p or.b32 %1, %1, %8;\n\t"
        "}"
        : "=r"(idx), "+r"(open)
        : "r"(__float_as_uint(s)), "r"(magic_bits), "r"(frac_hi), "r"(limit), "r"(frac_bits), "r"(last + 1u),
          "r"(bit));
    return idx;
  }
  // Tiers 2 and 3 for an element tier 1 left open (or every element when tier 1 is off).
  __device__ __forceinline__ void place(float v) const {
    if (v >= flo && v <= fhi)  // false for NaN
      atomicAdd(sh + bin_in_binary64(__dsub_rn((double)v, lo), step, rstep, last), 1u);
  }
};

// Sixteen elements (four 16-byte vectors of binary32, or two of bfloat16) at a time: classify
// and count without a branch, then revisit the group only if some element was left open.
template <bool TIER1>
__device__ __forceinline__ void count16(const float (&e)[16], const Binner& b, float& mn, float& mx) {
#pragma unroll
  for (int j = 0; j < 16; j += 2) mn = min3(mn, e[j], e[j + 1]), mx = max3(mx, e[j], e[j + 1]);
  if (TIER1) {
    // An element that is not certain counts into a spare word after the last bin instead: one
    // unconditional shared atomic per element, no branch around it.
    unsigned int open = 0u;
#pragma unroll
    for (int j = 0; j < 16; ++j) atomicAdd(b.sh + b.classify(e[j], open, 1u << j), 1u);
    if (open) {
      // each lane walks its own open elements; the copy lets it index them
      float again[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) again[j] = e[j];
      do {
        const int j = __ffs(open) - 1;
        open &= open - 1u;
        b.place(again[j]);
      } while (open);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) b.place(e[j]);
  }
}
template <bool TIER1>
__device__ __forceinline__ void count1(float v, const Binner& b, float& mn, float& mx) {
  mn = fminf(mn, v), mx = fmaxf(mx, v);
  unsigned int bin;
  if (TIER1 && b.certain(v, bin))
    atomicAdd(b.sh + bin, 1u);
  else
    b.place(v);
}

template <typename In>
struct Unpack;
template <>
struct Unpack<float> {
  static constexpr int kVecs = 4;  // vectors per group of sixteen
  static __device__ __forceinline__ void run(const uint4 (&u)[4], float (&e)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      e[4 * j] = __uint_as_float(u[j].x), e[4 * j + 1] = __uint_as_float(u[j].y);
      e[4 * j + 2] = __uint_as_float(u[j].z), e[4 * j + 3] = __uint_as_float(u[j].w);
    }
  }
};
template <>
struct Unpack<__nv_bfloat16> {
  static constexpr int kVecs = 2;
  static __device__ __forceinline__ void run(const uint4 (&u)[2], float (&e)[16]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t w[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        e[8 * j + 2 * i] = __uint_as_float(w[i] << 16);
        e[8 * j + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  }
};

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

// Fold of the previous histogram by the last CTA.  `smem` holds 3 * bins words (during the
// counting phase: the bins, then the spare word of the branch-free counting).
__device__ void finish_histogram(const HistArgs& a, HistWorkspace* ws, unsigned int* smem) {
  const int bins = a.bins;
  float* s_prev = reinterpret_cast<float*>(smem);
  int* s_dst = reinterpret_cast<int*>(smem) + bins;
  float* s_acc = reinterpret_cast<float*>(smem) + 2 * bins;
  // All loads first (they are independent L2 round trips; interleaved with the stores they
  // would run one after another).  The previous histogram may be the output buffer.
  constexpr int kPer = kHistMaxBins / kHistThreads;
  unsigned long long cnt[kPer];
  float prv[kPer];
#pragma unroll
  for (int t = 0; t < kPer; ++t) {
    const int j = threadIdx.x + t * kHistThreads;
    cnt[t] = j < bins ? __ldcg(&ws->counts[j]) : 0ull;
    prv[t] = (j < bins && a.prev_mode != kPrevNone) ? __ldcg(a.prev + j) : 0.0f;
  }
#pragma unroll
  for (int t = 0; t < kPer; ++t) {
    const int j = threadIdx.x + t * kHistThreads;
    if (j < bins) {
      ws->counts[j] = 0ull;  // leave the workspace zeroed for the next call
      s_prev[j] = prv[t];
    }
  }
  __syncthreads();  // every thread has read its part of prev before anyone writes out
#pragma unroll
  for (int t = 0; t < kPer; ++t) {
    const int j = threadIdx.x + t * kHistThreads;
    if (j < bins) {
      float h = __ull2float_rn(cnt[t]);  // the reference counts in binary64, then casts to binary32
      if (a.prev_mode == kPrevAdd) h = __fadd_rn(h, prv[t]);
      a.out[j] = h;
    }
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

template <typename In, bool TIER1>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
histc_kernel(const In* __restrict__ x, size_t n, bool vec_ok, HistArgs a, HistWorkspace* ws) {
  extern __shared__ __align__(16) unsigned int smem[];
  for (int j = threadIdx.x; j < a.bins; j += kHistThreads) smem[j] = 0u;
  __syncthreads();

  const Binner b{smem, a.lo, a.step, a.rstep, a.flo, a.fhi, a.rstep32, a.magic32, a.magic_bits, a.limit32,
                 a.frac_bits32, a.frac_hi32, (unsigned int)(a.bins - 1)};
  float mn = INFINITY, mx = -INFINITY;
  constexpr int E = 16 / sizeof(In);
  constexpr int V = Unpack<In>::kVecs;
  const size_t nvec = vec_ok ? n / E : 0;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const size_t first = (size_t)blockIdx.x * kHistThreads + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * kHistThreads;
  size_t i = first;
  // Groups of sixteen elements, software-pipelined: the loads of the next group are issued
  // before the current group is counted, so a warp always has a group's loads in flight.
  if (i + (V - 1) * stride < nvec) {
    uint4 cur[V];
#pragma unroll
    for (int j = 0; j < V; ++j) cur[j] = ld_stream_u4(xv + i + j * stride);
    i += V * stride;
    for (; i + (V - 1) * stride < nvec; i += V * stride) {
      uint4 nxt[V];
#pragma unroll
      for (int j = 0; j < V; ++j) nxt[j] = ld_stream_u4(xv + i + j * stride);
      float e[16];
      Unpack<In>::run(cur, e);
      count16<TIER1>(e, b, mn, mx);
#pragma unroll
      for (int j = 0; j < V; ++j) cur[j] = nxt[j];
    }
    float e[16];
    Unpack<In>::run(cur, e);
    count16<TIER1>(e, b, mn, mx);
  }
  for (; i < nvec; i += stride) {
    const In* p = x + i * E;
#pragma unroll
    for (int j = 0; j < E; ++j) count1<TIER1>(load1<In>(p + j), b, mn, mx);
  }
  for (size_t e1 = nvec * E + first; e1 < n; e1 += stride) count1<TIER1>(load1<In>(x + e1), b, mn, mx);

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
  // tier 1 needs lo in binary32 and 1 / step, hi - lo well inside its exponent range
  // 2^k >= 2 * bins: the fraction's resolution 2^(k-23) then exceeds the error bound
  int k = 1;
  while ((1 << k) < 2 * bins) ++k;
  const bool tier1 = (double)a.flo == lo && a.step > 0x1p-100 && a.step < 0x1p100 && (hi - lo) < 0x1p100 &&
                     !getenv("LQ_HIST_BINARY64");
  if (tier1) {
    const float r = (float)(1.0 / a.step);
    int ex;
    frexpf(r, &ex);               // r = m * 2^ex, m in [0.5, 1)
    const int sc = 1 - ex;        // r * 2^sc in [1, 2)
    a.rstep32 = ldexpf(r, sc);
    const float pow2k = ldexpf(1.0f, k + sc);
    a.magic32 = nextafterf(pow2k, INFINITY);
    memcpy(&a.magic_bits, &pow2k, sizeof(float));
    a.frac_bits32 = (unsigned int)(23 - k);
    a.limit32 = (unsigned int)bins << a.frac_bits32;
    a.frac_hi32 = ((1u << a.frac_bits32) - 1u) & ~1u;
  }
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
  auto launch = [&](auto kernel, auto ptr) -> int {
    if (smem > 40 * 1024)  // static shared memory included, this passes the 48 KB default
      LQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kHistThreads, smem, (cudaStream_t)stream>>>(ptr, n, vec_ok, a, (HistWorkspace*)workspace);
    return LQ_OK;
  };
  int rc;
  if (in_dtype == LQ_F32)
    rc = tier1 ? launch(histc_kernel<float, true>, (const float*)x) : launch(histc_kernel<float, false>, (const float*)x);
  else
    rc = tier1 ? launch(histc_kernel<__nv_bfloat16, true>, (const __nv_bfloat16*)x)
               : launch(histc_kernel<__nv_bfloat16, false>, (const __nv_bfloat16*)x);
  if (rc != LQ_OK) return rc;
  return check_cuda(cudaGetLastError(), "lq_histc launch");
}
