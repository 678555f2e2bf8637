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

// What the first kernel of an observer step leaves for the second (see observe_pass1).
struct ObserveState {
  int pass2;  // 1: the batch must be binned again, on [new_lo, new_hi]
  int mode;   // PrevMode of that second pass
  double new_lo, new_hi, old_lo, old_hi;
};

struct HistWorkspace {
  unsigned int ticket;
  unsigned int pad[3];
  float pmin[kHistMaxCtas];
  float pmax[kHistMaxCtas];
  unsigned long long counts[kHistMaxBins];
  ObserveState observe;
};

enum PrevMode : int { kPrevNone = 0, kPrevAdd = 1, kPrevRebin = 2 };

struct HistArgs {
  double lo, step, rstep;  // rstep == 0 sends every element through the division
  float flo, fhi;          // v in [lo, hi]  <=>  flo <= v <= fhi  for every float v
  // tier 1 (see the head of the file): scaled factor, scaled M, bits of the scaled 2^k,
  // bins << f, f, and the fraction mask without its lowest bit
  float rstep32, magic32;
  unsigned int magic_bits, limit32, frac_bits32, frac_hi32;
  int tier1;
  float step32;  // the step, when binary32 holds it exactly (else 0): enables the binary32 tie-break
  int bins;
  int prev_mode;
  const float* prev;
  float old_min, old_width, new_min, new_width;  // re-binning, in binary32 as the reference
  float* out;
  float* out_min;
  float* out_max;
};

// Largest float <= d and smallest float >= d.
__host__ __device__ inline float float_at_most(double d) {
  const float f = (float)d;
  return (double)f > d ? nextafterf(f, -INFINITY) : f;
}
__host__ __device__ inline float float_at_least(double d) {
  const float f = (float)d;
  return (double)f < d ? nextafterf(f, INFINITY) : f;
}

// Everything the counting loop needs for the finite range lo < hi.  False when the step is
// not a positive finite number.  Runs on the host (lq_histc) and on the device (the observer
// kernels read their range from device memory).
__host__ __device__ inline bool derive_binning(double lo, double hi, int bins, bool allow_tier1, HistArgs& a) {
  a.bins = bins;
  a.lo = lo;
  a.step = (hi - lo) / (double)bins;
  if (!(a.step > 0.0) || !(a.step < INFINITY)) return false;
  a.rstep = (a.step > 0x1p-900 && a.step < 0x1p900) ? 1.0 / a.step : 0.0;
  a.flo = float_at_least(lo);
  a.fhi = float_at_most(hi);
  // 2^k >= 2 * bins: the fraction's resolution 2^(k-23) then exceeds the error bound
  int k = 1;
  while ((1 << k) < 2 * bins) ++k;
  // tier 1 needs lo in binary32 and 1 / step, hi - lo well inside its exponent range
  a.tier1 = allow_tier1 && (double)a.flo == lo && a.step > 0x1p-100 && a.step < 0x1p100 && (hi - lo) < 0x1p100;
  if (a.tier1) {
    const float r = (float)(1.0 / a.step);
    int ex;
    frexpf(r, &ex);         // r = m * 2^ex, m in [0.5, 1)
    const int sc = 1 - ex;  // r * 2^sc in [1, 2)
    a.rstep32 = ldexpf(r, sc);
    const float pow2k = ldexpf(1.0f, k + sc);
    a.magic32 = nextafterf(pow2k, INFINITY);
#ifdef __CUDA_ARCH__
    a.magic_bits = __float_as_uint(pow2k);
#else
    memcpy(&a.magic_bits, &pow2k, sizeof(float));
#endif
    a.frac_bits32 = (unsigned int)(23 - k);
    a.limit32 = (unsigned int)bins << a.frac_bits32;
    a.frac_hi32 = ((1u << a.frac_bits32) - 1u) & ~1u;
    a.step32 = (double)(float)a.step == a.step ? (float)a.step : 0.0f;
  }
  return true;
}

// Constants of the re-binning of a histogram on [old_lo, old_hi] onto [lo, lo + bins * step]:
// binary64 widths rounded to binary32, as the reference's Python scalars enter its tensors.
__host__ __device__ inline void derive_rebinning(double old_lo, double old_hi, HistArgs& a) {
  a.old_min = (float)old_lo;
  a.old_width = (float)((old_hi - old_lo) / (double)a.bins);
  a.new_min = (float)a.lo;
  a.new_width = (float)a.step;
}

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

// The CTA's copy of the binning constants and its bins (then 32 spare words).  The counting
// loop keeps the handful of tier-1 constants in registers; the out-of-line path for open
// elements reads everything from here, so it costs the loop no registers.
__shared__ HistArgs s_args;
extern __shared__ __align__(16) unsigned int s_bins[];

// Tiers 2 and 3 (and the binary32 tie-break) for an element tier 1 left open, or for every
// element when tier 1 is off.
__device__ __forceinline__ void place_open_inline(float v) {
  const HistArgs& a = s_args;
  if (!(v >= a.flo && v <= a.fhi)) return;  // outside the range, or NaN
  const unsigned int last = (unsigned int)a.bins - 1u;
  if (a.tier1 && a.step32 != 0.0f) {
    // Low-precision data on a binary32 step: when v - lo is exact in binary32 (checked with
    // the error term of the subtraction), the sign of fma(-n, step, v - lo) decides the edge
    // exactly, and a nonzero distance to it is far above what binary64 rounding could bridge.
    const float d = __fsub_rn(v, a.flo);
    const float bb = __fsub_rn(d, v);
    const float err = __fadd_rn(__fsub_rn(v, __fsub_rn(d, bb)), __fsub_rn(-a.flo, bb));
    const unsigned int u = __float_as_uint(__fadd_rz(__fmul_rn(d, a.rstep32), a.magic32)) - a.magic_bits;
    const unsigned int n = u >> a.frac_bits32;
    if (err == 0.0f && (u & a.frac_hi32) == 0u && n <= last + 1u) {
      const unsigned int b = __fmaf_rn(-(float)n, a.step32, d) >= 0.0f ? n : n - 1u;
      atomicAdd(s_bins + (b < last ? b : last), 1u);
      return;
    }
  }
  atomicAdd(s_bins + bin_in_binary64(__dsub_rn((double)v, a.lo), a.step, a.rstep, last), 1u);
}

__device__ __noinline__ void place_open(float v) { place_open_inline(v); }

struct Binner {
  float flo, rstep32, magic32;
  unsigned int magic_bits, limit, frac_bits, frac_hi;
  unsigned int spare;  // this lane's spare word after the bins (one per lane: no two lanes of a
                       // warp ever collide on it, however many elements are left open)

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
        : "r"(__float_as_uint(s)), "r"(magic_bits), "r"(frac_hi), "r"(limit), "r"(frac_bits), "r"(spare),
          "r"(bit));
    return idx;
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
    for (int j = 0; j < 16; ++j) atomicAdd(s_bins + b.classify(e[j], open, 1u << j), 1u);
    // Open elements, one element index at a time for the whole warp: the index runs over the
    // union of the lanes' masks, so sparse data costs an iteration or two and data that sits on
    // bin edges keeps the warp together (each lane walking its own mask diverged sixteen ways).
    const unsigned int lanes = __activemask();
    unsigned int todo = __reduce_or_sync(lanes, open);
    if (todo) {
      float again[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) again[j] = e[j];
      do {
        const int j = __ffs(todo) - 1;
        todo &= todo - 1u;
        if ((open >> j) & 1u) place_open_inline(again[j]);
      } while (todo);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) place_open(e[j]);
  }
}
template <bool TIER1>
__device__ __forceinline__ void count1(float v, const Binner& b, float& mn, float& mx) {
  mn = fminf(mn, v), mx = fmaxf(mx, v);
  unsigned int bin;
  if (TIER1 && b.certain(v, bin))
    atomicAdd(s_bins + bin, 1u);
  else
    place_open(v);
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

// Fold of the previous histogram by the last CTA.  `smem` holds hist_smem_bytes(bins): three
// arrays of `bins` words here; during the counting phase the bins, then 32 spare words.
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

// Counting phase of one CTA: x[0..n) into the shared-memory bins, min / max on the side.
template <typename In, bool TIER1>
__device__ __forceinline__ void count_stream(const In* __restrict__ x, size_t n, bool vec_ok, const HistArgs& a,
                                             unsigned int* smem, float& mn, float& mx) {
  const Binner b{a.flo, a.rstep32, a.magic32, a.magic_bits, a.limit32, a.frac_bits32, a.frac_hi32,
                 (unsigned int)a.bins + (threadIdx.x & 31u)};
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
}

template <typename In>
__device__ __forceinline__ void count_cta(const In* __restrict__ x, size_t n, bool vec_ok, const HistArgs& a,
                                          unsigned int* smem, float& mn, float& mx) {
  for (int j = threadIdx.x; j < a.bins; j += kHistThreads) smem[j] = 0u;
  if (threadIdx.x == 0) s_args = a;
  __syncthreads();
  if (a.tier1)
    count_stream<In, true>(x, n, vec_ok, a, smem, mn, mx);
  else
    count_stream<In, false>(x, n, vec_ok, a, smem, mn, mx);
}

// min / max only (the first batch of an observer has no range to bin on yet)
template <typename In>
__device__ __forceinline__ void range_stream(const In* __restrict__ x, size_t n, bool vec_ok, float& mn, float& mx) {
  constexpr int E = 16 / sizeof(In);
  constexpr int V = Unpack<In>::kVecs;
  const size_t nvec = vec_ok ? n / E : 0;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const size_t first = (size_t)blockIdx.x * kHistThreads + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * kHistThreads;
  size_t i = first;
  for (; i + (V - 1) * stride < nvec; i += V * stride) {
    uint4 cur[V];
#pragma unroll
    for (int j = 0; j < V; ++j) cur[j] = ld_stream_u4(xv + i + j * stride);
    float e[16];
    Unpack<In>::run(cur, e);
#pragma unroll
    for (int j = 0; j < 16; j += 2) mn = min3(mn, e[j], e[j + 1]), mx = max3(mx, e[j], e[j + 1]);
  }
  for (; i < nvec; i += stride) {
    const In* p = x + i * E;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float v = load1<In>(p + j);
      mn = fminf(mn, v), mx = fmaxf(mx, v);
    }
  }
  for (size_t e1 = nvec * E + first; e1 < n; e1 += stride) {
    const float v = load1<In>(x + e1);
    mn = fminf(mn, v), mx = fmaxf(mx, v);
  }
}

// Adds the CTA's bins (if any) to the global counters and takes a ticket.  True in the CTA
// that took the last one; there mn / mx come back reduced over the whole grid.
__device__ __forceinline__ bool flush_and_ticket(int bins, const unsigned int* smem, HistWorkspace* ws, float& mn,
                                                 float& mx) {
  block_minmax_h(mn, mx);  // also orders the shared atomics before the flush
  for (int j = threadIdx.x; j < bins; j += kHistThreads) {
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
  if (!is_last) return false;
  __threadfence();
  mn = INFINITY, mx = -INFINITY;
  for (unsigned int k = threadIdx.x; k < gridDim.x; k += kHistThreads) {
    mn = fminf(mn, __ldcg(&ws->pmin[k]));
    mx = fmaxf(mx, __ldcg(&ws->pmax[k]));
  }
  block_minmax_h(mn, mx);
  __shared__ float s_range[2];
  if (threadIdx.x == 0) {
    s_range[0] = mn, s_range[1] = mx;
    ws->ticket = 0;
  }
  __syncthreads();
  mn = s_range[0], mx = s_range[1];
  return true;
}

template <typename In>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
histc_kernel(const In* __restrict__ x, size_t n, bool vec_ok, HistArgs a, HistWorkspace* ws) {
  unsigned int* smem = s_bins;
  float mn = INFINITY, mx = -INFINITY;
  count_cta<In>(x, n, vec_ok, a, smem, mn, mx);
  if (!flush_and_ticket(a.bins, smem, ws, mn, mx)) return;
  if (threadIdx.x == 0) {
    if (a.out_min) *a.out_min = mn;
    if (a.out_max) *a.out_max = mx;
  }
  finish_histogram(a, ws, smem);
}

// ---- the histogram observer's step, with its state on the device ----------------------------
// HistogramObserver.forward (lucid/quantization/observer.py:819-838) reads the batch's min / max
// and its own range back to the host to decide how to bin.  Here the decision is taken by the
// kernels, so a step is two launches and no host synchronisation:
//   pass 1  bins the batch on the CURRENT range while measuring the batch's own range.  If the
//           range held (the common case once calibration has seen a few batches) its last CTA
//           folds the running histogram and the step is done after one pass over the batch.
//           Otherwise (first batch, range grew, constant history) it records the new range.
//   pass 2  returns at once unless pass 1 asked for it; else bins on the new range and folds
//           the running histogram, re-binned from the old range.
template <typename In>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
observe_pass1(const In* __restrict__ x, size_t n, bool vec_ok, int bins, bool allow_tier1, float* min_val,
              float* max_val, float* hist, HistWorkspace* ws) {
  unsigned int* smem = s_bins;
  const double lo = (double)__ldcg(min_val), hi = (double)__ldcg(max_val);
  const bool seeded = lo < INFINITY && hi > -INFINITY;  // the seed is (+inf, -inf)
  HistArgs a{};
  const bool speculate = seeded && hi > lo && derive_binning(lo, hi, bins, allow_tier1, a);
  float mn = INFINITY, mx = -INFINITY;
  if (speculate)
    count_cta<In>(x, n, vec_ok, a, smem, mn, mx);
  else
    range_stream<In>(x, n, vec_ok, mn, mx);
  if (!flush_and_ticket(speculate ? bins : 0, smem, ws, mn, mx)) return;

  const double new_lo = seeded ? fmin(lo, (double)mn) : (double)mn;
  const double new_hi = seeded ? fmax(hi, (double)mx) : (double)mx;
  const bool grew = !(new_lo == lo && new_hi == hi);
  if (speculate && !grew) {
    a.prev_mode = kPrevAdd, a.prev = hist, a.out = hist;
    finish_histogram(a, ws, smem);
    if (threadIdx.x == 0) ws->observe.pass2 = 0;
    return;
  }
  if (speculate)  // the speculative counts are void
    for (int j = threadIdx.x; j < bins; j += kHistThreads) ws->counts[j] = 0ull;
  if (threadIdx.x == 0) {
    // a batch without a finite value leaves the state as it was
    const bool usable = new_lo < INFINITY && new_lo > -INFINITY && new_hi < INFINITY && new_hi > -INFINITY;
    ws->observe.pass2 = usable ? 1 : 0;
    ws->observe.mode = !seeded ? kPrevNone : (grew ? kPrevRebin : kPrevAdd);
    ws->observe.new_lo = new_lo, ws->observe.new_hi = new_hi;
    ws->observe.old_lo = lo, ws->observe.old_hi = hi;
    if (usable) *min_val = (float)new_lo, *max_val = (float)new_hi;
  }
}

template <typename In>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
observe_pass2(const In* __restrict__ x, size_t n, bool vec_ok, int bins, bool allow_tier1, float* hist,
              HistWorkspace* ws) {
  unsigned int* smem = s_bins;
  if (__ldcg(&ws->observe.pass2) == 0) return;
  const double lo = __ldcg(&ws->observe.new_lo);
  double hi = __ldcg(&ws->observe.new_hi);
  if (!(hi > lo)) hi = lo + 1.0;  // a constant tensor is binned on [v, v + 1] (Stats.cpp:63-72)
  const int mode = __ldcg(&ws->observe.mode);
  const double old_lo = __ldcg(&ws->observe.old_lo), old_hi = __ldcg(&ws->observe.old_hi);
  HistArgs a{};
  if (!derive_binning(lo, hi, bins, allow_tier1, a)) return;  // uniform over the grid
  float mn = INFINITY, mx = -INFINITY;
  count_cta<In>(x, n, vec_ok, a, smem, mn, mx);
  if (!flush_and_ticket(bins, smem, ws, mn, mx)) return;
  a.prev_mode = mode, a.prev = hist, a.out = hist;
  if (mode == kPrevRebin) derive_rebinning(old_lo, old_hi, a);
  finish_histogram(a, ws, smem);
  if (threadIdx.x == 0) ws->observe.pass2 = 0;
}

}  // namespace
// LQ_HIST_BINARY64 (diagnostic: force the binary64 binning tier), read once and again by
// lq_reload_env().
static bool g_hist_binary64 = getenv("LQ_HIST_BINARY64") != nullptr;
static bool hist_force_binary64() { return g_hist_binary64; }
// LQ_HIST_CTAS_PER_SM (1..4): resident CTAs per SM of the binning kernels (measurement knob).
static int read_hist_ctas() {
  const char* e = getenv("LQ_HIST_CTAS_PER_SM");
  const int v = e ? atoi(e) : 0;
  return v >= 1 && v <= kHistCtasPerSm ? v : kHistCtasPerSm;
}
static int g_hist_ctas = read_hist_ctas();
void reload_hist_knobs() {
  g_hist_binary64 = getenv("LQ_HIST_BINARY64") != nullptr;
  g_hist_ctas = read_hist_ctas();
}
}  // namespace lq

using namespace lq;

namespace {
size_t hist_smem_bytes(int bins) {
  const size_t words = (size_t)bins * 3 > (size_t)bins + 32 ? (size_t)bins * 3 : (size_t)bins + 32;
  return words * sizeof(unsigned int);
}
// four 16-byte vectors per thread and iteration; grid capped at the resident CTA count
int hist_grid(size_t n, size_t esz) {
  const size_t per_cta = (size_t)kHistThreads * 4 * (16 / esz);
  const size_t want = (n + per_cta - 1) / per_cta;
  size_t cap = (size_t)sm_count() * g_hist_ctas;
  if (cap > (size_t)kHistMaxCtas) cap = (size_t)kHistMaxCtas;  // slots of the workspace
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}
int check_hist_common(const char* who, const void* x, size_t n, int in_dtype, int bins, const void* workspace,
                      size_t workspace_bytes) {
  const std::string w(who);
  if (!x) return fail(LQ_ERR_DEVICE, w + ": null pointer");
  if (n == 0) return fail(LQ_ERR_SHAPE, w + ": empty input");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, w + ": in_dtype");
  if (bins < 1 || bins > kHistMaxBins)
    return fail(LQ_ERR_UNSUPPORTED, w + ": bins must be in [1, " + std::to_string(kHistMaxBins) + "]");
  if (!workspace) return fail(LQ_ERR_DEVICE, w + ": workspace");
  if (workspace_bytes < sizeof(HistWorkspace))
    return fail(LQ_ERR_WORKSPACE, w + ": workspace smaller than lq_histc_workspace_bytes()");
  if (!aligned16(workspace)) return fail(LQ_ERR_ALIGNMENT, w + ": workspace alignment");
  return LQ_OK;
}
}  // namespace

extern "C" int lq_histogram_observe(const void* x, int in_dtype, size_t n, int bins, float* min_val,
                                    float* max_val, float* hist, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  if (int rc = check_hist_common("lq_histogram_observe", x, n, in_dtype, bins, workspace, workspace_bytes)) return rc;
  if (!min_val || !max_val || !hist) return fail(LQ_ERR_DEVICE, "lq_histogram_observe: null state pointer");
  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  const bool vec_ok = aligned16(x);
  const bool allow_tier1 = !hist_force_binary64();
  const int grid = hist_grid(n, esz);
  const size_t smem = hist_smem_bytes(bins);
  auto* ws = (HistWorkspace*)workspace;
  cudaStream_t st = (cudaStream_t)stream;
  auto launch = [&](auto k1, auto k2, auto ptr) -> int {
    if (smem > 40 * 1024) {  // static shared memory included, this passes the 48 KB default
      LQ_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      LQ_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    k1<<<grid, kHistThreads, smem, st>>>(ptr, n, vec_ok, bins, allow_tier1, min_val, max_val, hist, ws);
    k2<<<grid, kHistThreads, smem, st>>>(ptr, n, vec_ok, bins, allow_tier1, hist, ws);
    return LQ_OK;
  };
  const int rc = in_dtype == LQ_F32
                     ? launch(observe_pass1<float>, observe_pass2<float>, (const float*)x)
                     : launch(observe_pass1<__nv_bfloat16>, observe_pass2<__nv_bfloat16>, (const __nv_bfloat16*)x);
  if (rc != LQ_OK) return rc;
  return check_cuda(cudaGetLastError(), "lq_histogram_observe launch");
}

extern "C" size_t lq_histc_workspace_bytes(void) { return sizeof(HistWorkspace); }
extern "C" int lq_histc_max_bins(void) { return kHistMaxBins; }

extern "C" int lq_histc(const void* x, int in_dtype, size_t n, double lo, double hi, int bins,
                        const float* prev_hist, double prev_lo, double prev_hi, float* hist_out,
                        float* out_min, float* out_max, void* workspace, size_t workspace_bytes,
                        void* stream) {
  if (int rc = check_hist_common("lq_histc", x, n, in_dtype, bins, workspace, workspace_bytes)) return rc;
  if (!hist_out) return fail(LQ_ERR_DEVICE, "lq_histc: null pointer");
  if (!(hi > lo) || !isfinite(lo) || !isfinite(hi))
    return fail(LQ_ERR_SHAPE, "lq_histc: the range must be finite with lo < hi (the caller derives an empty "
                              "range from the data, as the reference's histc does)");

  HistArgs a{};
  if (!derive_binning(lo, hi, bins, !hist_force_binary64(), a))
    return fail(LQ_ERR_SHAPE, "lq_histc: (hi - lo) / bins is not a positive finite number");
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
    derive_rebinning(prev_lo, prev_hi, a);
  }

  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  const bool vec_ok = aligned16(x);
  const int grid = hist_grid(n, esz);
  const size_t smem = hist_smem_bytes(bins);
  auto launch = [&](auto kernel, auto ptr) -> int {
    if (smem > 40 * 1024)  // static shared memory included, this passes the 48 KB default
      LQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, kHistThreads, smem, (cudaStream_t)stream>>>(ptr, n, vec_ok, a, (HistWorkspace*)workspace);
    return LQ_OK;
  };
  const int rc = in_dtype == LQ_F32 ? launch(histc_kernel<float>, (const float*)x)
                                    : launch(histc_kernel<__nv_bfloat16>, (const __nv_bfloat16*)x);
  if (rc != LQ_OK) return rc;
  return check_cuda(cudaGetLastError(), "lq_histc launch");
}
