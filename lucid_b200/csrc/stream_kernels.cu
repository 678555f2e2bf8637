// HBM-bound streaming kernels: range reduction, qparams, quantize, dequantize,
// fake-quantize and the fused per-token encode.  All are 128-bit coalesced
// streams; lanes take consecutive 4-element groups (full-line warp accesses) and the grids are sized
// in multiples of the SM count.  Arithmetic follows the reference's order with
// one IEEE binary32 operation per step (see common.cuh).
#include <math.h>
#include <stdlib.h>

#include <mutex>
#include <string>

#include "common.cuh"

namespace lq {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;
constexpr int kMaxBlocks = kNumSMs * kCtasPerSm;  // 1184: per-CTA partial slots of the range-reduction workspace
inline size_t row_grid_cap() {
  const size_t c = (size_t)sm_count() * kCtasPerSm;
  return c < (size_t)kMaxBlocks ? c : (size_t)kMaxBlocks;
}

struct QParamRef {
  const float* s;
  const float* z;
  float sv, zv;
  int mode;
};

// ---- 16-element packets ----------------------------------------------------
template <typename T>
struct Packet;

template <>
struct Packet<float> {
  __device__ static void load(const float* p, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u = ld_stream_u4(p + 4 * i);
      v[4 * i + 0] = __uint_as_float(u.x);
      v[4 * i + 1] = __uint_as_float(u.y);
      v[4 * i + 2] = __uint_as_float(u.z);
      v[4 * i + 3] = __uint_as_float(u.w);
    }
  }
  __device__ static void store(float* p, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      st_stream_u4(p + 4 * i, make_uint4(__float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]),
                                         __float_as_uint(v[4 * i + 2]),
                                         __float_as_uint(v[4 * i + 3])));
  }
  __device__ static float load1(const float* p) { return *p; }
  __device__ static void store1(float* p, float v) { *p = v; }
};

template <>
struct Packet<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 u = ld_stream_u4(p + 8 * i);
      uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = bf16_bits_to_f32(w[j] & 0xffffu);
        v[8 * i + 2 * j + 1] = bf16_bits_to_f32(w[j] >> 16);
      }
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        w[j] = f32_to_bf16_bits(v[8 * i + 2 * j]) | (f32_to_bf16_bits(v[8 * i + 2 * j + 1]) << 16);
      st_stream_u4(p + 8 * i, make_uint4(w[0], w[1], w[2], w[3]));
    }
  }
  __device__ static float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// 8-bit codes (signed or unsigned share the packing: low byte of the int).
template <typename T>
struct Packet8 {
  __device__ static void load(const T* p, float (&v)[16]) {
    uint4 u = ld_stream_u4(p);
    uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int b = 0; b < 4; ++b) v[4 * j + b] = (float)(T)((w[j] >> (8 * b)) & 0xffu);
  }
  __device__ static void store(T* p, const float (&v)[16]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      w[j] = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) w[j] |= ((uint32_t)(int)v[4 * j + b] & 0xffu) << (8 * b);
    }
    st_stream_u4(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
  __device__ static float load1(const T* p) { return (float)*p; }
  __device__ static void store1(T* p, float v) { *p = (T)(int)v; }
};
template <>
struct Packet<int8_t> : Packet8<int8_t> {};
template <>
struct Packet<uint8_t> : Packet8<uint8_t> {};

template <>
struct Packet<int16_t> {
  __device__ static void load(const int16_t* p, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 u = ld_stream_u4(p + 8 * i);
      uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = (float)(int16_t)(w[j] & 0xffffu);
        v[8 * i + 2 * j + 1] = (float)(int16_t)(w[j] >> 16);
      }
    }
  }
  __device__ static void store(int16_t* p, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        w[j] = ((uint32_t)(int)v[8 * i + 2 * j] & 0xffffu) |
               (((uint32_t)(int)v[8 * i + 2 * j + 1] & 0xffffu) << 16);
      st_stream_u4(p + 8 * i, make_uint4(w[0], w[1], w[2], w[3]));
    }
  }
  __device__ static float load1(const int16_t* p) { return (float)*p; }
  __device__ static void store1(int16_t* p, float v) { *p = (int16_t)(int)v; }
};

// ---- 4-element groups: the unit of the coalesced streams ---------------------------------
// Consecutive lanes take consecutive groups, so every warp-level access is one contiguous
// run (512 B of f32, 256 B of bf16 / s16, 128 B of 8-bit codes): full lines, no sector is
// fetched twice.
template <typename T>
struct Quad;
template <>
struct Quad<float> {
  __device__ static void load(const float* p, float (&v)[4]) {
    const uint4 u = ld_stream_u4(p);
    v[0] = __uint_as_float(u.x), v[1] = __uint_as_float(u.y), v[2] = __uint_as_float(u.z), v[3] = __uint_as_float(u.w);
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    st_stream_u4(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
  }
};
__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream_u1(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_u2(void* p, uint2 v) {
  asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream_u1(void* p, uint32_t v) {
  asm volatile("st.global.L1::no_allocate.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <>
struct Quad<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = ld_stream_u2(p);
    v[0] = bf16_bits_to_f32(u.x & 0xffffu), v[1] = bf16_bits_to_f32(u.x >> 16);
    v[2] = bf16_bits_to_f32(u.y & 0xffffu), v[3] = bf16_bits_to_f32(u.y >> 16);
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[4]) {
    st_stream_u2(p, make_uint2(f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16),
                               f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16)));
  }
};
template <typename T>
struct Quad8 {
  __device__ static void load(const T* p, float (&v)[4]) {
    const uint32_t u = ld_stream_u1(p);
#pragma unroll
    for (int b = 0; b < 4; ++b) v[b] = (float)(T)((u >> (8 * b)) & 0xffu);
  }
  __device__ static void store(T* p, const float (&v)[4]) {
    // values arrive clipped to the grid, which lies inside the storage type
    st_stream_u1(p, sizeof(T) == 1 && T(-1) < T(0) ? pack4_s8(v) : pack4_u8(v));
  }
};
template <typename T>
struct StoreRange;
template <>
struct StoreRange<int8_t> { static constexpr int lo = -128, hi = 127; };
template <>
struct StoreRange<uint8_t> { static constexpr int lo = 0, hi = 255; };
template <>
struct StoreRange<int16_t> { static constexpr int lo = -32768, hi = 32767; };
template <>
struct StoreRange<float> { static constexpr int lo = 0, hi = 0; };
template <>
struct StoreRange<__nv_bfloat16> { static constexpr int lo = 0, hi = 0; };
// four integer codes -> storage (saturating)
__device__ __forceinline__ void store_codes(int8_t* p, const int (&c)[4]) { st_stream_u1(p, pack4i_s8(c)); }
__device__ __forceinline__ void store_codes(uint8_t* p, const int (&c)[4]) { st_stream_u1(p, pack4i_u8(c)); }
__device__ __forceinline__ void store_codes(int16_t* p, const int (&c)[4]) {
  uint32_t lo, hi;
  asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(lo) : "r"(c[1]), "r"(c[0]));
  asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(hi) : "r"(c[3]), "r"(c[2]));
  st_stream_u2(p, make_uint2(lo, hi));
}
__device__ __forceinline__ void store_codes(float*, const int (&)[4]) {}
__device__ __forceinline__ void store_codes(__nv_bfloat16*, const int (&)[4]) {}
template <>
struct Quad<int8_t> : Quad8<int8_t> {};
template <>
struct Quad<uint8_t> : Quad8<uint8_t> {};
template <>
struct Quad<int16_t> {
  __device__ static void load(const int16_t* p, float (&v)[4]) {
    const uint2 u = ld_stream_u2(p);
    v[0] = (float)(int16_t)(u.x & 0xffffu), v[1] = (float)(int16_t)(u.x >> 16);
    v[2] = (float)(int16_t)(u.y & 0xffffu), v[3] = (float)(int16_t)(u.y >> 16);
  }
  __device__ static void store(int16_t* p, const float (&v)[4]) {
    st_stream_u2(p, make_uint2(((uint32_t)(int)v[0] & 0xffffu) | (((uint32_t)(int)v[1] & 0xffffu) << 16),
                               ((uint32_t)(int)v[2] & 0xffffu) | (((uint32_t)(int)v[3] & 0xffffu) << 16)));
  }
};

__device__ __forceinline__ void quad_params(const QParamRef& q, size_t elem, size_t cols,
                                            float (&s)[4], float (&z)[4]) {
  if (q.mode == LQ_PER_COL) {
    const size_t col = elem % cols;
    const float4 a = __ldg(reinterpret_cast<const float4*>(q.s + col));
    const float4 b = __ldg(reinterpret_cast<const float4*>(q.z + col));
    s[0] = a.x, s[1] = a.y, s[2] = a.z, s[3] = a.w;
    z[0] = b.x, z[1] = b.y, z[2] = b.z, z[3] = b.w;
  } else {
    float sv, zv;
    if (q.mode == LQ_PER_ROW) {
      const size_t row = elem / cols;
      sv = __ldg(q.s + row), zv = __ldg(q.z + row);
    } else if (q.s != nullptr) {
      sv = __ldg(q.s), zv = __ldg(q.z);
    } else {
      sv = q.sv, zv = q.zv;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = sv, z[i] = zv;
  }
}

__device__ __forceinline__ void scalar_params(const QParamRef& q, size_t row, size_t col, float& s,
                                              float& z) {
  if (q.mode == LQ_PER_COL) {
    s = q.s[col], z = q.z[col];
  } else if (q.mode == LQ_PER_ROW) {
    s = q.s[row], z = q.z[row];
  } else if (q.s != nullptr) {
    s = q.s[0], z = q.z[0];
  } else {
    s = q.sv, z = q.zv;
  }
}

enum class Op { kQuantize, kDequantize, kFakeQuantize };

template <Op OP>
__device__ __forceinline__ float apply(float x, const Divisor& d, float z, float qmin, float qmax,
                                       float* mask) {
  const float s = d.s;
  if (OP == Op::kQuantize) return code_f32(x, d, z, qmin, qmax);
  if (OP == Op::kDequantize) return __fmul_rn(__fsub_rn(x, z), s);
  // fake-quantize: q_pre, clip, (q - z) * s
  float q_pre = __fadd_rn(rintf(div_rn(x, d)), z);
  float q = q_pre < qmin ? qmin : (q_pre > qmax ? qmax : q_pre);
  if (mask) *mask = (q_pre >= qmin ? 1.0f : 0.0f) * (q_pre <= qmax ? 1.0f : 0.0f);
  return __fmul_rn(__fsub_rn(q, z), s);
}

// One 4-element group sharing (scale, zero point): branch-free in the common case.
template <Op OP, bool MASK>
__device__ __forceinline__ void apply4(float (&v)[4], const Divisor& d, float z, float qmin,
                                       float qmax, float (&m)[4]) {
  if (OP == Op::kDequantize) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(__fsub_rn(v[i], z), d.s);
  } else if (OP == Op::kQuantize) {
    float c[4];
    code4_f32(v, d, z, qmin, qmax, c);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = c[i];
  } else {
    float q[4];
    div_rn4(v, d, q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float q_pre = __fadd_rn(rintf(q[i]), z);
      const float c = q_pre < qmin ? qmin : (q_pre > qmax ? qmax : q_pre);
      if (MASK) m[i] = (q_pre >= qmin ? 1.0f : 0.0f) * (q_pre <= qmax ? 1.0f : 0.0f);
      v[i] = __fmul_rn(__fsub_rn(c, z), d.s);
    }
  }
}

// Divisor of a group: hoisted for per-tensor parameters, rebuilt per group otherwise.
template <Op OP>
__device__ __forceinline__ Divisor group_divisor(float s) {
  Divisor d;
  d.s = s, d.y = 0.0f, d.fast = false;
  if (OP != Op::kDequantize) d = make_divisor(s);
  return d;
}

// Vector kernel: kUnroll coalesced 4-element groups per thread-iteration, grid-stride.
// MODE = LQ_PER_TENSOR compiles the per-tensor case on its own (parameters, divisor and integer
// grid live in registers for the whole thread; a group costs its load, the arithmetic and its
// store), MODE < 0 reads the mode at run time.  The encode is issue-bound, so the instructions a
// group does not need are what the specialisation buys.
template <Op OP, typename In, typename Out, bool MASK, int kUnroll, int kMinBlocks, int MODE>
__global__ void __launch_bounds__(kThreads, kMinBlocks)
affine_vec_kernel(const In* __restrict__ x, Out* __restrict__ out, float* __restrict__ mask,
                  size_t rows, size_t cols, QParamRef q, float qmin, float qmax) {
  pdl_wait();  // launched through launch_pdl(): nothing above touches global memory
  pdl_launch_dependents();
  const int mode = MODE >= 0 ? MODE : q.mode;
  const size_t ngroups = rows * cols / 4;
  const size_t span = (size_t)kThreads * kUnroll;
  float st = 1.0f, zt = 0.0f;
  if (mode == LQ_PER_TENSOR) {
    st = q.s != nullptr ? __ldcg(q.s) : q.sv;
    zt = q.z != nullptr ? __ldcg(q.z) : q.zv;
  }
  const Divisor dt = group_divisor<OP>(st);
  const IntGrid igt = make_int_grid(zt, qmin, qmax, StoreRange<Out>::lo, StoreRange<Out>::hi);
  for (size_t base = (size_t)blockIdx.x * span; base < ngroups; base += (size_t)gridDim.x * span) {
    // one pointer per stream; the groups of a thread sit at compile-time offsets from it
    const size_t g0 = base + threadIdx.x;
    const In* xp = x + g0 * 4;
    Out* op = out + g0 * 4;
    const bool whole = base + span <= ngroups;
    float v[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (whole || g0 + (size_t)u * kThreads < ngroups) Quad<In>::load(xp + (size_t)u * kThreads * 4, v[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (!whole && g0 + (size_t)u * kThreads >= ngroups) continue;
      constexpr size_t kStep = (size_t)kThreads * 4;
      float m[4];
      if (mode == LQ_PER_COL) {
        float s[4], z[4];
        quad_params(q, (g0 + (size_t)u * kThreads) * 4, cols, s, z);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          Divisor d;
          d.s = s[i], d.y = 0.0f, d.fast = false;
          if (OP != Op::kDequantize) d = make_divisor(s[i]);
          v[u][i] = apply<OP>(v[u][i], d, z[i], qmin, qmax, MASK ? &m[i] : nullptr);
        }
      } else {
        Divisor d = dt;
        IntGrid ig = igt;
        float z0 = zt;
        if (mode != LQ_PER_TENSOR) {
          float s[4], z[4];
          quad_params(q, (g0 + (size_t)u * kThreads) * 4, cols, s, z);
          d = group_divisor<OP>(s[0]);
          z0 = z[0];
          if (OP == Op::kQuantize) ig = make_int_grid(z0, qmin, qmax, StoreRange<Out>::lo, StoreRange<Out>::hi);
        }
        if (OP == Op::kQuantize) {
          int c[4];
          code4_int(v[u], d, ig, z0, qmin, qmax, c);
          store_codes(op + u * kStep, c);
          continue;
        }
        apply4<OP, MASK>(v[u], d, z0, qmin, qmax, m);
      }
      Quad<Out>::store(op + u * kStep, v[u]);
      if (MASK) Quad<float>::store(mask + g0 * 4 + u * kStep, m);
    }
  }
}

// Per-tensor encode, the lean form.  The encode is issue-bound, so a group costs only its
// load, five multiply-adds per element (reciprocal estimate + two correction steps = the correctly
// rounded quotient), the magic-number rounding and its store.  An element outside the short
// division's domain (|q| >= 2^22, infinity, NaN) only raises a flag; the thread then redoes its
// whole span through the full-range sequence, out of line and from memory, so that the hot loop
// keeps no registers alive for the rare case.
template <typename In, typename Out>
static __device__ __noinline__ void encode_span_full(const In* __restrict__ x, Out* __restrict__ out, size_t g0,
                                                     size_t ngroups, int unroll, const float* sp, const float* zp,
                                                     float sv, float zv, float qmin, float qmax) {
  const float z = zp != nullptr ? __ldcg(zp) : zv;
  Divisor d;
  d.s = sp != nullptr ? __ldcg(sp) : sv, d.y = 0.0f, d.fast = false;
  for (int u = 0; u < unroll; ++u) {
    const size_t g = g0 + (size_t)u * kThreads;
    if (g >= ngroups) break;
    for (int i = 0; i < 4; ++i) {
      const size_t e = g * 4 + i;
      Packet<Out>::store1(out + e, apply<Op::kQuantize>(Packet<In>::load1(x + e), d, z, qmin, qmax, nullptr));
    }
  }
}

template <typename In, typename Out, int kUnroll, int kMinBlocks, bool PACKED>
__global__ void __launch_bounds__(kThreads, kMinBlocks)
quantize_tensor_kernel(const In* __restrict__ x, Out* __restrict__ out, size_t ngroups, QParamRef q, float qmin,
                       float qmax) {
  pdl_wait();  // launched through launch_pdl(): nothing above touches global memory
  pdl_launch_dependents();
  // (scale, zero point) usually come from the kernel just before this one: read them through L2
  const Divisor d = make_divisor(q.s != nullptr ? __ldcg(q.s) : q.sv);
  const IntGrid ig = make_int_grid(q.z != nullptr ? __ldcg(q.z) : q.zv, qmin, qmax, StoreRange<Out>::lo, StoreRange<Out>::hi);
  const bool lean = d.fast && ig.fast;
  constexpr size_t kSpan = (size_t)kThreads * kUnroll;
  constexpr size_t kStep = (size_t)kThreads * 4;
  for (size_t base = (size_t)blockIdx.x * kSpan; base < ngroups; base += (size_t)gridDim.x * kSpan) {
    const size_t g0 = base + threadIdx.x;
    bool bad = !lean;
    if (lean) {
      const In* xp = x + g0 * 4;
      Out* op = out + g0 * 4;
      const bool whole = base + kSpan <= ngroups;
      float v[kUnroll][4];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (whole || g0 + (size_t)u * kThreads < ngroups) Quad<In>::load(xp + u * kStep, v[u]);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (!whole && g0 + (size_t)u * kThreads >= ngroups) continue;
        int c[4];
        if (PACKED) {
          const F2 y2 = f2_pack(d.y, d.y), ns2 = f2_pack(-d.s, -d.s), magic2 = f2_pack(12582912.0f, 12582912.0f);
          float big = 0.0f;
#pragma unroll
          for (int i = 0; i < 4; i += 2) {
            F2 q0;
            const F2 qq = f2_div_short(f2_pack(v[u][i], v[u][i + 1]), y2, ns2, q0);
            float a, b, t0, t1;
            f2_unpack(q0, a, b);
            // (a NaN input is out of contract -- the reference's integer cast of it is undefined --
            // and is the one value this maximum does not see)
            big = fmaxf(big, fmaxf(fabsf(a), fabsf(b)));
            f2_unpack(f2_add(qq, magic2), t0, t1);
            c[i] = __float_as_int(t0) + ig.zofs;
            c[i + 1] = __float_as_int(t1) + ig.zofs;
          }
          bad |= !(big < 0x1p22f);
          if (ig.clamp) {
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i] = min(max(c[i], ig.qmin), ig.qmax);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float q0 = __fmul_rn(v[u][i], d.y);
            float r = __fmaf_rn(-q0, d.s, v[u][i]);
            const float q1 = __fmaf_rn(r, d.y, q0);
            r = __fmaf_rn(-q1, d.s, v[u][i]);
            const float qq = __fmaf_rn(r, d.y, q1);
            bad |= !(fabsf(q0) < 0x1p22f);
            int t = __float_as_int(__fadd_rn(qq, 12582912.0f)) + ig.zofs;
            if (ig.clamp) t = min(max(t, ig.qmin), ig.qmax);
            c[i] = t;
          }
        }
        store_codes(op + u * kStep, c);
      }
    }
    if (bad) encode_span_full(x, out, g0, ngroups, kUnroll, q.s, q.z, q.sv, q.zv, qmin, qmax);
  }
}

// Scalar kernel: any shape / alignment.
template <Op OP, typename In, typename Out, bool MASK>
__global__ void __launch_bounds__(kThreads)
affine_scalar_kernel(const In* __restrict__ x, Out* __restrict__ out, float* __restrict__ mask,
                     size_t rows, size_t cols, QParamRef q, float qmin, float qmax) {
  const size_t n = rows * cols;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    const size_t row = i / cols, col = i - row * cols;
    float s, z, m;
    scalar_params(q, row, col, s, z);
    Divisor d;
    d.s = s, d.y = 0.0f, d.fast = false;
    float r = apply<OP>(Packet<In>::load1(x + i), d, z, qmin, qmax, MASK ? &m : nullptr);
    Packet<Out>::store1(out + i, r);
    if (MASK) mask[i] = m;
  }
}

inline int grid_for(size_t work_items, size_t ctas_per_sm = 64) {
  size_t blocks = (work_items + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * ctas_per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return (int)blocks;
}

int make_params(const float* scale, const float* zp, float sv, float zv, int ch_mode, QParamRef* q) {
  if (ch_mode < LQ_PER_TENSOR || ch_mode > LQ_PER_COL) return fail(LQ_ERR_SHAPE, "bad ch_mode");
  if (scale == nullptr && ch_mode != LQ_PER_TENSOR)
    return fail(LQ_ERR_DEVICE, "per-channel scale must be a device pointer");
  if ((scale == nullptr) != (zp == nullptr))
    return fail(LQ_ERR_DEVICE, "scale and zero_point must both be pointers or both be host scalars");
  q->s = scale, q->z = zp, q->sv = sv, q->zv = zv, q->mode = ch_mode;
  return LQ_OK;
}

// tuning knobs of the stream kernels (environment, read once; lq_reload_env re-reads)
struct StreamKnobs {
  int ctas_per_sm = 0, unroll = 4, minmax_ctas_per_sm = 6, lean = 1, minmax_pipe = 0;
  int token_pipe_min_row = 16 * 1024, token_ring_kb = 0, token_reg_threads = 256;
  void read() {
    ctas_per_sm = 0, unroll = 4, minmax_ctas_per_sm = 6, lean = 1, minmax_pipe = 0;
    token_pipe_min_row = 16 * 1024, token_ring_kb = 0, token_reg_threads = 256;
    if (const char* e = getenv("LQ_TOKEN_REG_THREADS")) token_reg_threads = atoi(e) == 128 ? 128 : 256;
    if (const char* e = getenv("LQ_TOKEN_PIPE_MIN_ROW")) token_pipe_min_row = atoi(e);
    if (const char* e = getenv("LQ_TOKEN_RING_KB")) token_ring_kb = atoi(e) > 0 && atoi(e) <= 96 ? atoi(e) : 0;
    if (const char* e = getenv("LQ_MINMAX_PIPE")) minmax_pipe = atoi(e);
    if (const char* e = getenv("LQ_QUANT_LEAN")) lean = atoi(e);
    if (const char* e = getenv("LQ_QUANT_CTAS_PER_SM")) ctas_per_sm = atoi(e);
    if (const char* e = getenv("LQ_QUANT_UNROLL")) unroll = atoi(e) == 2 ? 2 : 4;
    if (const char* e = getenv("LQ_MINMAX_CTAS_PER_SM")) minmax_ctas_per_sm = atoi(e) > 0 ? atoi(e) : 6;
  }
};
StreamKnobs& stream_knobs() {
  static StreamKnobs k = [] {
    StreamKnobs v;
    v.read();
    return v;
  }();
  return k;
}

// ---- range reduction -----------------------------------------------------------
struct MinMaxWorkspace {
  unsigned int ticket;
  unsigned int pad[3];
  float pmin[kMaxBlocks];
  float pmax[kMaxBlocks];
};

// Elements per 16-byte vector of the input type.
template <typename In>
struct VecOf {
  static constexpr int kElems = 16 / sizeof(In);
};
template <typename In>
__device__ __forceinline__ void vec_minmax(uint4 u, float& mn, float& mx);
template <>
__device__ __forceinline__ void vec_minmax<float>(uint4 u, float& mn, float& mx) {
  const float a = __uint_as_float(u.x), b = __uint_as_float(u.y), c = __uint_as_float(u.z), d = __uint_as_float(u.w);
  mn = fminf(mn, fminf(fminf(a, b), fminf(c, d)));
  mx = fmaxf(mx, fmaxf(fmaxf(a, b), fmaxf(c, d)));
}
template <>
__device__ __forceinline__ void vec_minmax<__nv_bfloat16>(uint4 u, float& mn, float& mx) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a = bf16_bits_to_f32(w[j] & 0xffffu), b = bf16_bits_to_f32(w[j] >> 16);
    mn = fminf(mn, fminf(a, b));
    mx = fmaxf(mx, fmaxf(a, b));
  }
}

// Abs-max over 16-byte vectors.  bf16 stays packed: the sign bits are masked off and pairs are
// folded with the two-wide bf16 maximum (one mask + one maximum per two elements).
template <typename In>
struct AbsMax;
template <>
struct AbsMax<float> {
  float m = 0.0f;
  __device__ __forceinline__ void add(uint4 u) {
    const float a = __uint_as_float(u.x), b = __uint_as_float(u.y), c = __uint_as_float(u.z), d = __uint_as_float(u.w);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(a), fabsf(b)), fmaxf(fabsf(c), fabsf(d))));
  }
  __device__ __forceinline__ float get() const { return m; }
};
template <>
struct AbsMax<__nv_bfloat16> {
  uint32_t m = 0u;
  __device__ __forceinline__ void add(uint4 u) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) asm("max.bf16x2 %0, %0, %1;" : "+r"(m) : "r"(w[j] & 0x7fff7fffu));
  }
  __device__ __forceinline__ float get() const {
    return fmaxf(bf16_bits_to_f32(m & 0xffffu), bf16_bits_to_f32(m >> 16));
  }
};

// x[0..n): lane `first` of `stride` cooperating threads.  16-byte vectors, consecutive
// threads on consecutive vectors, four loads in flight per thread.
template <typename In>
__device__ __forceinline__ void minmax_accumulate(const In* x, size_t n, size_t first, size_t stride,
                                                  bool vec_ok, float& mn, float& mx) {
  constexpr int E = VecOf<In>::kElems;
  const size_t nvec = vec_ok ? n / E : 0;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  size_t i = first;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = ld_stream_u4(xv + i), b = ld_stream_u4(xv + i + stride);
    const uint4 c = ld_stream_u4(xv + i + 2 * stride), d = ld_stream_u4(xv + i + 3 * stride);
    vec_minmax<In>(a, mn, mx), vec_minmax<In>(b, mn, mx), vec_minmax<In>(c, mn, mx), vec_minmax<In>(d, mn, mx);
  }
  if (i < nvec) {
    // up to three vectors left for this thread: issued together (one latency, not three); a
    // vector past the end re-reads the first one, which changes no min / max
    const size_t i1 = i + stride < nvec ? i + stride : i, i2 = i + 2 * stride < nvec ? i + 2 * stride : i;
    const uint4 a = ld_stream_u4(xv + i), b = ld_stream_u4(xv + i1), c = ld_stream_u4(xv + i2);
    vec_minmax<In>(a, mn, mx), vec_minmax<In>(b, mn, mx), vec_minmax<In>(c, mn, mx);
  }
  for (size_t e = nvec * E + first; e < n; e += stride) {
    const float v = Packet<In>::load1(x + e);
    mn = fminf(mn, v), mx = fmaxf(mx, v);
  }
}

__device__ __forceinline__ void block_minmax(float& mn, float& mx) {
  __shared__ float smn[kThreads / 32], smx[kThreads / 32];
  mn = warp_min(mn), mx = warp_max(mx);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) smn[w] = mn, smx[w] = mx;
  __syncthreads();
  if (w == 0) {
    mn = l < kThreads / 32 ? smn[l] : INFINITY;
    mx = l < kThreads / 32 ? smx[l] : -INFINITY;
    mn = warp_min(mn), mx = warp_max(mx);
  }
  __syncthreads();
}

// ---- bulk-copy pipelined variants ---------------------------------------------------------
// Reads are the long pole of these kernels: with register-staged loads a thread holds a few
// 16-byte loads in flight and idles until they land.  Here each persistent CTA keeps a ring of
// shared-memory slots filled by one-dimensional bulk copies (cp.async.bulk, completion counted
// on an mbarrier): tens of KB per CTA stay in flight with no registers tied up, threads read
// the slot with conflict-free 16-byte shared loads and write results straight to HBM.
constexpr uint32_t kRingBytes = 64 * 1024;
constexpr uint32_t kChunkBytes = 8 * 1024;
constexpr int kRingHeader = 128;  // mbarriers

// Streams at least this large use the bulk-copy ring (LQ_STREAM_PIPE_MIN overrides, bytes).
inline size_t pipe_min_bytes() {
  static const size_t v = [] {
    const char* e = getenv("LQ_STREAM_PIPE_MIN");
    return e ? (size_t)strtoull(e, nullptr, 10) : (size_t)256 * 1024;
  }();
  return v;
}

__device__ __forceinline__ uint4 lds_u4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds_u2(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u1(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
// four consecutive elements of type T from a shared-memory slot
template <typename T>
__device__ __forceinline__ void lds_quad(uint32_t a, float (&v)[4]);
template <>
__device__ __forceinline__ void lds_quad<float>(uint32_t a, float (&v)[4]) {
  const uint4 u = lds_u4(a);
  v[0] = __uint_as_float(u.x), v[1] = __uint_as_float(u.y), v[2] = __uint_as_float(u.z), v[3] = __uint_as_float(u.w);
}
template <>
__device__ __forceinline__ void lds_quad<__nv_bfloat16>(uint32_t a, float (&v)[4]) {
  const uint2 u = lds_u2(a);
  v[0] = bf16_bits_to_f32(u.x & 0xffffu), v[1] = bf16_bits_to_f32(u.x >> 16);
  v[2] = bf16_bits_to_f32(u.y & 0xffffu), v[3] = bf16_bits_to_f32(u.y >> 16);
}
template <>
__device__ __forceinline__ void lds_quad<int16_t>(uint32_t a, float (&v)[4]) {
  const uint2 u = lds_u2(a);
  v[0] = (float)(int16_t)(u.x & 0xffffu), v[1] = (float)(int16_t)(u.x >> 16);
  v[2] = (float)(int16_t)(u.y & 0xffffu), v[3] = (float)(int16_t)(u.y >> 16);
}
template <>
__device__ __forceinline__ void lds_quad<int8_t>(uint32_t a, float (&v)[4]) {
  const uint32_t u = lds_u1(a);
#pragma unroll
  for (int b = 0; b < 4; ++b) v[b] = (float)(int8_t)((u >> (8 * b)) & 0xffu);
}
template <>
__device__ __forceinline__ void lds_quad<uint8_t>(uint32_t a, float (&v)[4]) {
  const uint32_t u = lds_u1(a);
#pragma unroll
  for (int b = 0; b < 4; ++b) v[b] = (float)((u >> (8 * b)) & 0xffu);
}

// Persistent chunk pipeline.  CTA b consumes chunks b, b + G, b + 2G, ... of `chunk_bytes`
// (the last one may be shorter; all sizes are multiples of 16).  `consume(slot_addr, chunk,
// bytes)` is called by every thread of the CTA once the chunk has landed.  Returns false if a
// bounded wait ran out (nothing more is consumed).
template <typename F>
__device__ __forceinline__ bool run_chunks(const uint8_t* src, size_t total_bytes, uint32_t chunk_bytes,
                                           int stages, uint8_t* smem, F&& consume) {
  const uint32_t bar0 = pipe::smem_addr(smem);
  const uint32_t buf0 = bar0 + kRingHeader;
  const size_t nchunks = (total_bytes + chunk_bytes - 1) / chunk_bytes;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) pipe::bar_init(bar0 + 8 * s, 1);
    pipe::bar_init_fence();
  }
  __syncthreads();
  auto bytes_of = [&](size_t c) {
    const size_t rem = total_bytes - c * chunk_bytes;
    return (uint32_t)(rem < chunk_bytes ? rem : chunk_bytes);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      const size_t c = blockIdx.x + (size_t)s * gridDim.x;
      if (c < nchunks) pipe::load_async(buf0 + s * chunk_bytes, src + c * chunk_bytes, bytes_of(c), bar0 + 8 * s);
    }
  }
  int s = 0;
  uint32_t phase = 0;
  for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    if (!__syncthreads_and(pipe::bar_wait(bar0 + 8 * s, phase) ? 1 : 0)) {
      // give copies still in flight time to land before the CTA's shared memory is released
      for (int i = 0; i < 50; ++i) __nanosleep(20000);
      return false;
    }
    consume(buf0 + s * chunk_bytes, c, bytes_of(c));
    pipe::fence_async_smem();  // this thread's reads of the slot precede its refill
    __syncthreads();
    const size_t cn = c + (size_t)stages * gridDim.x;
    if (threadIdx.x == 0 && cn < nchunks)
      pipe::load_async(buf0 + s * chunk_bytes, src + cn * chunk_bytes, bytes_of(cn), bar0 + 8 * s);
    if (++s == stages) s = 0, phase ^= 1u;
  }
  return true;
}

// Number of times a pipelined kernel gave up on a bounded wait (never expected; a copy that
// does not complete means the source range was not readable).  The output of such a launch is
// incomplete; lq_stream_timeouts() reports and clears the count.
__device__ unsigned int g_pipe_timeouts = 0;

template <Op OP, typename In, typename Out, bool MASK>
__global__ void __launch_bounds__(kThreads)
affine_pipe_kernel(const In* __restrict__ x, Out* __restrict__ out, float* __restrict__ mask,
                   size_t n, size_t cols, QParamRef q, float qmin, float qmax, int stages) {
  pdl_wait();  // launched through launch_pdl(): nothing above touches global memory
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t ring[];
  // the 16-byte multiple part goes through the ring; at most 15 bytes of elements are left
  const size_t main_bytes = (n * sizeof(In)) & ~(size_t)15;
  constexpr uint32_t kChunkElems = kChunkBytes / sizeof(In);
  Divisor dt = group_divisor<OP>(1.0f);
  if (q.mode == LQ_PER_TENSOR) dt = group_divisor<OP>(q.s != nullptr ? __ldg(q.s) : q.sv);
  const IntGrid igt = make_int_grid(q.mode == LQ_PER_TENSOR ? (q.z != nullptr ? __ldg(q.z) : q.zv) : 0.0f, qmin, qmax,
                                    StoreRange<Out>::lo, StoreRange<Out>::hi);
  const bool ok = run_chunks(reinterpret_cast<const uint8_t*>(x), main_bytes, kChunkBytes, stages, ring,
                             [&](uint32_t slot, size_t chunk, uint32_t bytes) {
    const uint32_t groups = bytes / (4 * sizeof(In));
    const size_t e0 = chunk * kChunkElems;
#pragma unroll 2
    for (uint32_t g = threadIdx.x; g < groups; g += kThreads) {
      float v[4], s[4], z[4], m[4];
      lds_quad<In>(slot + g * (4 * sizeof(In)), v);
      const size_t e = e0 + (size_t)g * 4;
      quad_params(q, e, cols, s, z);
      if (q.mode == LQ_PER_COL) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          Divisor d;
          d.s = s[i], d.y = 0.0f, d.fast = false;
          if (OP != Op::kDequantize) d = make_divisor(s[i]);
          v[i] = apply<OP>(v[i], d, z[i], qmin, qmax, MASK ? &m[i] : nullptr);
        }
      } else {
        const Divisor d = q.mode == LQ_PER_TENSOR ? dt : group_divisor<OP>(s[0]);
        if (OP == Op::kQuantize) {
          const IntGrid ig = q.mode == LQ_PER_TENSOR ? igt : make_int_grid(z[0], qmin, qmax, StoreRange<Out>::lo, StoreRange<Out>::hi);
          int c[4];
          code4_int(v, d, ig, z[0], qmin, qmax, c);
          store_codes(out + e, c);
          continue;
        }
        apply4<OP, MASK>(v, d, z[0], qmin, qmax, m);
      }
      Quad<Out>::store(out + e, v);
      if (MASK) Quad<float>::store(mask + e, m);
    }
  });
  if (!ok && threadIdx.x == 0) atomicAdd(&g_pipe_timeouts, 1u);
  // elements past the last 16-byte boundary (n % 4 == 0, so this is one group at most)
  const size_t done = main_bytes / sizeof(In);
  if (blockIdx.x == 0 && done < n) {
    for (size_t e = done + threadIdx.x; e < n; e += kThreads) {
      float s1, z1, m1;
      scalar_params(q, e / cols, e % cols, s1, z1);
      Divisor d;
      d.s = s1, d.y = 0.0f, d.fast = false;
      const float r = apply<OP>(Packet<In>::load1(x + e), d, z1, qmin, qmax, MASK ? &m1 : nullptr);
      Packet<Out>::store1(out + e, r);
      if (MASK) mask[e] = m1;
    }
  }
}

template <typename In>
__device__ __forceinline__ void smem_vec_minmax(uint32_t slot, uint32_t bytes, int first, int stride,
                                                float& mn, float& mx) {
  const uint32_t nvec = bytes / 16;
  for (uint32_t i = first; i < nvec; i += stride) vec_minmax<In>(lds_u4(slot + i * 16), mn, mx);
}

// Opt a pipelined kernel into its dynamic shared memory once.
template <typename K>
cudaError_t enable_ring(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <Op OP, typename In, typename Out, bool MASK = false>
int launch_affine(const void* x, void* out, float* mask, size_t rows, size_t cols,
                  const QParamRef& q, int qmin, int qmax, cudaStream_t st) {
  const bool vec = (cols % 4 == 0) && aligned16(x) && aligned16(out) &&
                   (!MASK || aligned16(mask)) &&
                   (q.mode != LQ_PER_COL || (aligned16(q.s) && aligned16(q.z)));
  const size_t n = rows * cols;
  // Measured on B200: the decode (write-heavy, 4 output bytes per input byte) is faster through
  // the bulk-copy ring with persistent CTAs; the encodes are issue-bound and faster with
  // register-staged loads and one CTA per span.
  if (vec && OP == Op::kDequantize && n * sizeof(In) >= pipe_min_bytes()) {
    auto kernel = affine_pipe_kernel<OP, In, Out, MASK>;
    constexpr int stages = kRingBytes / kChunkBytes;
    constexpr size_t smem = kRingHeader + kRingBytes;
    static PerDeviceOnce once;
    const cudaError_t attr = once.run([&] { return enable_ring(kernel, smem); });
    if (attr != cudaSuccess) return check_cuda(attr, "cudaFuncSetAttribute(ring)");
    const size_t nchunks = (n * sizeof(In) + kChunkBytes - 1) / kChunkBytes;
    const size_t cap = (size_t)sm_count() * 3;
    const int grid = (int)(nchunks < cap ? nchunks : cap);
    // an ordinary launch: three of these CTAs fill an SM's shared memory, so the next launch
    // cannot become resident early, and the attribute measured 14.8 against 14.0 us at config 1
    kernel<<<grid, kThreads, smem, st>>>((const In*)x, (Out*)out, mask, n, cols, q, (float)qmin, (float)qmax, stages);
    return check_cuda(cudaGetLastError(), "affine kernel launch");
  } else if (vec) {
    // 4 groups per thread at full occupancy (32 registers): measured fastest on B200
    const StreamKnobs& kn = stream_knobs();
    const size_t groups = n / 4;
    const int unroll = kn.unroll == 2 ? 2 : 4;
    const size_t spans = (groups + unroll - 1) / unroll;
    const int grid = kn.ctas_per_sm > 0 ? grid_for(spans, (size_t)kn.ctas_per_sm) : grid_for(spans);
    const bool tensor = q.mode == LQ_PER_TENSOR;
    if (kn.lean && OP == Op::kQuantize && tensor && !MASK && StoreRange<Out>::lo != StoreRange<Out>::hi) {
      // measured on B200 (config 1, 64 MB): 4 groups per thread at 6 CTAs/SM (40 registers, no
      // spill) 14.6 us; at 8 CTAs/SM (32 registers, 32 B spilled) 15.4 us; scalar multiply-adds
      // instead of the packed ones 15.4 us; the run-time-mode kernel 17.2 us
      return check_cuda(launch_pdl(quantize_tensor_kernel<In, Out, 4, 6, true>, dim3(grid_for((groups + 3) / 4)),
                                   dim3(kThreads), 0, st, (const In*)x, (Out*)out, groups, q, (float)qmin, (float)qmax),
                        "affine kernel launch");
    }
#define LQ_LAUNCH_VEC(U, M)                                                                                   \
  return check_cuda(launch_pdl(affine_vec_kernel<OP, In, Out, MASK, U, 8, M>, dim3(grid), dim3(kThreads), 0, st, \
                               (const In*)x, (Out*)out, mask, rows, cols, q, (float)qmin, (float)qmax),           \
                    "affine kernel launch")
    if (unroll == 2) {
      if (tensor) LQ_LAUNCH_VEC(2, LQ_PER_TENSOR);
      else LQ_LAUNCH_VEC(2, -1);
    } else {
      if (tensor) LQ_LAUNCH_VEC(4, LQ_PER_TENSOR);
      else LQ_LAUNCH_VEC(4, -1);
    }
#undef LQ_LAUNCH_VEC
  } else {
    affine_scalar_kernel<OP, In, Out, MASK><<<grid_for(n), kThreads, 0, st>>>(
        (const In*)x, (Out*)out, mask, rows, cols, q, (float)qmin, (float)qmax);
  }
  return check_cuda(cudaGetLastError(), "affine kernel launch");
}


// (scale, zero_point) of one observed range: the op sequence of calculate_qparams
// (lucid/quantization/_qparams.py:197-215).
__device__ __forceinline__ void qparams_one(float mn, float mx, int symmetric, int is_signed, int qmin, int qmax,
                                            float eps, float* scale, float* zp) {
  const float lo = fminf(mn, 0.0f), hi = fmaxf(mx, 0.0f);
  if (symmetric) {
    const float m = fmaxf(fabsf(lo), fabsf(hi));
    const float half = (float)((double)(qmax - qmin) / 2.0);
    *scale = fmaxf(__fdiv_rn(m, half), eps);
    *zp = is_signed ? 0.0f : (float)((qmax + qmin + 1) / 2);
  } else {
    const float s = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), (float)((double)qmax - (double)qmin)), eps);
    *scale = s;
    const float t = __fsub_rn((float)qmin, rintf(__fdiv_rn(lo, s)));
    const float fq0 = (float)qmin, fq1 = (float)qmax;
    *zp = t < fq0 ? fq0 : (t > fq1 ? fq1 : t);
  }
}
// What the reducing kernel may do with the final range before it returns: derive the grid.
struct FusedQParams {
  float* scale;  // null: nothing to derive
  float* zp;
  int symmetric, is_signed, qmin, qmax;
  float eps;
};

// Order-preserving map of a float onto unsigned integers (and back), so that integer atomics
// fold float minima / maxima.  -0.0 and +0.0 keep their order.
__device__ __forceinline__ unsigned int float_key(float f) {
  const unsigned int b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(unsigned int k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Per-tensor: every CTA folds its pair into two words of the workspace with integer atomics
// (max of the key for the maximum, max of the complemented key for the minimum, so that the
// zero-filled workspace is the identity of both); the CTA that takes the last ticket decodes
// them and re-arms the workspace.  Min / max are exact in any order.
__device__ __forceinline__ void finish_tensor_minmax(float mn, float mx, MinMaxWorkspace* ws,
                                                     float* out_min, float* out_max,
                                                     const FusedQParams& fq = FusedQParams{}) {
  block_minmax(mn, mx);
  if (threadIdx.x != 0) return;
  atomicMax(&ws->pad[0], float_key(mx));
  atomicMax(&ws->pad[1], ~float_key(mn));
  __threadfence();
  if (atomicAdd(&ws->ticket, 1u) != gridDim.x - 1) return;
  __threadfence();
  const unsigned int kmax = atomicExch(&ws->pad[0], 0u), kmin = atomicExch(&ws->pad[1], 0u);
  *out_max = key_float(kmax);
  *out_min = key_float(~kmin);
  if (fq.scale != nullptr)
    qparams_one(key_float(~kmin), key_float(kmax), fq.symmetric, fq.is_signed, fq.qmin, fq.qmax, fq.eps, fq.scale, fq.zp);
  ws->ticket = 0;  // leave the workspace zeroed for the next call
}

template <typename In>
__global__ void __launch_bounds__(kThreads)
minmax_tensor_kernel(const In* __restrict__ x, size_t n, bool vec_ok, MinMaxWorkspace* ws,
                     float* out_min, float* out_max, FusedQParams fq) {
  pdl_wait();  // launched through launch_pdl(): nothing above touches global memory
  pdl_launch_dependents();
  float mn = INFINITY, mx = -INFINITY;
  minmax_accumulate(x, n, (size_t)blockIdx.x * kThreads + threadIdx.x,
                    (size_t)gridDim.x * kThreads, vec_ok, mn, mx);
  finish_tensor_minmax(mn, mx, ws, out_min, out_max, fq);
}

// Per-tensor range reduction through the ring (same partial / ticket scheme as below).
template <typename In>
__global__ void __launch_bounds__(kThreads)
minmax_pipe_kernel(const In* __restrict__ x, size_t n, MinMaxWorkspace* ws, float* out_min,
                   float* out_max, int stages) {
  extern __shared__ __align__(128) uint8_t ring[];
  const size_t main_bytes = (n * sizeof(In)) & ~(size_t)15;
  float mn = INFINITY, mx = -INFINITY;
  const bool ok = run_chunks(reinterpret_cast<const uint8_t*>(x), main_bytes, kChunkBytes, stages, ring,
                             [&](uint32_t slot, size_t, uint32_t bytes) {
    smem_vec_minmax<In>(slot, bytes, threadIdx.x, kThreads, mn, mx);
  });
  if (!ok && threadIdx.x == 0) atomicAdd(&g_pipe_timeouts, 1u);
  if (blockIdx.x == 0)
    for (size_t e = main_bytes / sizeof(In) + threadIdx.x; e < n; e += kThreads) {
      const float v = Packet<In>::load1(x + e);
      mn = fminf(mn, v), mx = fmaxf(mx, v);
    }
  finish_tensor_minmax(mn, mx, ws, out_min, out_max);
}

// Fused per-token encode with the row held in shared memory: one HBM read per element.
// A chunk of the ring is one row; rows are prefetched while earlier ones are encoded.
template <typename In>
__global__ void __launch_bounds__(kThreads)
per_token_pipe_kernel(const In* __restrict__ x, size_t rows, size_t cols, float half, float eps,
                      float qmin, float qmax, int8_t* __restrict__ out, float* __restrict__ out_scale,
                      int stages) {
  pdl_wait();  // launched through launch_pdl(): nothing above touches global memory
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float s_scale;
  const uint32_t row_bytes = (uint32_t)(cols * sizeof(In));
  const bool ok = run_chunks(reinterpret_cast<const uint8_t*>(x), rows * (size_t)row_bytes, row_bytes, stages, ring,
                             [&](uint32_t slot, size_t r, uint32_t) {
    constexpr uint32_t E = VecOf<In>::kElems;
    const uint32_t nvec = row_bytes / 16;
    AbsMax<In> am;
    for (uint32_t i = threadIdx.x; i < nvec; i += kThreads) am.add(lds_u4(slot + i * 16));
    float m = am.get();
    // cols % 4 == 0: at most one 4-element group lies past the last whole vector
    const uint32_t groups = (uint32_t)(cols / 4), tail_g = nvec * (E / 4);
    if (threadIdx.x == 0 && tail_g < groups) {
      float v[4];
      lds_quad<In>(slot + tail_g * (4 * sizeof(In)), v);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
    }
    float lo = 0.0f;  // block_minmax folds a (min, max) pair; only the maximum is used
    block_minmax(lo, m);
    if (threadIdx.x == 0) {
      const float sc = fmaxf(__fdiv_rn(m, half), eps);
      s_scale = sc;
      out_scale[r] = sc;
    }
    __syncthreads();
    const Divisor d = make_divisor(s_scale);
    const IntGrid ig = make_int_grid(0.0f, qmin, qmax, -128, 127);
    const ShortDiv sd = make_short_div(d);
    int8_t* outr = out + r * cols;
    if (d.fast) {
      // every |x| <= abs-max = scale * half, so the short division covers the whole row
      for (uint32_t i = threadIdx.x; i < nvec; i += kThreads) {
        const uint4 u = lds_u4(slot + i * 16);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        if (E == 4) {
          const float f[4] = {__uint_as_float(w[0]), __uint_as_float(w[1]), __uint_as_float(w[2]), __uint_as_float(w[3])};
          int c[4];
          code4_short(f, sd, ig, c);
          st_stream_u1(outr + (size_t)i * 4, pack4i_s8(c));
        } else {
          const float f0[4] = {bf16_bits_to_f32(w[0] & 0xffffu), bf16_bits_to_f32(w[0] >> 16),
                               bf16_bits_to_f32(w[1] & 0xffffu), bf16_bits_to_f32(w[1] >> 16)};
          const float f1[4] = {bf16_bits_to_f32(w[2] & 0xffffu), bf16_bits_to_f32(w[2] >> 16),
                               bf16_bits_to_f32(w[3] & 0xffffu), bf16_bits_to_f32(w[3] >> 16)};
          int c0[4], c1[4];
          code4_short(f0, sd, ig, c0);
          code4_short(f1, sd, ig, c1);
          st_stream_u2(outr + (size_t)i * 8, make_uint2(pack4i_s8(c0), pack4i_s8(c1)));
        }
      }
      if (threadIdx.x == 0 && tail_g < groups) {
        float v[4];
        int c[4];
        lds_quad<In>(slot + tail_g * (4 * sizeof(In)), v);
        code4_short(v, sd, ig, c);
        store_codes(outr + (size_t)tail_g * 4, c);
      }
    } else {
      for (uint32_t g = threadIdx.x; g < groups; g += kThreads) {
        float v[4];
        int c[4];
        lds_quad<In>(slot + g * (4 * sizeof(In)), v);
        code4_int(v, d, ig, 0.0f, qmin, qmax, c);
        store_codes(outr + (size_t)g * 4, c);
      }
    }
  });
  if (!ok && threadIdx.x == 0) atomicAdd(&g_pipe_timeouts, 1u);
}


// Per-row: one CTA per row (grid-stride over rows).
template <typename In>
__global__ void __launch_bounds__(kThreads)
minmax_rows_kernel(const In* __restrict__ x, size_t rows, size_t cols, bool vec_ok,
                   float* __restrict__ out_min, float* __restrict__ out_max) {
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float mn = INFINITY, mx = -INFINITY;
    minmax_accumulate(x + r * cols, cols, threadIdx.x, kThreads, vec_ok, mn, mx);
    block_minmax(mn, mx);
    if (threadIdx.x == 0) out_min[r] = mn, out_max[r] = mx;
  }
}

// Per-row for short rows: one warp per row.
template <typename In>
__global__ void __launch_bounds__(kThreads)
minmax_rows_warp_kernel(const In* __restrict__ x, size_t rows, size_t cols, bool vec_ok,
                        float* __restrict__ out_min, float* __restrict__ out_max) {
  const size_t warps = (size_t)gridDim.x * (kThreads / 32);
  const int l = threadIdx.x & 31;
  for (size_t r = (size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
    float mn = INFINITY, mx = -INFINITY;
    minmax_accumulate(x + r * cols, cols, l, 32, vec_ok, mn, mx);
    mn = warp_min(mn), mx = warp_max(mx);
    if (l == 0) out_min[r] = mn, out_max[r] = mx;
  }
}

__global__ void qparams_kernel(const float* __restrict__ mn, const float* __restrict__ mx, size_t n,
                               int symmetric, int is_signed, int qmin, int qmax, float eps,
                               float* __restrict__ scale, float* __restrict__ zp) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  qparams_one(mn[i], mx[i], symmetric, is_signed, qmin, qmax, eps, scale + i, zp + i);
}

// Fused per-token encode: abs-max of the row, symmetric scale, codes.  The row
// is read twice; the second read is served by L2 (a row is at most ~115 KB).
template <typename In>
__global__ void __launch_bounds__(kThreads)
per_token_kernel(const In* __restrict__ x, size_t rows, size_t cols, bool vec_ok, float half,
                 float eps, float qmin, float qmax, int8_t* __restrict__ out,
                 float* __restrict__ out_scale) {
  __shared__ float s_scale;
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const In* xr = x + r * cols;
    float mn = INFINITY, mx = -INFINITY;
    // first pass: keep the lines in L2 (ld.global.cg through the packet loader's
    // non-allocating L1 policy does that already)
    minmax_accumulate(xr, cols, threadIdx.x, kThreads, vec_ok, mn, mx);
    block_minmax(mn, mx);
    if (threadIdx.x == 0) {
      // |min(mn,0)| v |max(mx,0)| == abs-max of the row
      const float m = fmaxf(fabsf(fminf(mn, 0.0f)), fabsf(fmaxf(mx, 0.0f)));
      const float s = fmaxf(__fdiv_rn(m, half), eps);
      s_scale = s;
      out_scale[r] = s;
    }
    __syncthreads();
    const Divisor s = make_divisor(s_scale);
    const IntGrid ig = make_int_grid(0.0f, qmin, qmax, -128, 127);
    int8_t* outr = out + r * cols;
    const size_t ngr = vec_ok ? cols / 4 : 0;
    for (size_t gi = threadIdx.x; gi < ngr; gi += kThreads) {
      float v[4];
      int c[4];
      Quad<In>::load(xr + gi * 4, v);
      code4_int(v, s, ig, 0.0f, qmin, qmax, c);
      store_codes(outr + gi * 4, c);
    }
    for (size_t i = ngr * 4 + threadIdx.x; i < cols; i += kThreads)
      outr[i] = (int8_t)(int)code_f32(Packet<In>::load1(xr + i), s, 0.0f, qmin, qmax);
    __syncthreads();  // s_scale is rewritten by the next row
  }
}

// Fused per-token encode for rows of at most 16 KB: the row lives in registers (four 16-byte
// vectors per thread, consecutive lanes on consecutive vectors), so HBM is read exactly once
// and nothing is re-read from L2.
template <typename In, int kT, int kV, int kMinBlocks>
__global__ void __launch_bounds__(kT, kMinBlocks)
per_token_reg_kernel(const In* __restrict__ x, size_t rows, size_t cols, float half, float eps,
                     float qmin, float qmax, int8_t* __restrict__ out, float* __restrict__ out_scale) {
  pdl_wait();  // launched through launch_pdl(): nothing above touches global memory
  pdl_launch_dependents();
  constexpr int E = VecOf<In>::kElems;  // elements per 16-byte vector
  __shared__ float s_part[2][kT / 32];
  const uint32_t nvec = (uint32_t)(cols / E);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  int flip = 0;
  uint4 v[kV], vn[kV];
  auto load_row = [&](size_t r, uint4 (&dst)[kV]) {
    const uint4* xv = reinterpret_cast<const uint4*>(x + r * cols);
#pragma unroll
    for (int k = 0; k < kV; ++k) {
      const uint32_t i = threadIdx.x + k * kT;
      dst[k] = i < nvec ? ld_stream_u4(xv + i) : make_uint4(0, 0, 0, 0);  // zeros do not move an abs-max
    }
  };
  if (blockIdx.x < rows) load_row(blockIdx.x, v);
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x, flip ^= 1) {
    // the next row's loads are in flight while this one is encoded
    const size_t rn = r + gridDim.x;
    if (rn < rows) load_row(rn, vn);
    AbsMax<In> acc;  // zero-filled vectors past the row do not move an abs-max
#pragma unroll
    for (int k = 0; k < kV; ++k) acc.add(v[k]);
    float am = warp_max(acc.get());
    if (l == 0) s_part[flip][w] = am;
    __syncthreads();  // the only block barrier per row (partials are double-buffered)
    float m = s_part[flip][0];
#pragma unroll
    for (int i = 1; i < kT / 32; ++i) m = fmaxf(m, s_part[flip][i]);
    const float sc = fmaxf(__fdiv_rn(m, half), eps);
    if (threadIdx.x == 0) out_scale[r] = sc;
    const Divisor d = make_divisor(sc);
    const IntGrid ig = make_int_grid(0.0f, qmin, qmax, -128, 127);
    const ShortDiv sd = make_short_div(d);
    int8_t* outr = out + r * cols;
#pragma unroll
    for (int k = 0; k < kV; ++k) {
      const uint32_t i = threadIdx.x + k * kT;
      if (i >= nvec) continue;
      const uint32_t wv[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
      // every |x| <= abs-max = scale * half: with a divisor in the short division's range the
      // whole row takes it (row-uniform branch)
      if (E == 4) {
        const float f[4] = {__uint_as_float(wv[0]), __uint_as_float(wv[1]), __uint_as_float(wv[2]), __uint_as_float(wv[3])};
        int c[4];
        if (d.fast) code4_short(f, sd, ig, c);
        else code4_int(f, d, ig, 0.0f, qmin, qmax, c);
        st_stream_u1(outr + (size_t)i * 4, pack4i_s8(c));
      } else {
        const float f0[4] = {bf16_bits_to_f32(wv[0] & 0xffffu), bf16_bits_to_f32(wv[0] >> 16),
                             bf16_bits_to_f32(wv[1] & 0xffffu), bf16_bits_to_f32(wv[1] >> 16)};
        const float f1[4] = {bf16_bits_to_f32(wv[2] & 0xffffu), bf16_bits_to_f32(wv[2] >> 16),
                             bf16_bits_to_f32(wv[3] & 0xffffu), bf16_bits_to_f32(wv[3] >> 16)};
        int c0[4], c1[4];
        if (d.fast) {
          code4_short(f0, sd, ig, c0);
          code4_short(f1, sd, ig, c1);
        } else {
          code4_int(f0, d, ig, 0.0f, qmin, qmax, c0);
          code4_int(f1, d, ig, 0.0f, qmin, qmax, c1);
        }
        st_stream_u2(outr + (size_t)i * 8, make_uint2(pack4i_s8(c0), pack4i_s8(c1)));
      }
    }
#pragma unroll
    for (int k = 0; k < kV; ++k) v[k] = vn[k];
  }
}

// sum_k b[n,k]: one warp per row.
__global__ void __launch_bounds__(kThreads)
rowsum_kernel(const int8_t* __restrict__ b, size_t N, size_t K, bool vec_ok,
              int32_t* __restrict__ out) {
  const size_t warps = (size_t)gridDim.x * (kThreads / 32);
  const int l = threadIdx.x & 31;
  for (size_t r = (size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); r < N; r += warps) {
    const int8_t* br = b + r * K;
    int acc = 0;
    const size_t npk = vec_ok ? K / 16 : 0;
    for (size_t p = l; p < npk; p += 32) {
      uint4 u = ld_stream_u4(br + p * 16);
      acc = __dp4a((int)u.x, 0x01010101, acc);
      acc = __dp4a((int)u.y, 0x01010101, acc);
      acc = __dp4a((int)u.z, 0x01010101, acc);
      acc = __dp4a((int)u.w, 0x01010101, acc);
    }
    for (size_t i = npk * 16 + l; i < K; i += 32) acc += (int)br[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (l == 0) out[r] = acc;
  }
}

}  // namespace
}  // namespace lq

using namespace lq;

namespace lq {
namespace {
// Per-tensor range reduction (and, optionally, the grid derived from it by the kernel's last
// CTA): shared by lq_minmax, lq_minmax_noalloc and lq_quantize_dynamic.
int minmax_tensor_launch(const void* x, int in_dtype, size_t n, MinMaxWorkspace* ws, float* out_min, float* out_max,
                         const FusedQParams& fq, cudaStream_t st) {
  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  const bool vec_ok = aligned16(x);
  // two packets per thread-iteration; grid in multiples of the SM count
  size_t want = (n / 16 + 2 * kThreads - 1) / (2 * kThreads);
  const size_t gcap = (size_t)sm_count() * stream_knobs().minmax_ctas_per_sm;
  int grid = (int)(want < 1 ? 1 : (want > gcap ? gcap : want));
  if (vec_ok && fq.scale == nullptr && stream_knobs().minmax_pipe && n * esz >= pipe_min_bytes()) {
    // bulk-copy ring variant (kept for comparison; the register-staged kernel is faster)
    constexpr int stages = kRingBytes / kChunkBytes;
    constexpr size_t smem = kRingHeader + kRingBytes;
    static PerDeviceOnce once;
    const cudaError_t attr = once.run([&] {
      const cudaError_t a32 = enable_ring(minmax_pipe_kernel<float>, smem);
      return a32 != cudaSuccess ? a32 : enable_ring(minmax_pipe_kernel<__nv_bfloat16>, smem);
    });
    if (attr != cudaSuccess) return check_cuda(attr, "cudaFuncSetAttribute(ring)");
    const size_t nchunks = (n * esz + kChunkBytes - 1) / kChunkBytes;
    const size_t pcap = (size_t)sm_count() * 3;
    const int pgrid = (int)(nchunks < pcap ? nchunks : pcap);
    if (in_dtype == LQ_F32)
      minmax_pipe_kernel<float><<<pgrid, kThreads, smem, st>>>((const float*)x, n, ws, out_min, out_max, stages);
    else
      minmax_pipe_kernel<__nv_bfloat16><<<pgrid, kThreads, smem, st>>>((const __nv_bfloat16*)x, n, ws, out_min, out_max, stages);
  } else if (in_dtype == LQ_F32) {
    return check_cuda(launch_pdl(minmax_tensor_kernel<float>, dim3(grid), dim3(kThreads), 0, st, (const float*)x, n, vec_ok,
                                 ws, out_min, out_max, fq), "minmax launch");
  } else {
    return check_cuda(launch_pdl(minmax_tensor_kernel<__nv_bfloat16>, dim3(grid), dim3(kThreads), 0, st,
                                 (const __nv_bfloat16*)x, n, vec_ok, ws, out_min, out_max, fq), "minmax launch");
  }
  return check_cuda(cudaGetLastError(), "range reduction launch");
}
}  // namespace
}  // namespace lq

namespace lq {
void reload_stream_knobs() { stream_knobs().read(); }
}  // namespace lq

extern "C" size_t lq_minmax_workspace_bytes(void) { return sizeof(MinMaxWorkspace); }

extern "C" int lq_stream_timeouts(unsigned int* count) {
  if (!count) return fail(LQ_ERR_DEVICE, "lq_stream_timeouts: null pointer");
  unsigned int v = 0;
  LQ_CUDA(cudaMemcpyFromSymbol(&v, g_pipe_timeouts, sizeof(v)));
  if (v != 0) {
    const unsigned int zero = 0;
    LQ_CUDA(cudaMemcpyToSymbol(g_pipe_timeouts, &zero, sizeof(zero)));
  }
  *count = v;
  return LQ_OK;
}

extern "C" int lq_minmax(const void* x, int in_dtype, size_t rows, size_t cols, int mode,
                         float* out_min, float* out_max, void* workspace, size_t workspace_bytes,
                         void* stream) {
  if (!x || !out_min || !out_max) return fail(LQ_ERR_DEVICE, "lq_minmax: null pointer");
  if (rows == 0 || cols == 0) return fail(LQ_ERR_SHAPE, "lq_minmax: empty input has no min/max");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_minmax: in_dtype");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  if (mode == LQ_PER_TENSOR) {
    if (!workspace) return fail(LQ_ERR_DEVICE, "lq_minmax: per-tensor mode needs a workspace");
    if (workspace_bytes < sizeof(MinMaxWorkspace))
      return fail(LQ_ERR_WORKSPACE, "lq_minmax: workspace smaller than lq_minmax_workspace_bytes()");
    if (!aligned16(workspace)) return fail(LQ_ERR_ALIGNMENT, "lq_minmax: workspace alignment");
    const int rc = minmax_tensor_launch(x, in_dtype, rows * cols, (MinMaxWorkspace*)workspace, out_min, out_max,
                                        FusedQParams{}, st);
    if (rc != LQ_OK) return rc;
  } else if (mode == LQ_PER_ROW) {
    const bool vec_ok = aligned16(x) && ((cols * esz) % 16 == 0);
    if (cols <= 2048) {
      int grid = grid_for(rows * 32);
      if (in_dtype == LQ_F32)
        minmax_rows_warp_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, vec_ok, out_min, out_max);
      else
        minmax_rows_warp_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, vec_ok, out_min, out_max);
    } else {
      int grid = (int)(rows < row_grid_cap() ? rows : row_grid_cap());
      if (in_dtype == LQ_F32)
        minmax_rows_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, vec_ok, out_min, out_max);
      else
        minmax_rows_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, vec_ok, out_min, out_max);
    }
  } else {
    return fail(LQ_ERR_SHAPE, "lq_minmax: mode must be LQ_PER_TENSOR or LQ_PER_ROW");
  }
  return check_cuda(cudaGetLastError(), "lq_minmax launch");
}

extern "C" int lq_calculate_qparams(const float* min_val, const float* max_val, size_t n,
                                    int symmetric, int is_signed, int qmin, int qmax, float eps,
                                    float* scale, float* zero_point, void* stream) {
  if (!min_val || !max_val || !scale || !zero_point)
    return fail(LQ_ERR_DEVICE, "lq_calculate_qparams: null pointer");
  if (n == 0) return LQ_OK;
  if (qmax <= qmin) return fail(LQ_ERR_SHAPE, "lq_calculate_qparams: qmax must exceed qmin");
  qparams_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      min_val, max_val, n, symmetric, is_signed, qmin, qmax, eps, scale, zero_point);
  return check_cuda(cudaGetLastError(), "lq_calculate_qparams launch");
}

extern "C" int lq_quantize(const void* x, int in_dtype, size_t rows, size_t cols,
                           const float* scale, const float* zero_point, float scale_value,
                           float zp_value, int ch_mode, int qmin, int qmax, void* out,
                           int out_dtype, void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!x || !out) return fail(LQ_ERR_DEVICE, "lq_quantize: null pointer");
  QParamRef q;
  int rc = make_params(scale, zero_point, scale_value, zp_value, ch_mode, &q);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
#define LQ_Q(IN, OUT) return launch_affine<Op::kQuantize, IN, OUT>(x, out, nullptr, rows, cols, q, qmin, qmax, st)
  if (in_dtype == LQ_F32) {
    if (out_dtype == LQ_S8) LQ_Q(float, int8_t);
    if (out_dtype == LQ_U8) LQ_Q(float, uint8_t);
    if (out_dtype == LQ_S16) LQ_Q(float, int16_t);
  } else if (in_dtype == LQ_BF16) {
    if (out_dtype == LQ_S8) LQ_Q(__nv_bfloat16, int8_t);
    if (out_dtype == LQ_U8) LQ_Q(__nv_bfloat16, uint8_t);
    if (out_dtype == LQ_S16) LQ_Q(__nv_bfloat16, int16_t);
  }
#undef LQ_Q
  return fail(LQ_ERR_DTYPE, "lq_quantize: in_dtype must be f32|bf16 and out_dtype s8|u8|s16");
}

extern "C" int lq_dequantize(const void* qv, int q_dtype, size_t rows, size_t cols,
                             const float* scale, const float* zero_point, float scale_value,
                             float zp_value, int ch_mode, void* out, int out_dtype, void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!qv || !out) return fail(LQ_ERR_DEVICE, "lq_dequantize: null pointer");
  QParamRef q;
  int rc = make_params(scale, zero_point, scale_value, zp_value, ch_mode, &q);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
#define LQ_D(IN, OUT) return launch_affine<Op::kDequantize, IN, OUT>(qv, out, nullptr, rows, cols, q, 0, 0, st)
  if (out_dtype == LQ_F32) {
    if (q_dtype == LQ_S8) LQ_D(int8_t, float);
    if (q_dtype == LQ_U8) LQ_D(uint8_t, float);
    if (q_dtype == LQ_S16) LQ_D(int16_t, float);
  } else if (out_dtype == LQ_BF16) {
    if (q_dtype == LQ_S8) LQ_D(int8_t, __nv_bfloat16);
    if (q_dtype == LQ_U8) LQ_D(uint8_t, __nv_bfloat16);
    if (q_dtype == LQ_S16) LQ_D(int16_t, __nv_bfloat16);
  }
#undef LQ_D
  return fail(LQ_ERR_DTYPE, "lq_dequantize: q_dtype must be s8|u8|s16 and out_dtype f32|bf16");
}

extern "C" int lq_fake_quantize(const float* x, size_t rows, size_t cols, const float* scale,
                                const float* zero_point, float scale_value, float zp_value,
                                int ch_mode, int qmin, int qmax, float* out, float* mask,
                                void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!x || !out) return fail(LQ_ERR_DEVICE, "lq_fake_quantize: null pointer");
  QParamRef q;
  int rc = make_params(scale, zero_point, scale_value, zp_value, ch_mode, &q);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (mask)
    return launch_affine<Op::kFakeQuantize, float, float, true>(x, out, mask, rows, cols, q, qmin, qmax, st);
  return launch_affine<Op::kFakeQuantize, float, float, false>(x, out, nullptr, rows, cols, q, qmin, qmax, st);
}

extern "C" int lq_quantize_per_token(const void* x, int in_dtype, size_t rows, size_t cols,
                                     int qmin, int qmax, float eps, int8_t* out, float* out_scale,
                                     void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!x || !out || !out_scale) return fail(LQ_ERR_DEVICE, "lq_quantize_per_token: null pointer");
  if (qmax <= qmin || qmin < -128 || qmax > 127)
    return fail(LQ_ERR_SHAPE, "lq_quantize_per_token: grid must lie inside int8");
  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  const bool vec_ok = aligned16(x) && aligned16(out) && ((cols * esz) % 16 == 0) && (cols % 16 == 0);
  const float half = (float)((double)(qmax - qmin) / 2.0);
  const int grid = (int)(rows < row_grid_cap() ? rows : row_grid_cap());
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16)
    return fail(LQ_ERR_DTYPE, "lq_quantize_per_token: in_dtype must be f32|bf16");
  const size_t row_bytes = cols * esz;
  constexpr size_t kRowRing = 96 * 1024;
  const StreamKnobs& kn = stream_knobs();
  if (vec_ok && row_bytes >= (size_t)kn.token_pipe_min_row && row_bytes <= kRowRing && rows * row_bytes >= pipe_min_bytes()) {
    // rows held in shared memory: one HBM read per element, rows prefetched through the ring.
    // Measured on B200 (4096 x 8192 bf16): resident CTAs matter more than ring depth -- 6 stages
    // at 2 CTAs/SM 28.2 us, 3 stages at 4 CTAs/SM 24.0 us, 2 stages at 6 CTAs/SM 22.3 us (the
    // register-staged kernel: 24.1 us) -- so the ring holds two rows, or `LQ_TOKEN_RING_KB`.
    size_t ring = kn.token_ring_kb > 0 ? (size_t)kn.token_ring_kb * 1024 : 2 * row_bytes;
    if (ring < row_bytes) ring = row_bytes;
    if (ring > kRowRing) ring = kRowRing;
    int stages = (int)(ring / row_bytes);
    if (stages > 8) stages = 8;
    const size_t smem = kRingHeader + (size_t)stages * row_bytes;
    static PerDeviceOnce once;
    const cudaError_t attr = once.run([&] {
      const cudaError_t a32 = enable_ring(per_token_pipe_kernel<float>, kRingHeader + kRowRing);
      return a32 != cudaSuccess ? a32 : enable_ring(per_token_pipe_kernel<__nv_bfloat16>, kRingHeader + kRowRing);
    });
    if (attr != cudaSuccess) return check_cuda(attr, "cudaFuncSetAttribute(ring)");
    int ctas_per_sm = (int)((200 * 1024) / smem);
    if (ctas_per_sm > 8) ctas_per_sm = 8;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    const size_t cap = (size_t)sm_count() * ctas_per_sm;
    const int pgrid = (int)(rows < cap ? rows : cap);
    if (in_dtype == LQ_F32)
      return check_cuda(launch_pdl(per_token_pipe_kernel<float>, dim3(pgrid), dim3(kThreads), smem, st, (const float*)x, rows,
                                   cols, half, eps, (float)qmin, (float)qmax, out, out_scale, stages),
                        "lq_quantize_per_token launch");
    else
      return check_cuda(launch_pdl(per_token_pipe_kernel<__nv_bfloat16>, dim3(pgrid), dim3(kThreads), smem, st,
                                   (const __nv_bfloat16*)x, rows, cols, half, eps, (float)qmin, (float)qmax, out, out_scale,
                                   stages), "lq_quantize_per_token launch");
    return check_cuda(cudaGetLastError(), "lq_quantize_per_token launch");
  }
  if (vec_ok && row_bytes <= 16 * 1024) {
    // one row per CTA-iteration, held in registers; narrow CTAs (more rows in flight per SM)
    // when LQ_TOKEN_REG_THREADS=128
    const int t = kn.token_reg_threads;
    const size_t cap = (size_t)sm_count() * (t == 128 ? 6 : 4);
    const int rgrid = (int)(rows < cap ? rows : cap);
#define LQ_LAUNCH_REG(T, KT, KV, MB) \
  return check_cuda(launch_pdl(per_token_reg_kernel<T, KT, KV, MB>, dim3(rgrid), dim3(KT), 0, st, (const T*)x, rows, cols, \
                               half, eps, (float)qmin, (float)qmax, out, out_scale), "lq_quantize_per_token launch")
    if (in_dtype == LQ_F32) {
      if (t == 128) LQ_LAUNCH_REG(float, 128, 8, 6);
      else LQ_LAUNCH_REG(float, 256, 4, 4);
    } else {
      if (t == 128) LQ_LAUNCH_REG(__nv_bfloat16, 128, 8, 6);
      else LQ_LAUNCH_REG(__nv_bfloat16, 256, 4, 4);
    }
#undef LQ_LAUNCH_REG
    return check_cuda(cudaGetLastError(), "lq_quantize_per_token launch");
  }
  if (in_dtype == LQ_F32)
    per_token_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, vec_ok, half, eps, (float)qmin, (float)qmax, out, out_scale);
  else if (in_dtype == LQ_BF16)
    per_token_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, vec_ok, half, eps, (float)qmin, (float)qmax, out, out_scale);
  else
    return fail(LQ_ERR_DTYPE, "lq_quantize_per_token: in_dtype must be f32|bf16");
  return check_cuda(cudaGetLastError(), "lq_quantize_per_token launch");
}

extern "C" int lq_rowsum_s8(const int8_t* b, size_t N, size_t K, int32_t* out, void* stream) {
  if (N == 0) return LQ_OK;
  if (!b || !out) return fail(LQ_ERR_DEVICE, "lq_rowsum_s8: null pointer");
  const bool vec_ok = aligned16(b) && (K % 16 == 0);
  rowsum_kernel<<<grid_for(N * 32), kThreads, 0, (cudaStream_t)stream>>>(b, N, K, vec_ok, out);
  return check_cuda(cudaGetLastError(), "lq_rowsum_s8 launch");
}

// ---- allocation-free variant of the per-tensor range reduction -------------------------------
//
// Some callers must not allocate device memory at the point where they need a range: code
// running inside a memory-pool or arena owner that forbids nested allocation, a real-time
// serving thread that may not take the allocator lock, or a host written in another language
// that binds only this C ABI and has no device allocator of its own.  For them the scratch
// of the reduction (one partial min/max pair per CTA and the arrival counter) lives in a
// fixed array inside the library image instead of a caller-supplied workspace.
namespace lq {
namespace {
constexpr size_t kNoAllocMaxElems = size_t(1) << 30;  // 2^30 elements per call
static __device__ __align__(256) unsigned char g_minmax_scratch[sizeof(MinMaxWorkspace)];
std::mutex g_scratch_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device.  In host code the array's name
// is only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device with that device current.
int scratch_address(void** out) {
  int dev = 0;
  LQ_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(LQ_ERR_UNSUPPORTED, "lq_minmax_noalloc: device index out of range");
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    LQ_CUDA(cudaGetSymbolAddress(&p, g_minmax_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return LQ_OK;
}
}  // namespace
}  // namespace lq

extern "C" size_t lq_minmax_noalloc_max_elems(void) { return lq::kNoAllocMaxElems; }

extern "C" int lq_minmax_noalloc(const void* x, int in_dtype, size_t n, float* out_min,
                                 float* out_max, void* stream) {
  if (!x || !out_min || !out_max) return fail(LQ_ERR_DEVICE, "lq_minmax_noalloc: null pointer");
  if (n == 0) return fail(LQ_ERR_SHAPE, "lq_minmax_noalloc: empty input has no min/max");
  if (n > kNoAllocMaxElems)
    return fail(LQ_ERR_SHAPE, "lq_minmax_noalloc: " + std::to_string(n) + " elements exceed the built-in scratch's limit of " +
                                  std::to_string(kNoAllocMaxElems) + " per call; use lq_minmax with a workspace");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_minmax_noalloc: in_dtype");
  void* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc != LQ_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps whatever the previous call left: re-arm the arrival counter
  LQ_CUDA(cudaMemsetAsync(scratch, 0, 16, st));
  return minmax_tensor_launch(x, in_dtype, n, (MinMaxWorkspace*)scratch, out_min, out_max, FusedQParams{}, st);
}

// Dynamic per-tensor encode in one call: range reduction -> qparams -> codes (three launches,
// no host round trip; scale and zero point stay on the device for the GEMM epilogue).
extern "C" int lq_quantize_dynamic(const void* x, int in_dtype, size_t rows, size_t cols, int symmetric,
                                   int is_signed, int qmin, int qmax, float eps, void* workspace,
                                   size_t workspace_bytes, void* out, int out_dtype, float* out_scale,
                                   float* out_zp, float* out_minmax, void* stream) {
  if (rows == 0 || cols == 0) return fail(LQ_ERR_SHAPE, "lq_quantize_dynamic: empty input has no range");
  if (!out_scale || !out_zp || !out_minmax) return fail(LQ_ERR_DEVICE, "lq_quantize_dynamic: null pointer");
  if (!x) return fail(LQ_ERR_DEVICE, "lq_quantize_dynamic: null pointer");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_quantize_dynamic: in_dtype");
  if (qmax <= qmin) return fail(LQ_ERR_SHAPE, "lq_quantize_dynamic: qmax must exceed qmin");
  if (!workspace) return fail(LQ_ERR_DEVICE, "lq_quantize_dynamic: needs the range-reduction workspace");
  if (workspace_bytes < sizeof(MinMaxWorkspace))
    return fail(LQ_ERR_WORKSPACE, "lq_quantize_dynamic: workspace smaller than lq_minmax_workspace_bytes()");
  if (!aligned16(workspace)) return fail(LQ_ERR_ALIGNMENT, "lq_quantize_dynamic: workspace alignment");
  // two launches: the range reduction, whose last CTA also derives (scale, zero_point), and the encode
  FusedQParams fq;
  fq.scale = out_scale, fq.zp = out_zp, fq.symmetric = symmetric, fq.is_signed = is_signed;
  fq.qmin = qmin, fq.qmax = qmax, fq.eps = eps;
  int rc = minmax_tensor_launch(x, in_dtype, rows * cols, (MinMaxWorkspace*)workspace, out_minmax, out_minmax + 1, fq,
                                (cudaStream_t)stream);
  if (rc != LQ_OK) return rc;
  return lq_quantize(x, in_dtype, rows, cols, out_scale, out_zp, 0.0f, 0.0f, LQ_PER_TENSOR, qmin, qmax, out,
                     out_dtype, stream);
}

// ---- element-wise merges and table-driven activations of the quantized region -------------------
// QFunctional (lucid/nn/quantized/functional_module.py:230-258) snaps x + y, x * y, relu(x + y),
// x + c, x * c or x itself (the pieces of a cat) to one calibrated grid.  The reference does it on
// float32 tensors that carry int8 numerics (three passes: the op, the activation, fake_quantize);
// here the operands may arrive as their 8-bit codes (1 byte per element instead of 4), the
// dequantize / op / activation / encode chain runs in registers with the reference's float32
// operation order, and the result leaves as codes, as the fake-quantized float32, or both.
namespace lq {

struct MergeOperand {
  const void* p;   // nullptr: the scalar
  int dtype;
  const float* s;  // nullptr: p holds values, not codes
  const float* z;
  float scalar;
};

__device__ __forceinline__ void merge_load4(const MergeOperand& o, size_t e, float (&v)[4]) {
  switch (o.dtype) {
    case LQ_F32: Quad<float>::load((const float*)o.p + e, v); break;
    case LQ_BF16: Quad<__nv_bfloat16>::load((const __nv_bfloat16*)o.p + e, v); break;
    case LQ_S8: Quad<int8_t>::load((const int8_t*)o.p + e, v); break;
    case LQ_U8: Quad<uint8_t>::load((const uint8_t*)o.p + e, v); break;
    default: Quad<int16_t>::load((const int16_t*)o.p + e, v); break;
  }
}
__device__ __forceinline__ float merge_load1(const MergeOperand& o, size_t e) {
  switch (o.dtype) {
    case LQ_F32: return ((const float*)o.p)[e];
    case LQ_BF16: return __bfloat162float(((const __nv_bfloat16*)o.p)[e]);
    case LQ_S8: return (float)((const int8_t*)o.p)[e];
    case LQ_U8: return (float)((const uint8_t*)o.p)[e];
    default: return (float)((const int16_t*)o.p)[e];
  }
}
__device__ __forceinline__ float merge_op(int op, float a, float b) {
  switch (op) {
    case LQ_MERGE_ADD: return __fadd_rn(a, b);
    case LQ_MERGE_MUL: return __fmul_rn(a, b);
    case LQ_MERGE_ADD_RELU: {
      const float t = __fadd_rn(a, b);
      return t > 0.0f ? t : 0.0f;
    }
    default: return a;  // LQ_MERGE_COPY
  }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads, 4)
merge_kernel(int op, MergeOperand x, MergeOperand y, size_t n, const float* __restrict__ out_scale,
             const float* __restrict__ out_zp, float qmin, float qmax, void* __restrict__ codes, int codes_dtype,
             float* __restrict__ out_f32) {
  const float S = __ldg(out_scale), Z = __ldg(out_zp);
  const Divisor d = make_divisor(S);
  const float sx = x.s ? __ldg(x.s) : 1.0f, zx = x.s ? __ldg(x.z) : 0.0f;
  const float sy = y.s ? __ldg(y.s) : 1.0f, zy = y.s ? __ldg(y.z) : 0.0f;
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (VEC) {
    for (size_t g = first; g < n / 4; g += stride) {
      float a[4], b[4], t[4], c[4];
      merge_load4(x, g * 4, a);
      if (y.p) merge_load4(y, g * 4, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (x.s) a[i] = __fmul_rn(__fsub_rn(a[i], zx), sx);
        if (!y.p) b[i] = y.scalar;
        else if (y.s) b[i] = __fmul_rn(__fsub_rn(b[i], zy), sy);
        t[i] = merge_op(op, a[i], b[i]);
      }
      code4_f32(t, d, Z, qmin, qmax, c);
      if (codes) {
        if (codes_dtype == LQ_S8) Quad<int8_t>::store((int8_t*)codes + g * 4, c);
        else if (codes_dtype == LQ_U8) Quad<uint8_t>::store((uint8_t*)codes + g * 4, c);
        else Quad<int16_t>::store((int16_t*)codes + g * 4, c);
      }
      if (out_f32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = __fmul_rn(__fsub_rn(c[i], Z), S);
        Quad<float>::store(out_f32 + g * 4, c);
      }
    }
  }
  for (size_t e = (VEC ? (n / 4) * 4 : 0) + first; e < n; e += stride) {
    float a = merge_load1(x, e);
    if (x.s) a = __fmul_rn(__fsub_rn(a, zx), sx);
    float b = y.scalar;
    if (y.p) {
      b = merge_load1(y, e);
      if (y.s) b = __fmul_rn(__fsub_rn(b, zy), sy);
    }
    const float c = code_f32(merge_op(op, a, b), d, Z, qmin, qmax);
    if (codes) {
      if (codes_dtype == LQ_S8) ((int8_t*)codes)[e] = (int8_t)(int)c;
      else if (codes_dtype == LQ_U8) ((uint8_t*)codes)[e] = (uint8_t)(int)c;
      else ((int16_t*)codes)[e] = (int16_t)(int)c;
    }
    if (out_f32) out_f32[e] = __fmul_rn(__fsub_rn(c, Z), S);
  }
}

// out[i] = table[in[i]]: a unary function of 8-bit codes is 256 bytes of table.  16 codes per
// 16-byte load, looked up in a shared-memory copy of the table.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
lut_kernel(const uint8_t* __restrict__ in, size_t n, const uint8_t* __restrict__ table, uint8_t* __restrict__ out) {
  __shared__ __align__(16) uint8_t t[256];
  t[threadIdx.x] = table[threadIdx.x];  // kThreads == 256
  __syncthreads();
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (VEC) {
    for (size_t g = first; g < n / 16; g += stride) {
      const uint4 u = ld_stream_u4(in + g * 16);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint32_t r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        r[j] = (uint32_t)t[w[j] & 0xffu] | ((uint32_t)t[(w[j] >> 8) & 0xffu] << 8) |
               ((uint32_t)t[(w[j] >> 16) & 0xffu] << 16) | ((uint32_t)t[w[j] >> 24] << 24);
      st_stream_u4(out + g * 16, make_uint4(r[0], r[1], r[2], r[3]));
    }
  }
  for (size_t e = (VEC ? (n / 16) * 16 : 0) + first; e < n; e += stride) out[e] = t[in[e]];
}

static bool merge_dtype_ok(int dt, bool codes) {
  return codes ? (dt == LQ_S8 || dt == LQ_U8 || dt == LQ_S16) : (dt == LQ_F32 || dt == LQ_BF16);
}
static size_t merge_elem_size(int dt) { return dt == LQ_F32 ? 4 : (dt == LQ_BF16 || dt == LQ_S16) ? 2 : 1; }

}  // namespace lq

extern "C" int lq_qmerge(int op, const void* x, int x_dtype, const float* x_scale, const float* x_zp,
                         const void* y, int y_dtype, const float* y_scale, const float* y_zp, float y_scalar,
                         size_t n, const float* out_scale, const float* out_zp, int qmin, int qmax,
                         void* out_codes, int codes_dtype, float* out_f32, void* stream) {
  if (n == 0) return LQ_OK;
  if (op < LQ_MERGE_ADD || op > LQ_MERGE_COPY) return fail(LQ_ERR_UNSUPPORTED, "lq_qmerge: unknown op");
  if (!x || !out_scale || !out_zp) return fail(LQ_ERR_DEVICE, "lq_qmerge: null pointer");
  if (!out_codes && !out_f32) return fail(LQ_ERR_DEVICE, "lq_qmerge: no output requested");
  if ((x_scale == nullptr) != (x_zp == nullptr) || (y_scale == nullptr) != (y_zp == nullptr))
    return fail(LQ_ERR_DEVICE, "lq_qmerge: scale and zero_point of an operand go together");
  if (!merge_dtype_ok(x_dtype, x_scale != nullptr)) return fail(LQ_ERR_DTYPE, "lq_qmerge: x dtype");
  if (y && !merge_dtype_ok(y_dtype, y_scale != nullptr)) return fail(LQ_ERR_DTYPE, "lq_qmerge: y dtype");
  if (out_codes && !merge_dtype_ok(codes_dtype, true)) return fail(LQ_ERR_DTYPE, "lq_qmerge: codes dtype");
  if (qmin > qmax) return fail(LQ_ERR_SHAPE, "lq_qmerge: qmin > qmax");
  const MergeOperand mx{x, x_dtype, x_scale, x_zp, 0.0f};
  const MergeOperand my{y, y ? y_dtype : LQ_F32, y ? y_scale : nullptr, y ? y_zp : nullptr, y_scalar};
  auto al = [](const void* p, size_t esz) { return p == nullptr || ((uintptr_t)p % (4 * esz)) == 0; };
  const bool vec = n >= 4 && al(x, merge_elem_size(x_dtype)) && al(y, merge_elem_size(my.dtype)) &&
                   al(out_codes, merge_elem_size(codes_dtype)) && al(out_f32, 4);
  const int grid = grid_for(vec ? n / 4 : n, 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (vec)
    merge_kernel<true><<<grid, kThreads, 0, st>>>(op, mx, my, n, out_scale, out_zp, (float)qmin, (float)qmax,
                                                  out_codes, codes_dtype, out_f32);
  else
    merge_kernel<false><<<grid, kThreads, 0, st>>>(op, mx, my, n, out_scale, out_zp, (float)qmin, (float)qmax,
                                                   out_codes, codes_dtype, out_f32);
  return check_cuda(cudaGetLastError(), "lq_qmerge launch");
}

extern "C" int lq_lut_u8(const void* in_codes, size_t n, const uint8_t* table, void* out_codes, void* stream) {
  if (n == 0) return LQ_OK;
  if (!in_codes || !table || !out_codes) return fail(LQ_ERR_DEVICE, "lq_lut_u8: null pointer");
  const bool vec = n >= 16 && aligned16(in_codes) && aligned16(out_codes);
  const int grid = grid_for(vec ? n / 16 : n, 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (vec)
    lut_kernel<true><<<grid, kThreads, 0, st>>>((const uint8_t*)in_codes, n, table, (uint8_t*)out_codes);
  else
    lut_kernel<false><<<grid, kThreads, 0, st>>>((const uint8_t*)in_codes, n, table, (uint8_t*)out_codes);
  return check_cuda(cudaGetLastError(), "lq_lut_u8 launch");
}

// out[i] = table[x[i] * 256 + y[i]]: a binary function of two 8-bit codes is 64 KB of table,
// which fits in shared memory.  The exact merge (two decodes, the op, an IEEE division, round,
// clip: about twenty dependent float instructions per element) becomes one byte permute, one
// shared load and one insert; the caller fills the table by running lq_qmerge once over the
// 65536 code pairs of its grids.
namespace lq {
constexpr int kLut2Bytes = 65536;

__global__ void __launch_bounds__(kThreads)
lut2_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ y, size_t n, const uint8_t* __restrict__ table,
            uint8_t* __restrict__ out, float* __restrict__ out_f32, const float* __restrict__ out_scale,
            const float* __restrict__ out_zp, int out_signed, bool vec) {
  extern __shared__ __align__(16) uint8_t t2[];
  for (int i = threadIdx.x; i < kLut2Bytes / 16; i += kThreads)
    reinterpret_cast<uint4*>(t2)[i] = __ldg(reinterpret_cast<const uint4*>(table) + i);
  __syncthreads();
  const float S = out_f32 ? __ldg(out_scale) : 1.0f, Z = out_f32 ? __ldg(out_zp) : 0.0f;
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const size_t nvec = vec ? n / 16 : 0;
  for (size_t g = first; g < nvec; g += stride) {
    const uint4 a = ld_stream_u4(x + g * 16), b = ld_stream_u4(y + g * 16);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // index = x byte in bits 8-15, y byte in bits 0-7; one byte permute interleaves two pairs
      const uint32_t lo = __byte_perm(bw[j], aw[j], 0x5140), hi = __byte_perm(bw[j], aw[j], 0x7362);
      r[j] = (uint32_t)t2[lo & 0xffffu] | ((uint32_t)t2[lo >> 16] << 8) | ((uint32_t)t2[hi & 0xffffu] << 16) |
             ((uint32_t)t2[hi >> 16] << 24);
    }
    st_stream_u4(out + g * 16, make_uint4(r[0], r[1], r[2], r[3]));
    if (out_f32) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t byte = (r[j] >> (8 * k)) & 0xffu;
          const float c = out_signed ? (float)(int8_t)byte : (float)byte;
          v[k] = __fmul_rn(__fsub_rn(c, Z), S);
        }
        Quad<float>::store(out_f32 + g * 16 + j * 4, v);
      }
    }
  }
  for (size_t e = nvec * 16 + first; e < n; e += stride) {
    const uint8_t c = t2[((uint32_t)x[e] << 8) | y[e]];
    out[e] = c;
    if (out_f32) out_f32[e] = __fmul_rn(__fsub_rn(out_signed ? (float)(int8_t)c : (float)c, Z), S);
  }
}
}  // namespace lq

extern "C" int lq_lut2_u8(const void* x_codes, const void* y_codes, size_t n, const uint8_t* table,
                          void* out_codes, float* out_f32, const float* out_scale, const float* out_zp,
                          int out_signed, void* stream) {
  if (n == 0) return LQ_OK;
  if (!x_codes || !y_codes || !table || !out_codes) return fail(LQ_ERR_DEVICE, "lq_lut2_u8: null pointer");
  if (out_f32 && (!out_scale || !out_zp)) return fail(LQ_ERR_DEVICE, "lq_lut2_u8: out_f32 needs the output grid");
  if (!aligned16(table)) return fail(LQ_ERR_ALIGNMENT, "lq_lut2_u8: the table must be 16-byte aligned");
  static PerDeviceOnce once;
  const cudaError_t attr = once.run([&] {
    return cudaFuncSetAttribute(lut2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLut2Bytes);
  });
  if (attr != cudaSuccess) return check_cuda(attr, "cudaFuncSetAttribute(lut2)");
  const bool vec = n >= 16 && aligned16(x_codes) && aligned16(y_codes) && aligned16(out_codes) &&
                   (!out_f32 || aligned16(out_f32));
  // persistent CTAs, three per SM (3 x 64 KB of tables); small inputs take fewer
  const size_t want = ((vec ? n / 16 : n) + kThreads - 1) / kThreads;
  const size_t lcap = (size_t)sm_count() * 3;
  const int grid = (int)(want < lcap ? (want ? want : 1) : lcap);
  lut2_kernel<<<grid, kThreads, kLut2Bytes, (cudaStream_t)stream>>>(
      (const uint8_t*)x_codes, (const uint8_t*)y_codes, n, table, (uint8_t*)out_codes, out_f32, out_scale, out_zp,
      out_signed, vec);
  return check_cuda(cudaGetLastError(), "lq_lut2_u8 launch");
}

// ---- per-token encode of a column shard, stored into every rank's operand buffer ----------------
// Output-channel-sharded layers: when a sharded GEMM's output only feeds the per-token int8
// encode of the next layer, exchanging it as bf16 and encoding the whole tensor on every rank
// moves twice the bytes and repeats the encode w times.  Instead each rank reduces the per-token
// abs-max of its own column shard, the ranks all-reduce those (max is order-free, so the scales
// equal the single-GPU ones bit for bit), and this kernel encodes the rank's shard with the
// global scales and stores the CODES into the column slice of every rank's (rows, ldo) buffer:
// its own and, with plain peer stores over NVLink, the peers'.
namespace lq {
struct BcastDst {
  int8_t* p[8];
};

template <typename In>
__global__ void __launch_bounds__(kThreads)
quantize_rows_bcast_kernel(const In* __restrict__ x, size_t rows, size_t cols, size_t ldx,
                           const float* __restrict__ row_absmax, int absmax_parts, size_t absmax_stride,
                           float half, float eps, float qmin, float qmax,
                           BcastDst dst, int n_dst, bool multicast, size_t ldo, size_t col0,
                           float* __restrict__ out_scale) {
  constexpr int E = VecOf<In>::kElems;  // 4 (binary32) or 8 (bfloat16) elements per 16-byte vector
  const uint32_t nvec = (uint32_t)(cols / E);
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    // the same expressions as the single-GPU per-token encode
    // (max over the shards' maxima: order-free, so the value is the unsharded row's abs-max)
    float am = __ldcg(row_absmax + r);
    for (int p = 1; p < absmax_parts; ++p) am = fmaxf(am, __ldcg(row_absmax + p * absmax_stride + r));
    const float sc = fmaxf(__fdiv_rn(am, half), eps);
    if (threadIdx.x == 0 && out_scale) out_scale[r] = sc;
    const Divisor d = make_divisor(sc);
    const IntGrid ig = make_int_grid(0.0f, qmin, qmax, -128, 127);
    const uint4* xv = reinterpret_cast<const uint4*>(x + r * ldx);
    const size_t obase = r * ldo + col0;
    for (uint32_t i = threadIdx.x; i < nvec; i += kThreads) {
      const uint4 v = ld_stream_u4(xv + i);
      const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
      if (E == 4) {
        const float f[4] = {__uint_as_float(wv[0]), __uint_as_float(wv[1]), __uint_as_float(wv[2]), __uint_as_float(wv[3])};
        int c[4];
        code4_int(f, d, ig, 0.0f, qmin, qmax, c);
        const uint32_t w = pack4i_s8(c);
        if (multicast)
          asm volatile("multimem.st.weak.global.b32 [%0], %1;" ::"l"(dst.p[0] + obase + (size_t)i * 4), "r"(w) : "memory");
        else
          for (int k = 0; k < n_dst; ++k) *reinterpret_cast<uint32_t*>(dst.p[k] + obase + (size_t)i * 4) = w;
      } else {
        const float f0[4] = {bf16_bits_to_f32(wv[0] & 0xffffu), bf16_bits_to_f32(wv[0] >> 16),
                             bf16_bits_to_f32(wv[1] & 0xffffu), bf16_bits_to_f32(wv[1] >> 16)};
        const float f1[4] = {bf16_bits_to_f32(wv[2] & 0xffffu), bf16_bits_to_f32(wv[2] >> 16),
                             bf16_bits_to_f32(wv[3] & 0xffffu), bf16_bits_to_f32(wv[3] >> 16)};
        int c0[4], c1[4];
        code4_int(f0, d, ig, 0.0f, qmin, qmax, c0);
        code4_int(f1, d, ig, 0.0f, qmin, qmax, c1);
        const uint2 w = make_uint2(pack4i_s8(c0), pack4i_s8(c1));
        if (multicast)
          asm volatile("multimem.st.weak.global.b64 [%0], %1;" ::"l"(dst.p[0] + obase + (size_t)i * 8),
                       "l"((unsigned long long)w.x | ((unsigned long long)w.y << 32)) : "memory");
        else
          for (int k = 0; k < n_dst; ++k) *reinterpret_cast<uint2*>(dst.p[k] + obase + (size_t)i * 8) = w;
      }
    }
  }
}
}  // namespace lq

extern "C" int lq_quantize_rows_bcast(const void* x, int in_dtype, size_t rows, size_t cols, size_t ldx,
                                      const float* row_absmax, int absmax_parts, size_t absmax_stride,
                                      int qmin, int qmax, float eps,
                                      void* const* outs, int n_dst, size_t ldo, size_t col0,
                                      float* out_scale, void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!x || !row_absmax || !outs) return fail(LQ_ERR_DEVICE, "lq_quantize_rows_bcast: null pointer");
  // n_dst == -1: outs[0] is an NVSwitch multicast address (one multimem store reaches every rank)
  const bool multicast = n_dst == -1;
  if (multicast) n_dst = 1;
  if (n_dst < 1 || n_dst > 8) return fail(LQ_ERR_SHAPE, "lq_quantize_rows_bcast: 1..8 destinations (or -1: multicast)");
  if (absmax_parts < 1 || absmax_parts > 64 || (absmax_parts > 1 && absmax_stride < rows))
    return fail(LQ_ERR_SHAPE, "lq_quantize_rows_bcast: abs-max parts / stride");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_quantize_rows_bcast: in_dtype");
  if (qmin < -128 || qmax > 127 || qmin >= qmax) return fail(LQ_ERR_SHAPE, "lq_quantize_rows_bcast: grid outside int8");
  const size_t e = in_dtype == LQ_F32 ? 4 : 8;
  if (cols % e || ldx % e || !aligned16(x) || ldo % 8 || col0 % 8 || ldo < col0 + cols)
    return fail(LQ_ERR_ALIGNMENT, "lq_quantize_rows_bcast: shard and destination must be vector aligned");
  BcastDst dst{};
  for (int k = 0; k < n_dst; ++k) {
    if (!outs[k] || (reinterpret_cast<uintptr_t>(outs[k]) & 7u)) return fail(LQ_ERR_ALIGNMENT, "lq_quantize_rows_bcast: destination pointer");
    dst.p[k] = (int8_t*)outs[k];
  }
  const float half = (float)((qmax - qmin) / 2.0);
  const int grid = (int)(rows < row_grid_cap() ? rows : row_grid_cap());
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == LQ_F32)
    quantize_rows_bcast_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, ldx, row_absmax, absmax_parts,
                                                                 absmax_stride, half, eps, (float)qmin, (float)qmax, dst, n_dst,
                                                                 multicast, ldo, col0, out_scale);
  else
    quantize_rows_bcast_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, ldx,
                                                                         row_absmax, absmax_parts, absmax_stride, half, eps,
                                                                         (float)qmin, (float)qmax, dst, n_dst, multicast, ldo,
                                                                         col0, out_scale);
  return check_cuda(cudaGetLastError(), "lq_quantize_rows_bcast launch");
}

// ---- pieces of the exchange that are not a GEMM ------------------------------------------------
namespace lq {
struct FloatDst {
  float* p[8];
};

// Per-row abs-max of this rank's column shard, stored into slot `slot0 + r` of every rank's
// (parts, rows) table: the max all-reduce of the sharded per-token encode as plain peer stores.
template <typename In>
__global__ void __launch_bounds__(kThreads)
absmax_rows_bcast_kernel(const In* __restrict__ x, size_t rows, size_t cols, size_t ldx, bool vec_ok,
                         FloatDst dst, int n_dst, size_t slot0) {
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float mn = 0.0f, mx = 0.0f;  // the range is extended to include 0 anyway
    minmax_accumulate(x + r * ldx, cols, threadIdx.x, kThreads, vec_ok, mn, mx);
    block_minmax(mn, mx);
    if (threadIdx.x < n_dst) dst.p[threadIdx.x][slot0 + r] = fmaxf(fabsf(mn), fabsf(mx));
  }
}

// Per-token encode of a ROW shard with the exchange fused in: this rank encodes its rows of a
// replicated activation (abs-max, scale, codes: the expressions of lq_quantize_per_token) and
// stores codes and scales at rows [row0, row0 + rows) of every rank's buffers.
template <typename In>
__global__ void __launch_bounds__(kThreads)
per_token_bcast_kernel(const In* __restrict__ x, size_t rows, size_t cols, float half, float eps, float qmin,
                       float qmax, BcastDst dst, FloatDst sdst, int n_dst, bool multicast, size_t row0) {
  constexpr int E = VecOf<In>::kElems;
  __shared__ float s_scale;
  const uint32_t nvec = (uint32_t)(cols / E);
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const In* xr = x + r * cols;
    float mn = 0.0f, mx = 0.0f;
    minmax_accumulate(xr, cols, threadIdx.x, kThreads, true, mn, mx);
    block_minmax(mn, mx);
    if (threadIdx.x == 0) s_scale = fmaxf(__fdiv_rn(fmaxf(fabsf(mn), fabsf(mx)), half), eps);
    __syncthreads();
    const float sc = s_scale;
    // every destination receives the scale with a plain store (a multicast address is used for
    // the codes only)
    if (threadIdx.x < n_dst) sdst.p[threadIdx.x][row0 + r] = sc;
    const Divisor d = make_divisor(sc);
    const IntGrid ig = make_int_grid(0.0f, qmin, qmax, -128, 127);
    const ShortDiv sd = make_short_div(d);  // |x| <= this row's abs-max: no quotient leaves its domain
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    const size_t obase = (row0 + r) * cols;
    for (uint32_t i = threadIdx.x; i < nvec; i += kThreads) {
      const uint4 v = __ldcg(xv + i);  // second read of the row: served by L2
      const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
      if (E == 4) {
        const float f[4] = {__uint_as_float(wv[0]), __uint_as_float(wv[1]), __uint_as_float(wv[2]), __uint_as_float(wv[3])};
        int c[4];
        if (d.fast) code4_short(f, sd, ig, c);
        else code4_int(f, d, ig, 0.0f, qmin, qmax, c);
        const uint32_t w = pack4i_s8(c);
        if (multicast)
          asm volatile("multimem.st.weak.global.b32 [%0], %1;" ::"l"(dst.p[0] + obase + (size_t)i * 4), "r"(w) : "memory");
        else
          for (int k = 0; k < n_dst; ++k) *reinterpret_cast<uint32_t*>(dst.p[k] + obase + (size_t)i * 4) = w;
      } else {
        const float f0[4] = {bf16_bits_to_f32(wv[0] & 0xffffu), bf16_bits_to_f32(wv[0] >> 16),
                             bf16_bits_to_f32(wv[1] & 0xffffu), bf16_bits_to_f32(wv[1] >> 16)};
        const float f1[4] = {bf16_bits_to_f32(wv[2] & 0xffffu), bf16_bits_to_f32(wv[2] >> 16),
                             bf16_bits_to_f32(wv[3] & 0xffffu), bf16_bits_to_f32(wv[3] >> 16)};
        int c0[4], c1[4];
        if (d.fast) {
          code4_short(f0, sd, ig, c0);
          code4_short(f1, sd, ig, c1);
        } else {
          code4_int(f0, d, ig, 0.0f, qmin, qmax, c0);
          code4_int(f1, d, ig, 0.0f, qmin, qmax, c1);
        }
        const uint2 w = make_uint2(pack4i_s8(c0), pack4i_s8(c1));
        if (multicast)
          asm volatile("multimem.st.weak.global.b64 [%0], %1;" ::"l"(dst.p[0] + obase + (size_t)i * 8),
                       "l"((unsigned long long)w.x | ((unsigned long long)w.y << 32)) : "memory");
        else
          for (int k = 0; k < n_dst; ++k) *reinterpret_cast<uint2*>(dst.p[k] + obase + (size_t)i * 8) = w;
      }
    }
    __syncthreads();  // s_scale is rewritten by the next row
  }
}
}  // namespace lq

extern "C" int lq_absmax_rows_bcast(const void* x, int in_dtype, size_t rows, size_t cols, size_t ldx,
                                    float* const* outs, int n_dst, size_t slot0, void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!x || !outs) return fail(LQ_ERR_DEVICE, "lq_absmax_rows_bcast: null pointer");
  if (n_dst < 1 || n_dst > 8) return fail(LQ_ERR_SHAPE, "lq_absmax_rows_bcast: 1..8 destinations");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_absmax_rows_bcast: in_dtype");
  const size_t esz = in_dtype == LQ_F32 ? 4 : 2;
  const bool vec_ok = aligned16(x) && ((cols * esz) % 16 == 0) && ((ldx * esz) % 16 == 0);
  FloatDst dst{};
  for (int k = 0; k < n_dst; ++k) {
    if (!outs[k]) return fail(LQ_ERR_DEVICE, "lq_absmax_rows_bcast: null destination");
    dst.p[k] = outs[k];
  }
  const int grid = (int)(rows < row_grid_cap() ? rows : row_grid_cap());
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == LQ_F32)
    absmax_rows_bcast_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, ldx, vec_ok, dst, n_dst, slot0);
  else
    absmax_rows_bcast_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, ldx, vec_ok, dst,
                                                                        n_dst, slot0);
  return check_cuda(cudaGetLastError(), "lq_absmax_rows_bcast launch");
}

extern "C" int lq_quantize_per_token_bcast(const void* x, int in_dtype, size_t rows, size_t cols, int qmin, int qmax,
                                           float eps, void* const* outs, float* const* scale_outs, int n_dst,
                                           void* multicast_out, size_t row0, void* stream) {
  if (rows == 0 || cols == 0) return LQ_OK;
  if (!x || !scale_outs || (!outs && !multicast_out)) return fail(LQ_ERR_DEVICE, "lq_quantize_per_token_bcast: null pointer");
  if (n_dst < 1 || n_dst > 8) return fail(LQ_ERR_SHAPE, "lq_quantize_per_token_bcast: 1..8 destinations");
  if (in_dtype != LQ_F32 && in_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_quantize_per_token_bcast: in_dtype");
  if (qmin < -128 || qmax > 127 || qmin >= qmax) return fail(LQ_ERR_SHAPE, "lq_quantize_per_token_bcast: grid outside int8");
  const size_t e = in_dtype == LQ_F32 ? 4 : 8;
  if (cols % 16 || !aligned16(x)) return fail(LQ_ERR_ALIGNMENT, "lq_quantize_per_token_bcast: cols % 16 and a 16-byte aligned input");
  (void)e;
  BcastDst dst{};
  FloatDst sdst{};
  for (int k = 0; k < n_dst; ++k) {
    if (!scale_outs[k]) return fail(LQ_ERR_DEVICE, "lq_quantize_per_token_bcast: null scale destination");
    sdst.p[k] = scale_outs[k];
    if (!multicast_out) {
      if (!outs[k] || (reinterpret_cast<uintptr_t>(outs[k]) & 7u)) return fail(LQ_ERR_ALIGNMENT, "lq_quantize_per_token_bcast: destination pointer");
      dst.p[k] = (int8_t*)outs[k];
    }
  }
  if (multicast_out) {
    if (reinterpret_cast<uintptr_t>(multicast_out) & 7u) return fail(LQ_ERR_ALIGNMENT, "lq_quantize_per_token_bcast: multicast address");
    dst.p[0] = (int8_t*)multicast_out;
  }
  const float half = (float)((qmax - qmin) / 2.0);
  const int grid = (int)(rows < row_grid_cap() ? rows : row_grid_cap());
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == LQ_F32)
    per_token_bcast_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, half, eps, (float)qmin, (float)qmax,
                                                             dst, sdst, n_dst, multicast_out != nullptr, row0);
  else
    per_token_bcast_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, half, eps,
                                                                     (float)qmin, (float)qmax, dst, sdst, n_dst,
                                                                     multicast_out != nullptr, row0);
  return check_cuda(cudaGetLastError(), "lq_quantize_per_token_bcast launch");
}
