// Shared helpers for the lucid_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

#include "lucid_b200.h"

namespace lq {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs (sizes static tables; grids ask sm_count())
constexpr int kMaxDevices = 64;

// ---- host-side error plumbing -------------------------------------------
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int check_cuda(cudaError_t e, const char* what);

#define LQ_CUDA(expr)                                   \
  do {                                                  \
    int _rc = ::lq::check_cuda((expr), #expr);          \
    if (_rc != LQ_OK) return _rc;                       \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Index of the current device, or -1.
int current_device();
// Multiprocessor count of the current device (asked once per device).
int sm_count();

// Per-device one-time set-up at a call site.  Function attributes (the opt-in to more than
// 48 KB of dynamic shared memory) and occupancy answers belong to a device, not to the process:
// a process that drives a second GPU has to repeat them there.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[kMaxDevices] = {};
  cudaError_t err[kMaxDevices] = {};
  template <typename F>
  cudaError_t run(F&& fn) {
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
      err[dev] = fn();
      done[dev] = true;
    }
    return err[dev];
  }
};

// ---- programmatic dependent launch ------------------------------------------------------
// Kernels launched through launch_pdl() may become resident while the kernel before them in
// the stream is still draining: their CTAs run their set-up (barrier initialisation, TMEM
// allocation, parameter derivation from kernel arguments), then pdl_wait() holds them until
// that kernel has completed and its writes are visible.  Such a kernel must execute pdl_wait()
// on every thread before its first access to global memory; pdl_launch_dependents() right after
// lets the kernel behind it do the same.  After a kernel that does not take part (or with
// LQ_PDL=0) the launch is an ordinary one and both calls are no-ops.
bool pdl_enabled();
void reload_pdl_knob();
template <typename... P, typename... A>
cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at, cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// ---- device-side exact arithmetic ---------------------------------------
// Every step is a separate IEEE binary32 operation; the intrinsics keep the
// compiler from contracting or approximating them.

// Correctly rounded x / s with the divisor's reciprocal hoisted out of the element loop.
// q0 = RN(x * y) with y = RN(1 / s) is within 1.5 ulp of x / s; two residual corrections
// (r = x - s*q exactly, by FMA; q += r*y) give the correctly rounded quotient (Markstein), the
// same value `__fdiv_rn` returns.  The short form is used only where no intermediate can
// overflow or lose bits to underflow: |s| in [2^-60, 2^60] and |q| < 2^24; everything else
// (huge quotients, denormal or huge scales, inf / NaN) takes the full-range division.
struct Divisor {
  float s, y;
  bool fast;
};
// Full-range IEEE division, kept out of line: it is the rare path, and inlining its
// expansion at every element bloats the hot loops past the instruction cache.
static __device__ __noinline__ float div_full(float x, float s) { return __fdiv_rn(x, s); }
__device__ __forceinline__ Divisor make_divisor(float s) {
  Divisor d;
  const float a = fabsf(s);
  d.s = s;
  d.fast = a > 0x1p-60f && a < 0x1p60f;
  d.y = d.fast ? __frcp_rn(s) : 0.0f;
  return d;
}
__device__ __forceinline__ float div_rn(float x, const Divisor& d) {
  if (d.fast) {
    float q = __fmul_rn(x, d.y);
    if (fabsf(q) < 0x1p24f && fabsf(x) > 0x1p-90f) {
      float r = __fmaf_rn(-q, d.s, x);
      q = __fmaf_rn(r, d.y, q);
      r = __fmaf_rn(-q, d.s, x);
      return __fmaf_rn(r, d.y, q);
    }
    if (x == 0.0f) return q;  // +-0 / s
  }
  return div_full(x, d.s);
}

// Two-wide float arithmetic (sm_100 packed f32x2 instructions): one issue slot carries two
// multiply-adds, each rounded exactly like its scalar form.  The stream encodes are issue-bound,
// so halving the slots of the division chain is what these buy.  One trap, found by a parity
// test: ptxas contracts an f2_mul whose result feeds an f2_add into one fused multiply-add
// (`.rn` on both notwithstanding), so a product that must be rounded before an addition is
// computed with the scalar intrinsics.  The division chain below has no such pair.
struct F2 {
  unsigned long long b;
};
__device__ __forceinline__ F2 f2_pack(float lo, float hi) {
  F2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.b) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(F2 a, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.b));
}
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
  F2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.b) : "l"(a.b), "l"(b.b));
  return r;
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
  F2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.b) : "l"(a.b), "l"(b.b));
  return r;
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
  F2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.b) : "l"(a.b), "l"(b.b), "l"(c.b));
  return r;
}
// The short division of div_rn4 on a pair: x * y corrected twice by the residual (`ns` = -s).
// Returns the quotient pair; `q0` receives the first estimate (the domain check reads it).
__device__ __forceinline__ F2 f2_div_short(F2 x, F2 y, F2 ns, F2& q0) {
  q0 = f2_mul(x, y);
  F2 r = f2_fma(q0, ns, x);
  const F2 q1 = f2_fma(r, y, q0);
  r = f2_fma(q1, ns, x);
  return f2_fma(r, y, q1);
}

// Four quotients by the same divisor.  The short form runs unconditionally on all four (no
// per-element branch, so the four dependency chains overlap); the rare elements outside its
// domain are redone with the full-range division afterwards.
// Returns true when at least one element took the full division (its quotient is >= `limit`
// in magnitude, infinite or NaN).
__device__ __forceinline__ bool div_rn4(const float (&x)[4], const Divisor& d, float (&q)[4],
                                        float limit = 0x1p24f) {
  bool any = false;
  if (d.fast) {
    bool redo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float q0 = __fmul_rn(x[i], d.y);
      float r = __fmaf_rn(-q0, d.s, x[i]);
      const float q1 = __fmaf_rn(r, d.y, q0);
      r = __fmaf_rn(-q1, d.s, x[i]);
      q[i] = __fmaf_rn(r, d.y, q1);
      // Outside |q| < limit (overflowing or NaN quotients included) the full division decides.
      // Tiny operands need no guard: |s| >= 2^-60 keeps any quotient that lost bits to
      // underflow far below 1/2, and every caller rounds the quotient to an integer next.
      redo[i] = !(fabsf(q0) < limit);
      any |= redo[i];
    }
    if (any) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (redo[i]) q[i] = div_full(x[i], d.s);
    }
  } else {
    any = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = div_full(x[i], d.s);
  }
  return any;
}

// clip(rint(x / s) + z, qmin, qmax) for four elements sharing (s, z).
__device__ __forceinline__ void code4_f32(const float (&x)[4], const Divisor& d, float z, float qmin,
                                          float qmax, float (&c)[4]) {
  float q[4];
  div_rn4(x, d, q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float t = __fadd_rn(rintf(q[i]), z);
    // max-then-min equals the compare-based clip for every non-NaN t (NaN is out of contract:
    // the reference's integer cast of it is undefined)
    c[i] = fminf(fmaxf(t, qmin), qmax);
  }
}

// Integer-domain tail of the encode.  For |q| < 2^22, q + 1.5*2^23 rounds q to the nearest
// integer (ties to even) in the low mantissa bits, so rint, "+ z", the clip and the integer cast
// collapse into one float add and integer ops, with the same result as the float sequence
// whenever z is an integer of modest size.  `zofs` = z - bits(1.5*2^23).
struct IntGrid {
  int zofs, qmin, qmax;
  bool fast;   // z integral, |z|, |qmin|, |qmax| < 2^22
  bool clamp;  // grid narrower than the saturating pack of the storage type
};
__device__ __forceinline__ IntGrid make_int_grid(float z, float qmin, float qmax, int store_lo, int store_hi) {
  IntGrid g;
  g.fast = z == rintf(z) && fabsf(z) < 0x1p22f && fabsf(qmin) < 0x1p22f && fabsf(qmax) < 0x1p22f;
  g.zofs = (g.fast ? (int)z : 0) - 0x4B400000;
  g.qmin = (int)qmin, g.qmax = (int)qmax;
  g.clamp = !(g.qmin <= store_lo && g.qmax >= store_hi);
  return g;
}
// clip(rint(x / s) + z, qmin, qmax) as integers, four elements sharing (s, z).
__device__ __forceinline__ void code4_int(const float (&x)[4], const Divisor& d, const IntGrid& g,
                                          float z, float qmin, float qmax, int (&c)[4]) {
  float q[4];
  const bool any = div_rn4(x, d, q, 0x1p22f);
  if (!any && g.fast) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int v = __float_as_int(__fadd_rn(q[i], 12582912.0f)) + g.zofs;
      if (g.clamp) v = min(max(v, g.qmin), g.qmax);
      c[i] = v;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float t = __fadd_rn(rintf(q[i]), z);
      c[i] = __float2int_rz(t < qmin ? qmin : (t > qmax ? qmax : t));
    }
  }
}
// code4_int without the domain check, on the packed pipe: for callers that know every quotient is
// below 2^22 in magnitude (a per-token symmetric encode: |x| <= abs-max = s * half) and whose
// divisor is in the short division's range (d.fast) with an integral zero point (g.fast).
struct ShortDiv {
  F2 y2, ns2;
};
__device__ __forceinline__ ShortDiv make_short_div(const Divisor& d) {
  ShortDiv sd;
  sd.y2 = f2_pack(d.y, d.y), sd.ns2 = f2_pack(-d.s, -d.s);
  return sd;
}
__device__ __forceinline__ void code4_short(const float (&x)[4], const ShortDiv& sd, const IntGrid& g, int (&c)[4]) {
  const F2 magic2 = f2_pack(12582912.0f, 12582912.0f);
#pragma unroll
  for (int i = 0; i < 4; i += 2) {
    F2 q0;
    const F2 qq = f2_div_short(f2_pack(x[i], x[i + 1]), sd.y2, sd.ns2, q0);
    float t0, t1;
    f2_unpack(f2_add(qq, magic2), t0, t1);
    c[i] = __float_as_int(t0) + g.zofs;
    c[i + 1] = __float_as_int(t1) + g.zofs;
  }
  if (g.clamp) {
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = min(max(c[i], g.qmin), g.qmax);
  }
}
// four ints -> four packed 8-bit codes (saturating to the storage type)
__device__ __forceinline__ uint32_t pack4i_s8(const int (&c)[4]) {
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(c[3]), "r"(c[2]), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(c[1]), "r"(c[0]), "r"(hi));
  return out;
}
__device__ __forceinline__ uint32_t pack4i_u8(const int (&c)[4]) {
  uint32_t hi, out;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(c[3]), "r"(c[2]), "r"(0));
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(c[1]), "r"(c[0]), "r"(hi));
  return out;
}

// Four integral floats (already clipped to the storage range) -> four packed 8-bit codes.
__device__ __forceinline__ uint32_t pack4_s8(const float (&c)[4]) {
  const int a = __float2int_rz(c[0]), b = __float2int_rz(c[1]), d = __float2int_rz(c[2]), e = __float2int_rz(c[3]);
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(e), "r"(d), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
  return out;
}
__device__ __forceinline__ uint32_t pack4_u8(const float (&c)[4]) {
  const int a = __float2int_rz(c[0]), b = __float2int_rz(c[1]), d = __float2int_rz(c[2]), e = __float2int_rz(c[3]);
  uint32_t hi, out;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(e), "r"(d), "r"(0));
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
  return out;
}

// clip(rint(x / s) + z, qmin, qmax): the reference's quantize, float domain.
__device__ __forceinline__ float code_f32(float x, const Divisor& d, float z, float qmin, float qmax) {
  float t = div_rn(x, d);
  t = rintf(t);  // ties to even
  t = __fadd_rn(t, z);
  // compare-based clip, lower bound first; NaN falls through
  return t < qmin ? qmin : (t > qmax ? qmax : t);
}
__device__ __forceinline__ float code_f32(float x, float s, float z, float qmin, float qmax) {
  float t = __fdiv_rn(x, s);
  t = rintf(t);
  t = __fadd_rn(t, z);
  return t < qmin ? qmin : (t > qmax ? qmax : t);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) {
  return __uint_as_float(b16 << 16);
}

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Streaming (read-once) 128-bit load that does not pollute L1.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_stream_u4(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- bulk-copy pipeline pieces (HBM -> shared memory without register staging) ---------------
namespace pipe {
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// One-dimensional bulk copy global -> shared; `bytes` and both addresses are multiples of 16.
// The bytes are counted on `bar`, whose single arrival this call also performs.
__device__ __forceinline__ void load_async(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Orders this thread's earlier generic-proxy reads of shared memory before later
// asynchronous-proxy writes to it (a slot is refilled after it was read).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Bounded wait on a phase; false when the poll budget (seconds) ran out.
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
}  // namespace pipe

}  // namespace lq
