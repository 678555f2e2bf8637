// Shared helpers for the lucid_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "lucid_b200.h"

namespace lq {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

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

// ---- device-side exact arithmetic ---------------------------------------
// Every step is a separate IEEE binary32 operation; the intrinsics keep the
// compiler from contracting or approximating them.

// clip(rint(x / s) + z, qmin, qmax): the reference's quantize, float domain.
__device__ __forceinline__ float code_f32(float x, float s, float z, float qmin, float qmax) {
  float t = __fdiv_rn(x, s);
  t = rintf(t);  // ties to even
  t = __fadd_rn(t, z);
  // compare-based clip, lower bound first; NaN falls through
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

}  // namespace lq
