// Group-wise weight-only codes (4 or 8 bits) and the decode-shape matmul on them.
//
// The reference reaches this through its MLX route (lucid/quantization/_qgemm.py:69-320,
// lucid/_C/ops/quantized/QuantizedMatmul.cpp:47-109): the weight's input axis is cut into groups
// of `group` elements, each with an affine (scale, bias); codes are unsigned `bits`-wide integers
// packed little-endian into 32-bit words; y = x * w_hat^T with w_hat = code * scale + bias decoded
// inside the kernel.  The formulas are the ones the reference documents
// (_qgemm.py:84-97): scale = (max - min) / (2^bits - 1), bias = min,
// code = clip(rint((w - bias) / scale), 0, 2^bits - 1); a constant group takes scale 1 (all codes
// 0, w_hat = bias exactly).
//
// The matmul is the bandwidth-bound decode shape (few activation rows): one warp per output
// row, 16 bytes of packed codes per lane and step, activations read through L1 (they are a few
// KB), float32 accumulation as  sum_g scale_g * (sum_k x_k * code_k) + bias_g * (sum_k x_k),
// which keeps the decode to one integer-to-float conversion per code.
#include "common.cuh"

namespace lq {
namespace {

constexpr int kGwThreads = 256;

template <int BITS>
__global__ void __launch_bounds__(kGwThreads)
gw_quantize_kernel(const float* __restrict__ w, size_t n_groups, int group, uint32_t* __restrict__ packed,
                   float* __restrict__ scales, float* __restrict__ biases) {
  constexpr int kPerWord = 32 / BITS;
  constexpr float kTop = (float)((1 << BITS) - 1);
  // one warp per group: lanes stride over the group's elements (coalesced), two passes
  const size_t g = ((size_t)blockIdx.x * kGwThreads + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (g >= n_groups) return;
  const float* wg = w + g * (size_t)group;
  float mn = INFINITY, mx = -INFINITY;
  for (int i = lane; i < group; i += 32) {
    const float v = __ldg(wg + i);
    mn = fminf(mn, v), mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  float s = __fdiv_rn(__fsub_rn(mx, mn), kTop);
  if (!(s > 0.0f)) s = 1.0f;  // constant group: every code 0, bias carries the value
  if (lane == 0) scales[g] = s, biases[g] = mn;
  // each lane packs whole words: word j of the group holds elements [j * kPerWord, (j + 1) * kPerWord)
  const int words = group / kPerWord;
  uint32_t* pg = packed + g * (size_t)words;
  for (int j = lane; j < words; j += 32) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < kPerWord; ++e) {
      const float q = rintf(__fdiv_rn(__fsub_rn(__ldg(wg + j * kPerWord + e), mn), s));
      const float c = q < 0.0f ? 0.0f : (q > kTop ? kTop : q);
      word |= (uint32_t)(int)c << (e * BITS);
    }
    pg[j] = word;
  }
}

template <int BITS>
__global__ void __launch_bounds__(kGwThreads)
gw_dequantize_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scales,
                     const float* __restrict__ biases, size_t n_words, int group, float* __restrict__ out) {
  constexpr int kPerWord = 32 / BITS;
  constexpr uint32_t kMask = (1u << BITS) - 1u;
  const size_t j = (size_t)blockIdx.x * kGwThreads + threadIdx.x;
  if (j >= n_words) return;
  const uint32_t word = __ldg(packed + j);
  const size_t e0 = j * kPerWord;
  const size_t g = e0 / (size_t)group;
  const float s = __ldg(scales + g), b = __ldg(biases + g);
#pragma unroll
  for (int e = 0; e < kPerWord; ++e)
    out[e0 + e] = __fadd_rn(__fmul_rn((float)((word >> (e * BITS)) & kMask), s), b);
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T>
__device__ __forceinline__ void store1(T* p, float v);
template <>
__device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One warp per output row n; MT activation rows at a time.  Per step a lane takes one 16-byte
// piece of the row's packed codes (128 / BITS consecutive input positions, inside one group as
// group % (128 / BITS) == 0) and accumulates  scale * sum(x * code) + bias * sum(x)  per
// activation row; lanes are reduced with shuffles at the end.
template <int BITS, int MT, typename T>
__global__ void __launch_bounds__(kGwThreads)
gw_matvec_kernel(const T* __restrict__ x, size_t ldx, const uint32_t* __restrict__ packed,
                 const float* __restrict__ scales, const float* __restrict__ biases, size_t N, size_t K, int group,
                 const float* __restrict__ bias, int relu, T* __restrict__ out, size_t ldo) {
  constexpr int kPerPiece = 128 / BITS;  // codes per 16-byte piece: 32 (4 bits) or 16 (8 bits)
  constexpr uint32_t kMask = (1u << BITS) - 1u;
  const size_t n = ((size_t)blockIdx.x * kGwThreads + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (n >= N) return;
  const size_t pieces = K / kPerPiece;
  const uint4* wrow = reinterpret_cast<const uint4*>(packed + n * (K * BITS / 32));
  const size_t groups_per_row = K / (size_t)group;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
  for (size_t p = lane; p < pieces; p += 32) {
    uint4 u;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                 : "l"(wrow + p));
    const size_t k0 = p * kPerPiece;
    const size_t g = n * groups_per_row + k0 / (size_t)group;
    const float s = __ldg(scales + g), b = __ldg(biases + g);
    const uint32_t words[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float dot = 0.0f, sum = 0.0f;
#pragma unroll
      for (int q = 0; q < kPerPiece / 8; ++q) {
        float xv[8];
        load8<T>(x + (size_t)m * ldx + k0 + q * 8, xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int idx = q * 8 + e;
          const uint32_t word = words[idx / (32 / BITS)];
          const float c = (float)((word >> ((idx % (32 / BITS)) * BITS)) & kMask);
          dot = fmaf(xv[e], c, dot);
          sum += xv[e];
        }
      }
      acc[m] = fmaf(s, dot, fmaf(b, sum, acc[m]));
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) {
      if (bias) v += __ldg(bias + n);
      if (relu) v = fmaxf(v, 0.0f);
      store1<T>(out + (size_t)m * ldo + n, v);
    }
  }
}

int check_gw(const char* who, size_t K, int group, int bits) {
  const std::string w(who);
  if (bits != 4 && bits != 8) return fail(LQ_ERR_UNSUPPORTED, w + ": bits must be 4 or 8");
  if (group != 32 && group != 64 && group != 128) return fail(LQ_ERR_UNSUPPORTED, w + ": group_size must be 32, 64 or 128");
  if (K == 0 || K % (size_t)group != 0) return fail(LQ_ERR_SHAPE, w + ": in_features must be a multiple of group_size");
  return LQ_OK;
}

template <int BITS, typename T>
int launch_matvec(const T* x, size_t M, size_t ldx, const uint32_t* packed, const float* scales, const float* biases,
                  size_t N, size_t K, int group, const float* bias, int relu, T* out, size_t ldo, cudaStream_t st) {
  const int grid = (int)((N * 32 + kGwThreads - 1) / kGwThreads);
  size_t m0 = 0;
  // activation rows in blocks of 4, then 2, then 1 (every block re-reads the packed weight: the
  // kernel is for decode shapes; larger batches are better served by dequantize + a library GEMM)
  while (m0 < M) {
    const size_t left = M - m0;
    const T* xm = x + m0 * ldx;
    T* om = out + m0 * ldo;
    if (left >= 4) {
      gw_matvec_kernel<BITS, 4, T><<<grid, kGwThreads, 0, st>>>(xm, ldx, packed, scales, biases, N, K, group, bias, relu, om, ldo);
      m0 += 4;
    } else if (left >= 2) {
      gw_matvec_kernel<BITS, 2, T><<<grid, kGwThreads, 0, st>>>(xm, ldx, packed, scales, biases, N, K, group, bias, relu, om, ldo);
      m0 += 2;
    } else {
      gw_matvec_kernel<BITS, 1, T><<<grid, kGwThreads, 0, st>>>(xm, ldx, packed, scales, biases, N, K, group, bias, relu, om, ldo);
      m0 += 1;
    }
  }
  return check_cuda(cudaGetLastError(), "lq_groupwise_matmul launch");
}

}  // namespace
}  // namespace lq

using namespace lq;

extern "C" int lq_groupwise_quantize(const float* w, size_t N, size_t K, int group_size, int bits, uint32_t* packed,
                                     float* scales, float* biases, void* stream) {
  if (N == 0) return LQ_OK;
  if (!w || !packed || !scales || !biases) return fail(LQ_ERR_DEVICE, "lq_groupwise_quantize: null pointer");
  if (int rc = check_gw("lq_groupwise_quantize", K, group_size, bits)) return rc;
  const size_t n_groups = N * (K / (size_t)group_size);
  const int grid = (int)((n_groups * 32 + kGwThreads - 1) / kGwThreads);
  if (bits == 4)
    gw_quantize_kernel<4><<<grid, kGwThreads, 0, (cudaStream_t)stream>>>(w, n_groups, group_size, packed, scales, biases);
  else
    gw_quantize_kernel<8><<<grid, kGwThreads, 0, (cudaStream_t)stream>>>(w, n_groups, group_size, packed, scales, biases);
  return check_cuda(cudaGetLastError(), "lq_groupwise_quantize launch");
}

extern "C" int lq_groupwise_dequantize(const uint32_t* packed, const float* scales, const float* biases, size_t N,
                                       size_t K, int group_size, int bits, float* out, void* stream) {
  if (N == 0) return LQ_OK;
  if (!out || !packed || !scales || !biases) return fail(LQ_ERR_DEVICE, "lq_groupwise_dequantize: null pointer");
  if (int rc = check_gw("lq_groupwise_dequantize", K, group_size, bits)) return rc;
  const size_t n_words = N * K * (size_t)bits / 32;
  const int grid = (int)((n_words + kGwThreads - 1) / kGwThreads);
  if (bits == 4)
    gw_dequantize_kernel<4><<<grid, kGwThreads, 0, (cudaStream_t)stream>>>(packed, scales, biases, n_words, group_size, out);
  else
    gw_dequantize_kernel<8><<<grid, kGwThreads, 0, (cudaStream_t)stream>>>(packed, scales, biases, n_words, group_size, out);
  return check_cuda(cudaGetLastError(), "lq_groupwise_dequantize launch");
}

extern "C" int lq_groupwise_matmul(const void* x, int x_dtype, size_t M, size_t ldx, const uint32_t* packed,
                                   const float* scales, const float* biases, size_t N, size_t K, int group_size,
                                   int bits, const float* bias, int relu, void* out, size_t ldo, void* stream) {
  if (M == 0 || N == 0) return LQ_OK;
  if (!x || !out || !packed || !scales || !biases) return fail(LQ_ERR_DEVICE, "lq_groupwise_matmul: null pointer");
  if (int rc = check_gw("lq_groupwise_matmul", K, group_size, bits)) return rc;
  if (x_dtype != LQ_F32 && x_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_groupwise_matmul: x must be f32|bf16");
  const size_t esz = x_dtype == LQ_F32 ? 4 : 2;
  if (!aligned16(x) || !aligned16(packed) || (ldx * esz) % 16 != 0 || ldx < K || ldo < N)
    return fail(LQ_ERR_ALIGNMENT, "lq_groupwise_matmul: x rows and the packed weight must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  if (x_dtype == LQ_F32)
    return bits == 4 ? launch_matvec<4, float>((const float*)x, M, ldx, packed, scales, biases, N, K, group_size, bias, relu, (float*)out, ldo, st)
                     : launch_matvec<8, float>((const float*)x, M, ldx, packed, scales, biases, N, K, group_size, bias, relu, (float*)out, ldo, st);
  using B = __nv_bfloat16;
  return bits == 4 ? launch_matvec<4, B>((const B*)x, M, ldx, packed, scales, biases, N, K, group_size, bias, relu, (B*)out, ldo, st)
                   : launch_matvec<8, B>((const B*)x, M, ldx, packed, scales, biases, N, K, group_size, bias, relu, (B*)out, ldo, st);
}
