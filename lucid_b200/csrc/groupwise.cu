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
// The matmul is the bandwidth-bound decode shape (few activation rows): a CTA per group of output
// rows, 16 bytes of packed codes per thread, row and step, activations read through L1 (they are a few KB), codes decoded two at a time without a
// conversion instruction and multiplied on the packed float32 pipe; the group's (scale, bias)
// is applied once per 16-byte piece.
#include "common.cuh"

namespace lq {
namespace {

constexpr int kGwThreads = 256;  // quantize / dequantize
constexpr int kMvThreads = 128;  // decode matmul

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
__device__ __forceinline__ void store1(T* p, float v);
template <>
__device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Codes of one 32-bit word as float32 pairs without a conversion instruction: a byte permute
// drops a code into the mantissa of 2^23 (0x4B000000 | code == 2^23 + code exactly) and one
// packed subtraction brings two of them back.  The conversion unit runs at an eighth of the
// arithmetic rate and was what bounded the first form of this kernel.  Pair e holds the codes of
// input positions 2e and 2e + 1 of the word.
template <int BITS>
__device__ __forceinline__ void decode_pairs(uint32_t word, F2 neg, F2 (&c)[16 / BITS]);
template <>
__device__ __forceinline__ void decode_pairs<8>(uint32_t word, F2 neg, F2 (&c)[2]) {
  c[0] = f2_add(f2_pack(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7440)),
                        __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7441))), neg);
  c[1] = f2_add(f2_pack(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7442)),
                        __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7443))), neg);
}
template <>
__device__ __forceinline__ void decode_pairs<4>(uint32_t word, F2 neg, F2 (&c)[4]) {
  const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;  // even / odd nibbles
#pragma unroll
  for (int i = 0; i < 4; ++i)
    c[i] = f2_add(f2_pack(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7440 + i)),
                          __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7440 + i))), neg);
}

// kN consecutive activations (kN = 4 or 8, the positions of one packed word) as float32 pairs.
template <typename T, int kN>
__device__ __forceinline__ void load_pairs(const T* p, F2 (&v)[kN / 2]);
template <>
__device__ __forceinline__ void load_pairs<float, 4>(const float* p, F2 (&v)[2]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = f2_pack(a.x, a.y), v[1] = f2_pack(a.z, a.w);
}
template <>
__device__ __forceinline__ void load_pairs<float, 8>(const float* p, F2 (&v)[4]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = f2_pack(a.x, a.y), v[1] = f2_pack(a.z, a.w), v[2] = f2_pack(b.x, b.y), v[3] = f2_pack(b.z, b.w);
}
__device__ __forceinline__ F2 bf16_pair(uint32_t w) {
  return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
__device__ __forceinline__ void load_pairs<__nv_bfloat16, 4>(const __nv_bfloat16* p, F2 (&v)[2]) {
  const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
  v[0] = bf16_pair(u.x), v[1] = bf16_pair(u.y);
}
template <>
__device__ __forceinline__ void load_pairs<__nv_bfloat16, 8>(const __nv_bfloat16* p, F2 (&v)[4]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  v[0] = bf16_pair(u.x), v[1] = bf16_pair(u.y), v[2] = bf16_pair(u.z), v[3] = bf16_pair(u.w);
}

// One step of a thread: the same 16-byte piece (128 / BITS consecutive input positions starting
// at k0, inside one group as group % (128 / BITS) == 0) of each of R rows against MT activation
// rows.  With w_hat = code * s + b constant in (s, b) over the piece,
//   sum_k x_k * w_hat_k = s * sum_k x_k * code_k + b * sum_k x_k,
// so a code costs its decode and half a packed multiply-add; the activations (read through L1:
// they are a few KB) are loaded word by word, once for all R rows, and their sum is shared too.
template <int BITS, int MT, int R, typename T>
__device__ __forceinline__ void gw_consume(const uint4 (&u)[R], const float (&s)[R], const float (&b)[R],
                                           const T* __restrict__ x, size_t ldx, size_t k0, float (&acc)[R][MT]) {
  constexpr int kPerWord = 32 / BITS, kPairs = kPerWord / 2;
  const F2 zero = f2_pack(0.0f, 0.0f), neg = f2_pack(-8388608.0f, -8388608.0f);
  F2 d[R][MT], xs[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    xs[m] = zero;
#pragma unroll
    for (int r = 0; r < R; ++r) d[r][m] = zero;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    F2 xp[MT][kPairs];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      load_pairs<T, kPerWord>(x + (size_t)m * ldx + k0 + j * kPerWord, xp[m]);
#pragma unroll
      for (int e = 0; e < kPairs; ++e) xs[m] = f2_add(xs[m], xp[m][e]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t word = j == 0 ? u[r].x : (j == 1 ? u[r].y : (j == 2 ? u[r].z : u[r].w));
      F2 c[kPairs];
      decode_pairs<BITS>(word, neg, c);
#pragma unroll
      for (int e = 0; e < kPairs; ++e)
#pragma unroll
        for (int m = 0; m < MT; ++m) d[r][m] = f2_fma(xp[m][e], c[e], d[r][m]);
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float xl, xh;
    f2_unpack(xs[m], xl, xh);
    const float xsum = xl + xh;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float dl, dh;
      f2_unpack(d[r][m], dl, dh);
      acc[r][m] = fmaf(s[r], dl + dh, fmaf(b[r], xsum, acc[r][m]));
    }
  }
}

// The R x MT sums of a CTA's warps -> out (+ bias, ReLU).
template <int MT, int R, typename T>
__device__ __forceinline__ void gw_finish(float (&acc)[R][MT], float (*part)[R][MT], size_t n0, size_t N,
                                          const float* __restrict__ bias, int relu, T* __restrict__ out, size_t ldo) {
  constexpr int kWarps = kMvThreads / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) part[warp][r][m] = v;
    }
  __syncthreads();
  if (threadIdx.x < R * MT) {
    const int r = threadIdx.x / MT, m = threadIdx.x % MT;
    if (n0 + r < N) {
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += part[w][r][m];
      if (bias) v += __ldg(bias + n0 + r);
      if (relu) v = fmaxf(v, 0.0f);
      store1<T>(out + (size_t)m * ldo + n0 + r, v);
    }
  }
}

// One CTA of four warps per R consecutive output rows: the warps split the input axis and add
// up through shared memory (a decode-shape launch has too few rows to fill the GPU with one
// warp per row group, and small CTAs retire and refill in fine grains: 128 threads measured
// 10-15 % faster than 256, 64 and 32 no better); a thread's R row loads of a step are issued
// together.  Registers are capped for four resident CTAs (the two-activation-row W4 instance
// would otherwise take 149).
template <int BITS, int MT, int R, typename T>
__global__ void __launch_bounds__(kMvThreads, 4)
gw_matvec_kernel(const T* __restrict__ x, size_t ldx, const uint32_t* __restrict__ packed,
                 const float* __restrict__ scales, const float* __restrict__ biases, size_t N, size_t K, int group,
                 const float* __restrict__ bias, int relu, T* __restrict__ out, size_t ldo) {
  constexpr int kPerPiece = 128 / BITS;  // codes per 16-byte piece: 32 (4 bits) or 16 (8 bits)
  __shared__ float s_part[kMvThreads / 32][R][MT];
  const size_t n0 = (size_t)blockIdx.x * R;
  const size_t pieces = K / kPerPiece;
  const size_t row_words = K * BITS / 32;
  const int gshift = 31 - __clz(group);  // group sizes are powers of two
  const size_t groups_per_row = K >> gshift;
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;
  for (size_t p = threadIdx.x; p < pieces; p += kMvThreads) {
    const size_t k0 = p * kPerPiece;
    uint4 u[R];
    float s[R], b[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const size_t n = n0 + r < N ? n0 + r : N - 1;  // a row past the end repeats the last one (not stored)
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(u[r].x), "=r"(u[r].y), "=r"(u[r].z), "=r"(u[r].w)
                   : "l"(reinterpret_cast<const uint4*>(packed + n * row_words) + p));
      const size_t g = n * groups_per_row + (k0 >> gshift);
      s[r] = __ldg(scales + g), b[r] = __ldg(biases + g);
    }
    gw_consume<BITS, MT, R, T>(u, s, b, x, ldx, k0, acc);
  }
  gw_finish<MT, R, T>(acc, s_part, n0, N, bias, relu, out, ldo);
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
  constexpr int R = 4;  // output rows per CTA: the activations of a step are loaded once for all of them
  const unsigned grid = (unsigned)((N + R - 1) / R);
  size_t m0 = 0;
  // activation rows in pairs, then one (every pass re-reads the packed weight: the kernel is for
  // decode shapes; larger batches are better served by dequantize + a library GEMM)
  while (m0 < M) {
    const T* xm = x + m0 * ldx;
    T* om = out + m0 * ldo;
    if (M - m0 >= 2) {
      gw_matvec_kernel<BITS, 2, R, T><<<grid, kMvThreads, 0, st>>>(xm, ldx, packed, scales, biases, N, K, group, bias, relu, om, ldo);
      m0 += 2;
    } else {
      gw_matvec_kernel<BITS, 1, R, T><<<grid, kMvThreads, 0, st>>>(xm, ldx, packed, scales, biases, N, K, group, bias, relu, om, ldo);
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
