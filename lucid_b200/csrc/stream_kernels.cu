// HBM-bound streaming kernels: range reduction, qparams, quantize, dequantize,
// fake-quantize and the fused per-token encode.  All are 128-bit coalesced
// streams; each thread moves 16 elements per iteration and the grids are sized
// in multiples of the SM count.  Arithmetic follows the reference's order with
// one IEEE binary32 operation per step (see common.cuh).
#include <math.h>

#include <mutex>
#include <string>

#include "common.cuh"

namespace lq {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;
constexpr int kMaxBlocks = kNumSMs * kCtasPerSm;  // 1184

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

__device__ __forceinline__ void packet_params(const QParamRef& q, size_t row, size_t col0,
                                              float (&s)[16], float (&z)[16]) {
  if (q.mode == LQ_PER_COL) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 a = __ldg(reinterpret_cast<const float4*>(q.s + col0) + i);
      float4 b = __ldg(reinterpret_cast<const float4*>(q.z + col0) + i);
      s[4 * i] = a.x, s[4 * i + 1] = a.y, s[4 * i + 2] = a.z, s[4 * i + 3] = a.w;
      z[4 * i] = b.x, z[4 * i + 1] = b.y, z[4 * i + 2] = b.z, z[4 * i + 3] = b.w;
    }
  } else {
    float sv, zv;
    if (q.mode == LQ_PER_ROW) {
      sv = __ldg(q.s + row);
      zv = __ldg(q.z + row);
    } else if (q.s != nullptr) {
      sv = __ldg(q.s);
      zv = __ldg(q.z);
    } else {
      sv = q.sv;
      zv = q.zv;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = sv, z[i] = zv;
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
__device__ __forceinline__ float apply(float x, float s, float z, float qmin, float qmax,
                                       float* mask) {
  if (OP == Op::kQuantize) return code_f32(x, s, z, qmin, qmax);
  if (OP == Op::kDequantize) return __fmul_rn(__fsub_rn(x, z), s);
  // fake-quantize: q_pre, clip, (q - z) * s
  float q_pre = __fadd_rn(rintf(__fdiv_rn(x, s)), z);
  float q = q_pre < qmin ? qmin : (q_pre > qmax ? qmax : q_pre);
  if (mask) *mask = (q_pre >= qmin ? 1.0f : 0.0f) * (q_pre <= qmax ? 1.0f : 0.0f);
  return __fmul_rn(__fsub_rn(q, z), s);
}

// Vector kernel: one 16-element packet per thread-iteration, grid-stride.
template <Op OP, typename In, typename Out, bool MASK>
__global__ void __launch_bounds__(kThreads)
affine_vec_kernel(const In* __restrict__ x, Out* __restrict__ out, float* __restrict__ mask,
                  size_t rows, size_t cols, QParamRef q, float qmin, float qmax) {
  const size_t ppr = cols / 16;
  const size_t npackets = rows * ppr;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t p = (size_t)blockIdx.x * kThreads + threadIdx.x; p < npackets; p += stride) {
    const size_t row = p / ppr;
    const size_t col0 = (p - row * ppr) * 16;
    const size_t off = row * cols + col0;
    float v[16], s[16], z[16], m[16];
    Packet<In>::load(x + off, v);
    packet_params(q, row, col0, s, z);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = apply<OP>(v[i], s[i], z[i], qmin, qmax, MASK ? &m[i] : nullptr);
    Packet<Out>::store(out + off, v);
    if (MASK) Packet<float>::store(mask + off, m);
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
    float r = apply<OP>(Packet<In>::load1(x + i), s, z, qmin, qmax, MASK ? &m : nullptr);
    Packet<Out>::store1(out + i, r);
    if (MASK) mask[i] = m;
  }
}

inline int grid_for(size_t work_items) {
  size_t blocks = (work_items + kThreads - 1) / kThreads;
  if (blocks > (size_t)kMaxBlocks) blocks = kMaxBlocks;
  if (blocks == 0) blocks = 1;
  return (int)blocks;
}

template <Op OP, typename In, typename Out, bool MASK = false>
int launch_affine(const void* x, void* out, float* mask, size_t rows, size_t cols,
                  const QParamRef& q, int qmin, int qmax, cudaStream_t st) {
  const bool vec = (cols % 16 == 0) && aligned16(x) && aligned16(out) &&
                   (!MASK || aligned16(mask)) &&
                   (q.mode != LQ_PER_COL || (aligned16(q.s) && aligned16(q.z)));
  if (vec) {
    affine_vec_kernel<OP, In, Out, MASK><<<grid_for(rows * (cols / 16)), kThreads, 0, st>>>(
        (const In*)x, (Out*)out, mask, rows, cols, q, (float)qmin, (float)qmax);
  } else {
    affine_scalar_kernel<OP, In, Out, MASK><<<grid_for(rows * cols), kThreads, 0, st>>>(
        (const In*)x, (Out*)out, mask, rows, cols, q, (float)qmin, (float)qmax);
  }
  return check_cuda(cudaGetLastError(), "affine kernel launch");
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

// ---- range reduction -----------------------------------------------------------
struct MinMaxWorkspace {
  unsigned int ticket;
  unsigned int pad[3];
  float pmin[kMaxBlocks];
  float pmax[kMaxBlocks];
};

template <typename In>
__device__ __forceinline__ void minmax_accumulate(const In* x, size_t n, size_t first, size_t stride,
                                                  bool vec_ok, float& mn, float& mx) {
  // x[0..n): thread `first` of `stride` threads.  16 elements per packet.
  size_t npk = vec_ok ? n / 16 : 0;
  size_t p = first;
  // two packets in flight per iteration
  for (; p + stride < npk; p += 2 * stride) {
    float a[16], b[16];
    Packet<In>::load(x + p * 16, a);
    Packet<In>::load(x + (p + stride) * 16, b);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      mn = fminf(mn, fminf(a[i], b[i]));
      mx = fmaxf(mx, fmaxf(a[i], b[i]));
    }
  }
  for (; p < npk; p += stride) {
    float a[16];
    Packet<In>::load(x + p * 16, a);
#pragma unroll
    for (int i = 0; i < 16; ++i) mn = fminf(mn, a[i]), mx = fmaxf(mx, a[i]);
  }
  for (size_t i = npk * 16 + first; i < n; i += stride) {
    float v = Packet<In>::load1(x + i);
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

// Per-tensor: per-CTA partials go to the workspace; the CTA that takes the last
// ticket folds them (min/max are exact in any order) and re-arms the ticket.
template <typename In>
__global__ void __launch_bounds__(kThreads)
minmax_tensor_kernel(const In* __restrict__ x, size_t n, bool vec_ok, MinMaxWorkspace* ws,
                     float* out_min, float* out_max) {
  float mn = INFINITY, mx = -INFINITY;
  minmax_accumulate(x, n, (size_t)blockIdx.x * kThreads + threadIdx.x,
                    (size_t)gridDim.x * kThreads, vec_ok, mn, mx);
  block_minmax(mn, mx);
  __shared__ bool is_last;
  if (threadIdx.x == 0) {
    ws->pmin[blockIdx.x] = mn;
    ws->pmax[blockIdx.x] = mx;
    __threadfence();
    unsigned int t = atomicAdd(&ws->ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  mn = INFINITY, mx = -INFINITY;
  for (unsigned int i = threadIdx.x; i < gridDim.x; i += kThreads) {
    mn = fminf(mn, __ldcg(&ws->pmin[i]));
    mx = fmaxf(mx, __ldcg(&ws->pmax[i]));
  }
  block_minmax(mn, mx);
  if (threadIdx.x == 0) {
    *out_min = mn;
    *out_max = mx;
    ws->ticket = 0;  // leave the workspace zeroed for the next call
  }
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
  const float lo = fminf(mn[i], 0.0f), hi = fmaxf(mx[i], 0.0f);
  if (symmetric) {
    const float m = fmaxf(fabsf(lo), fabsf(hi));
    const float half = (float)((double)(qmax - qmin) / 2.0);
    scale[i] = fmaxf(__fdiv_rn(m, half), eps);
    zp[i] = is_signed ? 0.0f : (float)((qmax + qmin + 1) / 2);
  } else {
    const float s = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), (float)((double)qmax - (double)qmin)), eps);
    scale[i] = s;
    const float t = __fsub_rn((float)qmin, rintf(__fdiv_rn(lo, s)));
    const float fq0 = (float)qmin, fq1 = (float)qmax;
    zp[i] = t < fq0 ? fq0 : (t > fq1 ? fq1 : t);
  }
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
    const size_t npk = vec_ok ? cols / 16 : 0;
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
    const float s = s_scale;
    int8_t* outr = out + r * cols;
    for (size_t p = threadIdx.x; p < npk; p += kThreads) {
      float v[16];
      Packet<In>::load(xr + p * 16, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = code_f32(v[i], s, 0.0f, qmin, qmax);
      Packet<int8_t>::store(outr + p * 16, v);
    }
    for (size_t i = npk * 16 + threadIdx.x; i < cols; i += kThreads)
      outr[i] = (int8_t)(int)code_f32(Packet<In>::load1(xr + i), s, 0.0f, qmin, qmax);
    __syncthreads();  // s_scale is rewritten by the next row
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

extern "C" size_t lq_minmax_workspace_bytes(void) { return sizeof(MinMaxWorkspace); }

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
    const size_t n = rows * cols;
    const bool vec_ok = aligned16(x);
    // two packets per thread-iteration; grid in multiples of the SM count
    size_t want = (n / 16 + 2 * kThreads - 1) / (2 * kThreads);
    int grid = (int)(want < 1 ? 1 : (want > (size_t)(kNumSMs * 4) ? kNumSMs * 4 : want));
    auto* ws = (MinMaxWorkspace*)workspace;
    if (in_dtype == LQ_F32)
      minmax_tensor_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, n, vec_ok, ws, out_min, out_max);
    else
      minmax_tensor_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, n, vec_ok, ws, out_min, out_max);
  } else if (mode == LQ_PER_ROW) {
    const bool vec_ok = aligned16(x) && ((cols * esz) % 16 == 0);
    if (cols <= 2048) {
      int grid = grid_for(rows * 32);
      if (in_dtype == LQ_F32)
        minmax_rows_warp_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, vec_ok, out_min, out_max);
      else
        minmax_rows_warp_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, vec_ok, out_min, out_max);
    } else {
      int grid = (int)(rows < (size_t)kMaxBlocks ? rows : kMaxBlocks);
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
  const int grid = (int)(rows < (size_t)kMaxBlocks ? rows : kMaxBlocks);
  cudaStream_t st = (cudaStream_t)stream;
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
constexpr int kMaxDevices = 64;
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
  const bool vec_ok = aligned16(x);
  size_t want = (n / 16 + 2 * kThreads - 1) / (2 * kThreads);
  int grid = (int)(want < 1 ? 1 : (want > (size_t)(kNumSMs * 4) ? kNumSMs * 4 : want));
  auto* ws = (MinMaxWorkspace*)scratch;
  if (in_dtype == LQ_F32)
    minmax_tensor_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, n, vec_ok, ws, out_min, out_max);
  else
    minmax_tensor_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, n, vec_ok, ws, out_min, out_max);
  return check_cuda(cudaGetLastError(), "lq_minmax_noalloc launch");
}
