// Quantized embedding tables: gather + dequantize of the rows that are asked for.
// The reference dequantizes the WHOLE table to float32 on every forward and then gathers
// (lucid/nn/quantized/sparse.py:141-146, 292-301); here only the looked-up rows are read, as
// int8 codes, and decoded on the way out: (float(q) - zero_point[row]) * scale[row], the
// arithmetic of dequantize(..., ch_axis=0) (lucid/quantization/_functional.py:269-281).
//
// Row semantics follow the engine's CPU kernels: embedding_forward writes zeros for
// idx == padding_idx (lucid/_C/backend/cpu/CpuBackend.h:8970-9010); embedding_bag_forward
// (CpuBackend.h:5989-6080) walks each bag in index order, skips padding and out-of-range
// indices, sums in float32, divides a mean by the number of rows it added, and seeds a max
// with the lowest float (an empty bag gives zeros).
#include "common.cuh"

namespace lq {
namespace {

constexpr int kEmbThreads = 256;

template <typename Idx>
__device__ __forceinline__ long long read_index(const void* p, size_t k) {
  return (long long)reinterpret_cast<const Idx*>(p)[k];
}

__device__ __forceinline__ void decode4(uint32_t w, float z, float s, float (&v)[4]) {
#pragma unroll
  for (int b = 0; b < 4; ++b) v[b] = __fmul_rn(__fsub_rn((float)(int8_t)((w >> (8 * b)) & 0xffu), z), s);
}

// One warp per looked-up row.
template <typename Idx, typename Out>
__global__ void __launch_bounds__(kEmbThreads)
embedding_kernel(const int8_t* __restrict__ w, const float* __restrict__ scale, const float* __restrict__ zp,
                 long long num_emb, size_t dim, const void* __restrict__ idx, size_t n_idx, long long padding_idx,
                 Out* __restrict__ out, bool vec, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (kEmbThreads / 32);
  for (size_t r = (size_t)blockIdx.x * (kEmbThreads / 32) + (threadIdx.x >> 5); r < n_idx; r += warps) {
    const long long e = read_index<Idx>(idx, r);
    Out* dst = out + r * dim;
    const bool bad = e < 0 || e >= num_emb;
    if (bad && lane == 0 && status) *status = LQ_ERR_SHAPE;  // recorded; the row is left zero
    const bool zero = bad || e == padding_idx;
    const int8_t* src = w + (zero ? 0 : e) * (long long)dim;
    const float s = zero ? 0.0f : __ldg(scale + e), z = zero ? 0.0f : __ldg(zp + e);
    if (vec) {
      for (size_t c = (size_t)lane * 16; c < dim; c += 32 * 16) {
        uint4 u = make_uint4(0, 0, 0, 0);
        if (!zero) u = ld_stream_u4(src + c);
        const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          if (!zero) decode4(ww[j], z, s, v);
          if (sizeof(Out) == 4) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + c + 4 * j) = make_float4(v[0], v[1], v[2], v[3]);
          } else {
            const uint32_t lo = f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16);
            const uint32_t hi = f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16);
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(dst) + c + 4 * j) = make_uint2(lo, hi);
          }
        }
      }
    } else {
      for (size_t c = lane; c < dim; c += 32) {
        const float v = zero ? 0.0f : __fmul_rn(__fsub_rn((float)src[c], z), s);
        if (sizeof(Out) == 4) reinterpret_cast<float*>(dst)[c] = v;
        else reinterpret_cast<uint16_t*>(dst)[c] = (uint16_t)f32_to_bf16_bits(v);
      }
    }
  }
}

// One thread per (bag, column group of four): the bag is walked in index order, so every
// column sees the reference's sequence of float32 additions.
template <typename Idx>
__global__ void __launch_bounds__(kEmbThreads)
embedding_bag_kernel(const int8_t* __restrict__ w, const float* __restrict__ scale, const float* __restrict__ zp,
                     long long num_emb, size_t dim, const void* __restrict__ idx, size_t n_idx,
                     const void* __restrict__ offsets, size_t n_bags, bool include_last, int mode,
                     long long padding_idx, float* __restrict__ out, bool vec) {
  const size_t groups = (dim + 3) / 4;
  const size_t total = n_bags * groups;
  for (size_t t = (size_t)blockIdx.x * kEmbThreads + threadIdx.x; t < total; t += (size_t)gridDim.x * kEmbThreads) {
    const size_t b = t / groups, c = (t % groups) * 4;
    const int ncol = dim - c < 4 ? (int)(dim - c) : 4;
    long long s0 = read_index<Idx>(offsets, b);
    long long e0 = (b + 1 < n_bags && !include_last) ? read_index<Idx>(offsets, b + 1) : (long long)n_idx;
    if (include_last && b == n_bags - 1) e0 = read_index<Idx>(offsets, n_bags - 1);
    if (s0 < 0) s0 = 0;
    if (e0 > (long long)n_idx) e0 = (long long)n_idx;
    float acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = mode == 2 ? -3.402823466e+38f : 0.0f;
    int count = 0;
    for (long long k = s0; k < e0; ++k) {
      const long long e = read_index<Idx>(idx, (size_t)k);
      if (e == padding_idx || e < 0 || e >= num_emb) continue;
      const float s = __ldg(scale + e), z = __ldg(zp + e);
      const int8_t* src = w + e * (long long)dim + c;
      float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (vec) {
        decode4(__ldg(reinterpret_cast<const uint32_t*>(src)), z, s, v);
      } else {
        for (int j = 0; j < ncol; ++j) v[j] = __fmul_rn(__fsub_rn((float)src[j], z), s);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = mode == 2 ? (v[j] > acc[j] ? v[j] : acc[j]) : __fadd_rn(acc[j], v[j]);
      ++count;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (mode == 2 && count == 0) acc[j] = 0.0f;
      if (mode == 1 && count > 0) acc[j] = __fdiv_rn(acc[j], (float)count);
    }
    float* dst = out + b * dim + c;
    for (int j = 0; j < ncol; ++j) dst[j] = acc[j];
  }
}

}  // namespace
}  // namespace lq

using namespace lq;

extern "C" int lq_embedding_s8(const int8_t* weight, const float* scale, const float* zero_point,
                               size_t num_embeddings, size_t dim, const void* indices, int index_bits,
                               size_t n_idx, const void* offsets, size_t n_bags, int include_last_offset,
                               int mode, long long padding_idx, void* out, int out_dtype, int32_t* status,
                               void* stream) {
  if (n_idx == 0 && !offsets) return LQ_OK;
  if (!weight || !scale || !zero_point || !out) return fail(LQ_ERR_DEVICE, "lq_embedding_s8: null pointer");
  if (n_idx && !indices) return fail(LQ_ERR_DEVICE, "lq_embedding_s8: null indices");
  if (index_bits != 32 && index_bits != 64) return fail(LQ_ERR_DTYPE, "lq_embedding_s8: indices must be int32 or int64");
  if (dim == 0 || num_embeddings == 0) return fail(LQ_ERR_SHAPE, "lq_embedding_s8: empty table");
  cudaStream_t st = (cudaStream_t)stream;
  if (!offsets) {
    if (out_dtype != LQ_F32 && out_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, "lq_embedding_s8: out_dtype");
    const bool vec = dim % 16 == 0 && aligned16(weight) && aligned16(out);
    const size_t want = (n_idx + kEmbThreads / 32 - 1) / (kEmbThreads / 32);
    const int grid = (int)(want < (size_t)sm_count() * 32 ? want : (size_t)sm_count() * 32);
#define LQ_EMB(IDX, OUT) \
  embedding_kernel<IDX, OUT><<<grid, kEmbThreads, 0, st>>>(weight, scale, zero_point, (long long)num_embeddings, dim, \
                                                            indices, n_idx, padding_idx, (OUT*)out, vec, status)
    if (index_bits == 64) {
      if (out_dtype == LQ_F32) LQ_EMB(long long, float); else LQ_EMB(long long, __nv_bfloat16);
    } else {
      if (out_dtype == LQ_F32) LQ_EMB(int, float); else LQ_EMB(int, __nv_bfloat16);
    }
#undef LQ_EMB
    return check_cuda(cudaGetLastError(), "lq_embedding_s8 launch");
  }
  if (out_dtype != LQ_F32) return fail(LQ_ERR_DTYPE, "lq_embedding_s8: bags are pooled in float32");
  if (mode < 0 || mode > 2) return fail(LQ_ERR_UNSUPPORTED, "lq_embedding_s8: mode must be 0 (sum), 1 (mean) or 2 (max)");
  if (n_bags == 0) return LQ_OK;
  const bool vec = dim % 4 == 0 && (reinterpret_cast<uintptr_t>(weight) & 3u) == 0;
  const size_t total = n_bags * ((dim + 3) / 4);
  const size_t want = (total + kEmbThreads - 1) / kEmbThreads;
  const int grid = (int)(want < (size_t)sm_count() * 32 ? want : (size_t)sm_count() * 32);
  if (index_bits == 64)
    embedding_bag_kernel<long long><<<grid, kEmbThreads, 0, st>>>(weight, scale, zero_point, (long long)num_embeddings,
                                                                  dim, indices, n_idx, offsets, n_bags,
                                                                  include_last_offset != 0, mode, padding_idx,
                                                                  (float*)out, vec);
  else
    embedding_bag_kernel<int><<<grid, kEmbThreads, 0, st>>>(weight, scale, zero_point, (long long)num_embeddings, dim,
                                                            indices, n_idx, offsets, n_bags, include_last_offset != 0,
                                                            mode, padding_idx, (float*)out, vec);
  return check_cuda(cudaGetLastError(), "lq_embedding_s8 launch");
}
