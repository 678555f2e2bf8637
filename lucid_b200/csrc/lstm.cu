// Pointwise part of one LSTM time step (gate order i, f, g, o as in nn.LSTM):
//   c' = sigmoid(f) * c + sigmoid(i) * tanh(g);   h' = sigmoid(o) * tanh(c')
// on the pre-activations `gates` = x_t W_ih^T + b_ih + h W_hh^T + b_hh of a (batch, 4 * hidden)
// block.  The weight-only quantized LSTM (lucid/nn/quantized/dynamic/rnn.py:67-87) runs the
// float recurrence on dequantized weights; this kernel replaces the five element-wise passes
// per step of the float cell with one.
#include "common.cuh"

namespace lq {
namespace {

__device__ __forceinline__ float sigmoid_f32(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }

__global__ void __launch_bounds__(256)
lstm_cell_kernel(const float* __restrict__ gates, size_t ldg, const float* __restrict__ c_prev,
                 float* __restrict__ h_out, size_t ldh, float* __restrict__ c_out, size_t batch, size_t hidden) {
  const size_t n = batch * hidden;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t b = idx / hidden, j = idx - b * hidden;
    const float* g = gates + b * ldg;
    const float ig = sigmoid_f32(g[j]);
    const float fg = sigmoid_f32(g[hidden + j]);
    const float gg = tanhf(g[2 * hidden + j]);
    const float og = sigmoid_f32(g[3 * hidden + j]);
    const float c = __fadd_rn(__fmul_rn(fg, c_prev[idx]), __fmul_rn(ig, gg));
    c_out[idx] = c;
    h_out[b * ldh + j] = __fmul_rn(og, tanhf(c));
  }
}

}  // namespace
}  // namespace lq

using namespace lq;

extern "C" int lq_lstm_cell_f32(const float* gates, size_t ldg, const float* c_prev, float* h_out, size_t ldh,
                                float* c_out, size_t batch, size_t hidden, void* stream) {
  if (batch == 0 || hidden == 0) return LQ_OK;
  if (!gates || !c_prev || !h_out || !c_out) return fail(LQ_ERR_DEVICE, "lq_lstm_cell_f32: null pointer");
  if (ldg < 4 * hidden || ldh < hidden) return fail(LQ_ERR_SHAPE, "lq_lstm_cell_f32: row strides smaller than the rows");
  const size_t n = batch * hidden;
  size_t blocks = (n + 255) / 256;
  const size_t cap = (size_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  lstm_cell_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(gates, ldg, c_prev, h_out, ldh, c_out, batch, hidden);
  return check_cuda(cudaGetLastError(), "lq_lstm_cell_f32 launch");
}
