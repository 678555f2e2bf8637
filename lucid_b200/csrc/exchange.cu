// Flag protocol of the exchange step of a sharded layer (one process per GPU, buffers and flag
// words in memory every rank has mapped): a producer stores its tiles into the peers' buffers
// and then publishes its step count to its flag word on each peer; a consumer waits until the
// flag words of all producers have reached its own step count.  Only plain stores and loads
// cross NVLink (release / acquire at system scope); no collective library call, so a whole
// step can be captured in a CUDA graph.  Every wait is bounded and reports LQ_ERR_TIMEOUT
// through a status word instead of spinning forever.
#include "common.cuh"

namespace lq {
namespace {

struct FlagList {
  int32_t* p[8];
  int n;
};

__global__ void peer_signal_kernel(FlagList flags, int32_t* counter) {
  if (threadIdx.x != 0) return;
  // kernels enqueued before this one have completed; the fence orders their stores (as observed
  // by this thread) before the flag stores for every observer in the system
  __threadfence_system();
  const int v = *counter + 1;
  *counter = v;
  for (int i = 0; i < flags.n; ++i)
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.p[i]), "r"(v) : "memory");
}

__global__ void peer_wait_kernel(const int32_t* flags, int n, int32_t* epoch, long long budget,
                                 int32_t* status) {
  const int lane = threadIdx.x;
  const int want = *epoch + 1;
  bool ok = true;
  if (lane < n) {
    const long long t0 = clock64();
    for (unsigned it = 1;; ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
      if (v - want >= 0) break;  // the producers count steps too: "at least", wrap-safe
      __nanosleep(200);
      if ((it & 15u) == 0 && clock64() - t0 > budget) {
        ok = false;
        break;
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  __threadfence_system();
  if (lane == 0) {
    *epoch = want;  // also after a timeout, so that later steps line up again
    if (!ok && status) atomicExch(status, (int)LQ_ERR_TIMEOUT);
  }
}

}  // namespace
}  // namespace lq

using namespace lq;

extern "C" int lq_peer_signal(int32_t* const* peer_flags, int n_flags, int32_t* signal_counter, void* stream) {
  if (!peer_flags || !signal_counter) return fail(LQ_ERR_DEVICE, "lq_peer_signal: null pointer");
  if (n_flags < 1 || n_flags > 8) return fail(LQ_ERR_SHAPE, "lq_peer_signal: between 1 and 8 flag words");
  FlagList fl;
  fl.n = n_flags;
  for (int i = 0; i < n_flags; ++i) {
    if (!peer_flags[i]) return fail(LQ_ERR_DEVICE, "lq_peer_signal: null flag address");
    fl.p[i] = peer_flags[i];
  }
  peer_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(fl, signal_counter);
  return check_cuda(cudaGetLastError(), "lq_peer_signal launch");
}

extern "C" int lq_peer_wait(const int32_t* flags, int n, int32_t* epoch, long long timeout_cycles,
                            int32_t* status, void* stream) {
  if (!flags || !epoch) return fail(LQ_ERR_DEVICE, "lq_peer_wait: null pointer");
  if (n < 1 || n > 32) return fail(LQ_ERR_SHAPE, "lq_peer_wait: between 1 and 32 flag words");
  const long long budget = timeout_cycles > 0 ? timeout_cycles : (1ll << 31);
  peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, epoch, budget, status);
  return check_cuda(cudaGetLastError(), "lq_peer_wait launch");
}
