// Error plumbing and version query of the C ABI.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace lq {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return LQ_OK;
  g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return LQ_ERR_CUDA;
}

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return dev;
}

int sm_count() {
  static std::mutex mu;
  static int count[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return kNumSMs;
  std::lock_guard<std::mutex> lock(mu);
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMs;
    count[dev] = n;
  }
  return count[dev];
}

static bool read_pdl_knob() {
  const char* e = getenv("LQ_PDL");
  return e == nullptr || atoi(e) != 0;
}
static bool g_pdl = read_pdl_knob();
bool pdl_enabled() { return g_pdl; }
void reload_pdl_knob() { g_pdl = read_pdl_knob(); }

}  // namespace lq

extern "C" int lq_version(void) { return LQ_VERSION; }

extern "C" int lq_last_error(char* buf, size_t n) {
  if (!buf || n == 0) return LQ_ERR_DEVICE;
  const std::string& s = lq::g_last_error;
  size_t k = s.size() < n - 1 ? s.size() : n - 1;
  memcpy(buf, s.data(), k);
  buf[k] = '\0';
  return LQ_OK;
}
