// Library-level entry points: version, status strings, last CUDA error.
#include <cstdlib>

#include "common.cuh"

namespace twl {
static thread_local cudaError_t g_last_error = cudaSuccess;
void set_last_cuda_error(cudaError_t e) { g_last_error = e; }
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("TWL_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}
int num_sms() {
  // One slot per device ordinal; a value is written once and is the same from any thread.
  constexpr int kMaxDev = 64;
  static int cache[kMaxDev] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
  int n = __atomic_load_n(&cache[dev], __ATOMIC_RELAXED);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    __atomic_store_n(&cache[dev], n, __ATOMIC_RELAXED);
  }
  return n;
}
}  // namespace twl

extern "C" int twl_version(void) { return 200; }

extern "C" const char* twl_status_string(int status) {
  switch (status) {
    case TWL_OK: return "ok";
    case TWL_ERR_BAD_ARG: return "bad argument (null pointer or inconsistent sizes)";
    case TWL_ERR_MISALIGNED: return "misaligned pointer or stride";
    case TWL_ERR_UNSUPPORTED: return "unsupported configuration (dtype, head_dim, group size)";
    case TWL_ERR_LAUNCH: return "CUDA launch failed";
    case TWL_ERR_TOO_LARGE: return "size exceeds a kernel or workspace limit";
    case TWL_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" const char* twl_last_cuda_error(void) { return cudaGetErrorString(twl::g_last_error); }
