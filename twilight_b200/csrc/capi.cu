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
}  // namespace twl

extern "C" int twl_version(void) { return 100; }

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
