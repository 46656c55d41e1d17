// Status strings and the last-CUDA-error record of the C ABI.
#include <stdio.h>
#include <string.h>

#include "ssw_common.cuh"

namespace ssw {
static thread_local char g_cuda_error[256] = "";
void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}
void set_error_text(const char* text) { snprintf(g_cuda_error, sizeof(g_cuda_error), "%s", text); }
}  // namespace ssw

extern "C" const char* ssw_status_string(int status) {
  switch (status) {
    case SSW_OK: return "ok";
    case SSW_E_INVALID: return "invalid argument";
    case SSW_E_RANGE: return "size outside the int32 domain of the layout";
    case SSW_E_UNSUPPORTED: return "configuration outside the compiled variants";
    case SSW_E_CUDA: return "CUDA runtime error";
    case SSW_E_WORKSPACE: return "workspace too small";
    default: return "unknown status";
  }
}

extern "C" const char* ssw_last_cuda_error(void) { return ssw::g_cuda_error; }

extern "C" int ssw_version(void) { return 100; }
