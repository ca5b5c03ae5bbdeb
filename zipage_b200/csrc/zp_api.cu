// Error reporting and version of libzipage_b200.
#include <stdarg.h>
#include <stdio.h>

#include "zp_common.cuh"

namespace zp {
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return ZP_ERR_CUDA;
  }
  return ZP_OK;
}
}  // namespace zp

extern "C" const char* zp_last_error(void) { return zp::g_err; }
extern "C" int zp_version(void) { return 1; }
