// Host-side error record: every entry point returns a code; the text of the last failure of the
// calling thread is read back through gi_last_error().
#include <stdarg.h>
#include <stdio.h>

#include "api.h"
#include "common.cuh"

namespace {
thread_local char g_last_error[512] = "";
}

namespace gi {
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return GI_OK;
}
}  // namespace gi

extern "C" const char* gi_last_error(void) { return g_last_error; }
extern "C" int gi_abi_version(void) { return GI_ABI_VERSION; }
