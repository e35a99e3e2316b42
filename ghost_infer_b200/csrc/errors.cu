// Host-side error record: every entry point returns a code; the text of the last failure of the
// calling thread is read back through gi_last_error().
#include <stdarg.h>
#include <stdio.h>

#include "api.h"
#include "common.cuh"

namespace {
thread_local char g_last_error[512] = "";
int g_pdl = 1;
}

namespace gi {
bool pdl_enabled() { return g_pdl != 0; }
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

// Switches programmatic dependent launch on or off for the kernels that support it (process-wide).
extern "C" void gi_set_pdl(int on) { g_pdl = on ? 1 : 0; }
extern "C" int gi_get_pdl(void) { return g_pdl; }
