// Error state and small utilities of the C-ABI library.
#include "api_internal.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace mpsa {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(MPSA_ERR_LAUNCH, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return MPSA_OK;
}

}  // namespace mpsa

extern "C" int mpsa_last_error(char* buf, unsigned long long n) {
  if (!buf || n == 0) return MPSA_ERR_BAD_ARG;
  strncpy(buf, mpsa::g_err, n - 1);
  buf[n - 1] = 0;
  return MPSA_OK;
}

extern "C" int mpsa_version(void) { return 100; }
