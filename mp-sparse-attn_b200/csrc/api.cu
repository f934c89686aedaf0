// Error state and small utilities of the C-ABI library.
#include "api_internal.h"
#include "common.cuh"

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

namespace mpsa {
// One thread waits on an mbarrier that nothing arrives at, with the bounded wait every kernel of the library uses.
__global__ void selftest_wait_kernel(int* status, long long limit, int code) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    mbar_wait(&bar, 0, status, code, limit);      // expires: records `code` in *status and returns
  }
}
}  // namespace mpsa

extern "C" int mpsa_selftest_wait_timeout(int* status, long long limit_cycles, int code, void* stream) {
  if (!status) return mpsa::set_error(MPSA_ERR_BAD_ARG, "selftest_wait_timeout: null status");
  if (limit_cycles < 1 || limit_cycles > 2000000000ll)
    return mpsa::set_error(MPSA_ERR_BAD_ARG, "selftest_wait_timeout: limit must be 1 .. 2e9 cycles");
  if (code < 1 || code > 3) return mpsa::set_error(MPSA_ERR_BAD_ARG, "selftest_wait_timeout: code must be 1, 2 or 3");
  mpsa::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, limit_cycles, code);
  return mpsa::check_launch("selftest_wait_timeout");
}
