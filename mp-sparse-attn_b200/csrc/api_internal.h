// Error plumbing shared by the C-ABI entry points: every entry returns 0 on success or a negative
// code, and leaves a message retrievable with mpsa_last_error().  No exception crosses the
// boundary and nothing here allocates device memory.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#define MPSA_OK 0
#define MPSA_ERR_BAD_ARG (-1)
#define MPSA_ERR_UNSUPPORTED (-2)
#define MPSA_ERR_LAUNCH (-3)
#define MPSA_ERR_TIMEOUT (-4)

namespace mpsa {
int set_error(int code, const char* fmt, ...);
int check_launch(const char* what);
// launchers shared between translation units; run_if: a device word, the kernels do nothing while it is zero (may be null)
int launch_route_stat(const void* q4, const void* q4_sf, const void* k4, const void* k4_sf, void* stat, void* scratch, int B,
                      int Hq, int Hkv, int S, int Skv, int causal, int* status, const int* run_if, void* stream);
int launch_route_online(void* map, const void* stat, int B, int Hq, int S, int Skv, int causal, int band, float tau,
                        float skip_tau, int use_skip, const int* run_if, void* stream);
}  // namespace mpsa
