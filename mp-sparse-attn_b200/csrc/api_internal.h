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
}  // namespace mpsa
