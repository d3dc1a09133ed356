// Internal host-side helpers shared by the translation units of libb200_autotune.so.
#pragma once
#include <cuda_runtime.h>

#include "../../include/b200_autotune.h"

namespace b200 {

// Records `msg` as the calling thread's last error and returns `code`.
int set_error(int code, const char* fmt, ...);
// Returns B200_OK, or records the CUDA error text and returns B200_ERR_CUDA.
int check_cuda(cudaError_t e, const char* what);

}  // namespace b200
