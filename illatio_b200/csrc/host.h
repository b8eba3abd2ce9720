// host.h -- host-side helpers shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>

namespace ill {

// Records E as the calling thread's last CUDA error and returns ILL_ERR_CUDA.
int cuda_fail(cudaError_t e);

// Address of the current device's status word (a __device__ variable of the
// library; no allocation).  Null if the address cannot be taken.
unsigned int* device_status_word();

}  // namespace ill
