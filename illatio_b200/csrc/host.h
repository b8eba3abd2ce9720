// host.h -- host-side helpers shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>

namespace ill {

// Records E as the calling thread's last CUDA error and returns ILL_ERR_CUDA.
int cuda_fail(cudaError_t e);

// Address of the current device's status word (a __device__ variable of the
// library; no allocation).  Null if the address cannot be taken.
unsigned int* device_status_word();

// Whether launches carry the programmatic-stream-serialization attribute.
bool pdl_enabled();

// Launch FN (grid, block, dynamic shared bytes) on ST with ARGS, with the
// programmatic-dependent-launch attribute when enabled.
int launch_kernel(const void* fn, dim3 grid, dim3 block, size_t smem, void** args, cudaStream_t st);

}  // namespace ill
