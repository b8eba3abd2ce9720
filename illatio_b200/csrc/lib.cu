// lib.cu -- version, error text and the device status word.
#include "common.cuh"
#include "formats.cuh"
#include "host.h"

#include <stdlib.h>

namespace ill {

// Written by a kernel that gave up a bounded wait (first code wins).
__device__ unsigned int g_status_word;

static thread_local int t_last_cuda = 0;

int cuda_fail(cudaError_t e) {
  t_last_cuda = (int)e;
  (void)cudaGetLastError();  // clear the sticky-less error state
  return ILL_ERR_CUDA;
}

unsigned int* device_status_word() {
  unsigned int* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_status_word) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return p;
}

// Programmatic dependent launch is on unless the environment says ILL_PDL=0 when the library is
// loaded; it cannot be changed afterwards (the library keeps no mutable process-wide state).
static const bool g_pdl = [] {
  const char* v = getenv("ILL_PDL");
  return !(v && v[0] == '0');
}();
bool pdl_enabled() { return g_pdl; }

int launch_kernel(const void* fn, dim3 grid, dim3 block, size_t smem, void** args, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = g_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}

// A wait that is meant to run out: one warp waits LIMIT_NS for a phase of an mbarrier nobody arrives at, through
// the same bounded wait every kernel of the library uses.  It records ST_TEST_WAIT and returns.
__global__ void __launch_bounds__(32) test_wait_kernel(unsigned long long limit_ns, unsigned int* status, unsigned int* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  __syncwarp();
  const bool ok = mbar_wait(&bar, 0u, status, ST_TEST_WAIT, 0, limit_ns);
  if (threadIdx.x == 0 && gave_up) *gave_up = ok ? 0u : 1u;
}

}  // namespace ill

using namespace ill;

extern "C" int ill_test_wait_timeout(int64_t limit_ns, ill_dptr gave_up, ill_stream stream) {
  if (limit_ns < 1000 || limit_ns > 100000000ll || (gave_up & 3)) return ILL_ERR_ARG;  // 1 us .. 100 ms
  unsigned long long lim = (unsigned long long)limit_ns;
  unsigned int* st = device_status_word();
  unsigned int* gu = (unsigned int*)(uintptr_t)gave_up;
  void* args[] = {&lim, &st, &gu};
  return launch_kernel((const void*)test_wait_kernel, dim3(1), dim3(32), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_b200_version(void) { return 100; }

extern "C" const char* ill_error_string(int code) {
  switch (code) {
    case ILL_OK: return "ok";
    case ILL_ERR_ARG: return "bad argument: a size or flag is out of range, or a required pointer is null";
    case ILL_ERR_ALIGN: return "a pointer or stride is not aligned as the function requires";
    case ILL_ERR_UNSUPPORTED: return "no kernel for this shape";
    case ILL_ERR_CUDA: return "a CUDA runtime call failed (see ill_last_cuda_error)";
    case ILL_ERR_DEVICE_WAIT: return "a kernel gave up a bounded wait";
    case ILL_ERR_TOO_LARGE: return "a size exceeds a fixed maximum of this entry point";
  }
  return "unknown illatio_b200 status";
}

extern "C" int ill_last_cuda_error(void) { return t_last_cuda; }

extern "C" int ill_block_bytes(int fmt) { return fmt_block_bytes(fmt); }
extern "C" int ill_block_weights(int fmt) { return fmt_block_weights(fmt); }

extern "C" int ill_device_status(unsigned int* out, ill_stream stream) {
  if (!out) return ILL_ERR_ARG;
  unsigned int* p = device_status_word();
  if (!p) return cuda_fail(cudaErrorInvalidSymbol);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e);
  unsigned int v = 0;
  e = cudaMemcpyAsync(&v, p, sizeof v, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(p, 0, sizeof v, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e);
  *out = v;
  return v ? ILL_ERR_DEVICE_WAIT : ILL_OK;
}
