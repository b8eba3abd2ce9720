// lib.cu -- version, error text and the device status word.
#include "common.cuh"
#include "formats.cuh"
#include "host.h"

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

static int g_pdl = 1;
bool pdl_enabled() { return g_pdl != 0; }

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

}  // namespace ill

using namespace ill;

extern "C" int ill_set_pdl(int on) {
  const int prev = g_pdl;
  g_pdl = on ? 1 : 0;
  return prev;
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
