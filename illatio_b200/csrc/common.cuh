// common.cuh -- shared device helpers for the sm_100a kernels.
//
// Bulk asynchronous copies (cp.async.bulk) land raw GGUF bytes in shared
// memory; an mbarrier per stage counts the bytes.  Every wait on an mbarrier is
// bounded: after ILL_SPIN_LIMIT polls the waiter records a code in the device
// status word and returns false, and the kernel unwinds without touching the
// stage, so a lost copy can never hang the GPU.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/illatio_b200.h"

#define ILL_SPIN_LIMIT (1u << 22)

namespace ill {

typedef unsigned char u8;
typedef signed char i8;
typedef unsigned short u16;

// device status codes (written once, first writer wins)
enum { ST_OK = 0, ST_MV_WAIT = 0x100, ST_MM_WAIT_FULL = 0x200, ST_MM_WAIT_EMPTY = 0x300,
       ST_MM_WAIT_ACC = 0x400, ST_MM_WAIT_EPI = 0x500 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records CODE) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* status, unsigned int code) {
  for (uint32_t i = 0; i < ILL_SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
  if (status) atomicCAS(status, 0u, code);
  return false;
}

// 1-D bulk copy global -> this CTA's shared memory; 16-byte aligned addresses
// and size.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue / wait until the previous kernel's memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// N consecutive 32-bit words starting at an arbitrarily aligned shared-memory
// byte address: aligned loads of N+1 words, realigned with funnel shifts.
template <int N>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&out)[N]) {
  const uint32_t base = addr & ~3u, sh = (addr & 3u) * 8u;
  uint32_t prev = lds32(base);
#pragma unroll
  for (int i = 0; i < N; ++i) {
    uint32_t next = lds32(base + 4u * (i + 1));
    out[i] = __funnelshift_r(prev, next, sh);
    prev = next;
  }
}

__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace ill
