// common.cuh -- shared device helpers for the sm_100a kernels.
//
// Bulk asynchronous copies (cp.async.bulk) land raw GGUF bytes in shared
// memory; an mbarrier per stage counts the bytes.  Every wait on an mbarrier is
// bounded in time (ILL_WAIT_NS): a waiter that gives up records a code in the
// device status word and returns false, and the kernel unwinds without touching
// the stage, so a lost copy can never hang the GPU.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/illatio_b200.h"

#define ILL_WAIT_NS 2000000000ull  // a wait on an mbarrier gives up after two seconds

namespace ill {

typedef unsigned char u8;
typedef signed char i8;
typedef unsigned short u16;

// device status codes (written once, first writer wins)
enum { ST_OK = 0, ST_MV_WAIT = 0x100, ST_MM_WAIT_FULL = 0x200, ST_MM_WAIT_EMPTY = 0x300,
       ST_MM_WAIT_ACC = 0x400, ST_MM_WAIT_EPI = 0x500,
       ST_GROUP_SEL = 0x600 /* an expert number out of range in ill_moe_group's SEL */,
       ST_BARRIER_WAIT = 0x700 /* a barrier between CTAs or ranks never completed */,
       ST_TEST_WAIT = 0x800 /* ill_test_wait_timeout: the wait that is meant to run out */ };

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
// One poll: the thread may be suspended by the hardware for up to HINT_NS nanoseconds while the
// phase is incomplete (it takes no issue slots meanwhile).
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up about LIMIT_NS (by default ILL_WAIT_NS) nanoseconds after it began.  Returns false (and records CODE
// in the status word, first writer wins) when the phase never completes.  SLEEP_NS > 0 makes the
// waiter sleep between polls, so that a warp with slack leaves the issue slots to the others; the
// clock is read once in 64 polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* status, unsigned int code,
                                          unsigned sleep_ns = 0, unsigned long long limit_ns = ILL_WAIT_NS) {
  if (mbar_try_wait(bar, parity, 0)) return true;
  unsigned long long t0 = 0;
  for (unsigned it = 1;; ++it) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity, 20000)) return true;
    if ((it & 63u) == 0) {
      const unsigned long long now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) break;
    }
  }
  if (status) atomicCAS(status, 0u, code);
  return false;
}

// ---- ranks meet without a collective: flags in peer memory -------------------------------------
// Every rank owns an array of flags, EP_FLAG_SLOTS x EP_MAX_RANKS words, that its peers can store into
// (FLAG_PEERS[r] = the address of rank r's array).  A meeting in slot S with number EPOCH (counted up by the
// caller, the same on every rank): thread t < WORLD of the calling block stores EPOCH into rank t's
// flags[S][RANK] (a release at system scope: what this rank stored into peer memory before is visible to a
// peer that sees the flag), then waits until its own flags[S][t] has reached EPOCH.  The wait is bounded
// (WAIT_NS, 0 = ILL_WAIT_NS): on a time-out the status word gets ST_BARRIER_WAIT and the call returns false.
// No rank waits for anything but stores its peers make unconditionally, so ranks that run their kernels at
// different times cannot deadlock each other.
constexpr int EP_MAX_RANKS = 64, EP_FLAG_SLOTS = 4;

// A CTA's ticket on a device counter, taken by one thread after the CTA's barrier: release orders the CTA's stores
// (cumulative through the barrier) before the ticket, acquire lets the CTA that takes the last ticket see every
// other CTA's -- so that its one system-wide release (the signal of ep_meet) covers the whole grid's stores, with
// no system-wide fence in the other CTAs.
__device__ __forceinline__ unsigned take_ticket(unsigned* counter) {
  unsigned old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}
__device__ __forceinline__ bool ep_meet(const unsigned long long* flag_peers, unsigned* flags, int world, int rank, int slot,
                                        unsigned epoch, bool signal, unsigned long long wait_ns, unsigned int* status) {
  const int t = threadIdx.x;
  if (t >= world) return true;
  if (signal) {
    // a release at system scope: this thread's earlier stores, and those of other threads that it has observed
    // through a barrier or an acquire, are visible to whoever acquires the flag (no separate fence.sc needed)
    unsigned* dst = (unsigned*)(uintptr_t)flag_peers[t] + slot * EP_MAX_RANKS + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
  }
  const unsigned* mine = flags + slot * EP_MAX_RANKS + t;
  const unsigned long long limit = wait_ns ? wait_ns : ILL_WAIT_NS;
  unsigned long long t0 = 0;
  for (unsigned it = 1;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - epoch) >= 0) return true;
    if ((it & 255u) == 0) {
      const unsigned long long now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit) {
        if (status) atomicCAS(status, 0u, (unsigned)ST_BARRIER_WAIT);
        return false;
      }
    }
  }
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

__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace ill
