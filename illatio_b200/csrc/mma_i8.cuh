// The legacy tensor-core path for 8-bit integers (mma.sync m16n8k32 / m16n8k16) and the small loads around it,
// shared by the several-token product (mvt.cu) and the dense chunk product (mmd.cu).
//
// Fragment layout, lane = 4 g + t: A (16 rows x K): a0 = row g, k 4t..4t+3; a1 = row g + 8, same k; for k32 a2 / a3
// the same rows at k + 16.  B (K x 8 columns): b0 = column g, k 4t..4t+3; b1 (k32) at k + 16.  C: c0 / c1 = row g,
// columns 2t / 2t + 1; c2 / c3 = row g + 8.
#pragma once
#include "common.cuh"

namespace ill {

__device__ __forceinline__ void mma_k32(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], bool a_unsigned) {
  if (a_unsigned)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_k16_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0));
}

// a 32-bit word at any byte address of shared memory
__device__ __forceinline__ uint32_t lds32u(const u8* p) {
  const uint32_t mis = (uint32_t)(uintptr_t)p & 3u;
  const uint32_t* b = (const uint32_t*)(p - mis);
  return __funnelshift_r(b[0], b[1], 8u * mis);
}
__device__ __forceinline__ float ldh(const u8* p) { return h2f(*(const u16*)p); }  // p is 2-byte aligned

__device__ __forceinline__ void mma_k16_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0, bool b_unsigned) {
  if (b_unsigned)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// get_scale_min_k4 (src/kquant.lisp:64-72) for group J of the 12 packed bytes at Q
__device__ __forceinline__ void scale_min_k4(const u8* q, int j, int& sc, int& mn) {
  if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
  else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

}  // namespace ill
