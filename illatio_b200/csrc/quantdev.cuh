// quantdev.cuh -- the activation quantizers as warp-level device functions, shared by the stand-alone
// quantizer kernels (quant.cu) and the kernels that quantize their own input (decode.cu).
//
// Bit for bit the reference's CPU routines (QUANTIZE-Q8! src/tensor.lisp:245-262, QUANTIZE-Q8K!
// src/kquant.lisp:130-167): IEEE division and round-half-even conversion, no fused multiply-add, the
// first of equal maxima wins.  The output pointers may be global or shared memory.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace ill {

// One Q8_0 block: lane l holds element l.
// lane l's quant of element l of a Q8_0 block, and the scale to store for the block (all lanes)
__device__ __forceinline__ int q8_0_value(float v, int f16_scale, float& d_out) {
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
  d_out = f16_scale ? __half2float(__float2half_rn(d)) : d;
  return __float2int_rn(__fmul_rn(v, id));
}
__device__ __forceinline__ void quant_block_q8_0(float v, int lane, long long b, i8* xq, float* xs,
                                                 int* xsum, int f16_scale) {
  float d;
  const int q = q8_0_value(v, f16_scale, d);
  xq[b * 32 + lane] = (i8)q;
  if (xsum) {
    int t = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) xsum[b] = t;
  }
  if (lane == 0) xs[b] = d;
}

// One Q8_K super-block: lane l holds elements 8l .. 8l+7.  Its eight quants Q and the block's scale D (all lanes).
__device__ __forceinline__ void q8k_values(const float (&v)[8], int lane, int (&q)[8], float& d) {
  // the largest magnitude, the first of equal ones, and the value that has it
  float amax = 0.0f, mx = 0.0f;
  int idx = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float a = fabsf(v[j]);
    if (a > amax) { amax = a; mx = v[j]; idx = 8 * lane + j; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, o), om = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
  }
  d = 0.0f;
  // A block whose largest magnitude is so small (below 3.8e-37) that -127 / max overflows is taken as zeros: the
  // reference's arithmetic is not defined there (an infinite scale times zero), and such values add nothing.
  const float iscale = amax == 0.0f ? 0.0f : __fdiv_rn(-127.0f, mx);
  if (amax == 0.0f || fabsf(iscale) > 3.402823466e38f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = 0;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = min(127, __float2int_rn(__fmul_rn(iscale, v[j])));
    d = __fdiv_rn(1.0f, iscale);
  }
}
// the lane's eight quants as two words, and their sum
__device__ __forceinline__ int q8k_pack(const int (&q)[8], uint32_t& w0, uint32_t& w1) {
  int s = 0;
  w0 = 0; w1 = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    s += q[j] + q[4 + j];
    w0 |= (uint32_t)(q[j] & 0xff) << (8 * j);
    w1 |= (uint32_t)(q[4 + j] & 0xff) << (8 * j);
  }
  return s;
}

// One Q8_K super-block quantized into block B of the row's arrays.
__device__ __forceinline__ void quant_block_q8_k(const float (&v)[8], int lane, long long b, i8* xq,
                                                 float* xd, int16_t* bsums) {
  int q[8];
  float d;
  q8k_values(v, lane, q, d);
  uint32_t w0, w1;
  int s = q8k_pack(q, w0, w1);
  ((uint2*)(xq + b * 256))[lane] = make_uint2(w0, w1);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (!(lane & 1)) bsums[b * 16 + (lane >> 1)] = (int16_t)s;
  if (lane == 0) xd[b] = d;
}

// The same, and the block's fp16 forms for the tcgen05 products beside it (what act_f16_kernel makes of the bytes):
// XH[b*256 ..] the quants as halves, XE[b*64 ..] the sixteen sums of 16 as halves followed by 48 zeros.
__device__ __forceinline__ void quant_block_q8_k_f16(const float (&v)[8], int lane, long long b, i8* xq, float* xd,
                                                     int16_t* bsums, __half* xh, __half* xe) {
  int q[8];
  float d;
  q8k_values(v, lane, q, d);
  uint32_t w0, w1;
  int s = q8k_pack(q, w0, w1);
  ((uint2*)(xq + b * 256))[lane] = make_uint2(w0, w1);
  uint32_t h[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __half2 hh = __floats2half2_rn((float)q[2 * j], (float)q[2 * j + 1]);
    h[j] = *(const uint32_t*)&hh;
  }
  ((uint4*)(xh + b * 256))[lane] = make_uint4(h[0], h[1], h[2], h[3]);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (!(lane & 1)) {
    bsums[b * 16 + (lane >> 1)] = (int16_t)s;
    xe[b * 64 + (lane >> 1)] = __float2half_rn((float)s);
  }
  if (lane < 24) ((uint32_t*)(xe + b * 64 + 16))[lane] = 0u;
  if (lane == 0) xd[b] = d;
}

// ---- RMSNorm's sum of squares, in an order that depends on the row's length only ----------------
// Every kernel that normalizes (the stand-alone rmsnorm_q8 and the chain kernel's prologue) adds the squares in
// this order, so they agree to the bit whatever their thread counts: the row in groups of 256; in a group lane l
// of a warp squares its eight elements 8l .. 8l+7 (each square rounded to float, as RMSNORM! squares in single
// precision, src/model.lisp:205-216) and adds them in order in double, the lanes meet by xor-shuffle 16, 8, .. 1;
// the groups' sums are then added by a warp: lane l adds groups l, l+32, .. in order, and the lanes meet the same way.
constexpr int RMS_MAX_GROUPS = 256;  // rows of up to 65536 values

// CG: read around L1 (the values may have been written earlier in the same launch)
template <bool CG>
__device__ __forceinline__ void rms_load8(const float* x, int d, int i0, float (&v)[8]) {
  if (i0 + 8 <= d && (((uintptr_t)(x + i0)) & 15) == 0) {
    const float4 a = CG ? __ldcg((const float4*)(x + i0)) : *(const float4*)(x + i0);
    const float4 b = CG ? __ldcg((const float4*)(x + i0) + 1) : *((const float4*)(x + i0) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = i0 + j < d ? (CG ? __ldcg(x + i0 + j) : x[i0 + j]) : 0.0f;
  }
}
// the group's sum of squares from the lanes' values (all lanes get it)
__device__ __forceinline__ double rms_group_sum(const float (&v)[8]) {
  double s = 0.0;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += (double)__fmul_rn(v[j], v[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  return s;
}
// the row's sum from the NG group sums G (shared memory; all lanes get it)
__device__ __forceinline__ double rms_total(const double* G, int ng, int lane) {
  double s = 0.0;
  for (int g = lane; g < ng; g += 32) s += G[g];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  return s;
}
__device__ __forceinline__ float rms_scale(double total, int d, float eps) {
  return __fdiv_rn(1.0f, __fsqrt_rn((float)(total / (double)d + (double)eps)));
}

}  // namespace ill
