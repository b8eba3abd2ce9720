// quantdev.cuh -- the activation quantizers as warp-level device functions, shared by the stand-alone
// quantizer kernels (quant.cu) and the kernels that quantize their own input (decode.cu).
//
// Bit for bit the reference's CPU routines (QUANTIZE-Q8! src/tensor.lisp:245-262, QUANTIZE-Q8K!
// src/kquant.lisp:130-167): IEEE division and round-half-even conversion, no fused multiply-add, the
// first of equal maxima wins.  The output pointers may be global or shared memory.
#pragma once
#include "common.cuh"

namespace ill {

// One Q8_0 block: lane l holds element l.
__device__ __forceinline__ void quant_block_q8_0(float v, int lane, long long b, i8* xq, float* xs,
                                                 int* xsum, int f16_scale) {
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
  const int q = __float2int_rn(__fmul_rn(v, id));
  xq[b * 32 + lane] = (i8)q;
  if (xsum) {
    int t = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) xsum[b] = t;
  }
  if (lane == 0) xs[b] = f16_scale ? __half2float(__float2half_rn(d)) : d;
}

// One Q8_K super-block: lane l holds elements 8l .. 8l+7.
__device__ __forceinline__ void quant_block_q8_k(const float (&v)[8], int lane, long long b, i8* xq,
                                                 float* xd, int16_t* bsums) {
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
  int q[8];
  float d = 0.0f;
  if (amax == 0.0f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = 0;
  } else {
    const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = min(127, __float2int_rn(__fmul_rn(iscale, v[j])));
    d = __fdiv_rn(1.0f, iscale);
  }
  int s = 0;
  uint32_t w0 = 0, w1 = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    s += q[j] + q[4 + j];
    w0 |= (uint32_t)(q[j] & 0xff) << (8 * j);
    w1 |= (uint32_t)(q[4 + j] & 0xff) << (8 * j);
  }
  ((uint2*)(xq + b * 256))[lane] = make_uint2(w0, w1);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (!(lane & 1)) bsums[b * 16 + (lane >> 1)] = (int16_t)s;
  if (lane == 0) xd[b] = d;
}

}  // namespace ill
