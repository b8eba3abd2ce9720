// quant.cu -- activation quantizers and rows-as-floats.
//
// The quantizers reproduce the reference's CPU routines bit for bit
// (QUANTIZE-Q8! src/tensor.lisp:245-262, QUANTIZE-Q8K! src/kquant.lisp:130-167):
// IEEE division and round-half-even conversion, no fused multiply-add, the
// first of equal maxima wins.  They are what lets the products on the device
// follow the CPU kernels instead of the reference's own CUDA kernels, which feed
// K-quants Q8_0 blocks (src/cuda/kquant.cu:3-14).
#include "formats.cuh"
#include "iq2xxs_tables.cuh"
#include "quantdev.cuh"
#include "host.h"

namespace ill {

__global__ void __launch_bounds__(256) quant_q8_0_kernel(const float* __restrict__ x, i8* __restrict__ xq,
                                                         float* __restrict__ xs, int* __restrict__ xsum,
                                                         long long nblocks, int f16_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const long long b = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  quant_block_q8_0(x[b * 32 + lane], lane, b, xq, xs, xsum, f16_scale);
}

// A warp a super-block; lane l holds elements 8l .. 8l+7.  F16: also the block's fp16 forms (XH, XE).
template <bool F16>
__global__ void __launch_bounds__(256) quant_q8_k_kernel(const float* __restrict__ x, i8* __restrict__ xq,
                                                         float* __restrict__ xd, int16_t* __restrict__ bsums,
                                                         long long nblocks, __half* __restrict__ xh, __half* __restrict__ xe) {
  pdl_launch_dependents();
  pdl_wait();
  const long long b = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  const float4 v0 = ((const float4*)(x + b * 256))[2 * lane], v1 = ((const float4*)(x + b * 256))[2 * lane + 1];
  const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  if constexpr (F16) quant_block_q8_k_f16(v, lane, b, xq, xd, bsums, xh, xe);
  else quant_block_q8_k(v, lane, b, xq, xd, bsums);
}

// RMSNORM! (src/model.lisp:205-216) fused with the activation quantizer, as the reference's rmsnorm_q8
// launch is (src/cuda/dense.cu:144-160, RMSNORM-Q8 src/cuda-dense.lisp:260-264): the squares (rounded to
// float) summed in double, scale = 1 / sqrt(float(sum / d + eps)), value = (x * scale) * w, then the
// blocks quantized as the stand-alone quantizers do.  Grid (slices, rows): every CTA of a row works the
// row's scale out for itself (the row comes from L2) and takes a slice of its blocks, so that one token's
// norm is not one CTA's serial work.  The double sum is taken in the order quantdev.cuh fixes, not in the
// CPU loop's; the two agree until the float the sum is rounded to sits within 1e-16 of a rounding boundary.
template <int K8K, bool F16>
__global__ void __launch_bounds__(256) rmsnorm_q8_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                         float* __restrict__ h, i8* __restrict__ xq, float* __restrict__ xs,
                                                         void* __restrict__ xsum, int d, float eps, int f16_scale,
                                                         __half* __restrict__ xh, __half* __restrict__ xe) {
  __shared__ double group_s[RMS_MAX_GROUPS];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long base = (long long)blockIdx.y * d;
  const float* xr = x + base;
  const int ng = (d + 255) / 256;
  for (int g = warp; g < ng; g += 8) {
    float v[8];
    rms_load8<false>(xr, d, g * 256 + 8 * lane, v);
    const double s = rms_group_sum(v);
    if (lane == 0) group_s[g] = s;
  }
  __syncthreads();
  const float sc = rms_scale(rms_total(group_s, ng, lane), d, eps);
  constexpr int BW = K8K ? 256 : 32;
  const int nb = d / BW;
  for (int b = blockIdx.x * 8 + warp; b < nb; b += gridDim.x * 8) {
    const long long gb = base / BW + b;
    if constexpr (K8K) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = b * 256 + 8 * lane + j;
        v[j] = __fmul_rn(__fmul_rn(xr[i], sc), w[i]);
        if (h) h[base + i] = v[j];
      }
      if constexpr (F16) quant_block_q8_k_f16(v, lane, gb, xq, xs, (int16_t*)xsum, xh, xe);
      else quant_block_q8_k(v, lane, gb, xq, xs, (int16_t*)xsum);
    } else {
      const int i = b * 32 + lane;
      const float v = __fmul_rn(__fmul_rn(xr[i], sc), w[i]);
      if (h) h[base + i] = v;
      quant_block_q8_0(v, lane, gb, xq, xs, (int*)xsum, f16_scale);
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(256) dequant_rows_kernel(const u8* __restrict__ w, int cols, long long row_bytes,
                                                           const int* __restrict__ row_ids, long long first_row,
                                                           float* __restrict__ out) {
  const int i = blockIdx.x;
  const long long row = row_ids ? (long long)row_ids[i] : first_row + i;
  const u8* rp = w + row * row_bytes;
  for (int c = blockIdx.y * 256 + threadIdx.x; c < cols; c += gridDim.y * 256)
    out[(long long)i * cols + c] = dequant_weight<FMT>(rp, c, ill_iq2xxs_grid, ill_ksigns_iq2xs);
}

}  // namespace ill

using namespace ill;

extern "C" int ill_quant_q8_0(ill_dptr x, ill_dptr xq, ill_dptr xs, ill_dptr xsum, int64_t nblocks, int f16_scale,
                              ill_stream stream) {
  if (nblocks < 0 || !x || !xq || !xs) return ILL_ERR_ARG;
  if ((x & 3) || (xs & 3) || (xsum & 3)) return ILL_ERR_ALIGN;
  if (nblocks == 0) return ILL_OK;
  const float* xp = (const float*)(uintptr_t)x;
  i8* qp = (i8*)(uintptr_t)xq;
  float* sp = (float*)(uintptr_t)xs;
  int* sump = (int*)(uintptr_t)xsum;
  long long nb = nblocks;
  void* args[] = {&xp, &qp, &sp, &sump, &nb, &f16_scale};
  return launch_kernel((const void*)quant_q8_0_kernel, dim3((unsigned)((nblocks + 7) / 8)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

static int quant_q8_k_launch(ill_dptr x, ill_dptr xq, ill_dptr xd, ill_dptr bsums, int64_t nblocks, ill_dptr xh, ill_dptr xe,
                             ill_stream stream) {
  if (nblocks < 0 || !x || !xq || !xd || !bsums) return ILL_ERR_ARG;
  if ((x & 15) || (xq & 7) || (xd & 3) || (bsums & 1) || (xh & 15) || (xe & 15)) return ILL_ERR_ALIGN;
  if (nblocks == 0) return ILL_OK;
  const float* xp = (const float*)(uintptr_t)x;
  i8* qp = (i8*)(uintptr_t)xq;
  float* dp = (float*)(uintptr_t)xd;
  int16_t* bp = (int16_t*)(uintptr_t)bsums;
  __half *hp = (__half*)(uintptr_t)xh, *ep = (__half*)(uintptr_t)xe;
  long long nb = nblocks;
  void* args[] = {&xp, &qp, &dp, &bp, &nb, &hp, &ep};
  const void* k = xh ? (const void*)quant_q8_k_kernel<true> : (const void*)quant_q8_k_kernel<false>;
  return launch_kernel(k, dim3((unsigned)((nblocks + 7) / 8)), dim3(256), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_quant_q8_k(ill_dptr x, ill_dptr xq, ill_dptr xd, ill_dptr bsums, int64_t nblocks,
                              ill_stream stream) {
  return quant_q8_k_launch(x, xq, xd, bsums, nblocks, 0, 0, stream);
}

extern "C" int ill_quant_q8_k_f16(ill_dptr x, ill_dptr xq, ill_dptr xd, ill_dptr bsums, ill_dptr xh, ill_dptr xe, int64_t nblocks,
                                  ill_stream stream) {
  if (!xh || !xe) return ILL_ERR_ARG;
  return quant_q8_k_launch(x, xq, xd, bsums, nblocks, xh, xe, stream);
}

static int rmsnorm_q8_launch(int kind, ill_dptr x, ill_dptr w, ill_dptr h, ill_dptr xq, ill_dptr xs, ill_dptr xsum, int d, float eps,
                             int64_t n, int f16_scale, ill_dptr xh, ill_dptr xe, ill_stream stream);

extern "C" int ill_rmsnorm_q8(int kind, ill_dptr x, ill_dptr w, ill_dptr h, ill_dptr xq, ill_dptr xs, ill_dptr xsum, int d,
                              float eps, int64_t n, int f16_scale, ill_stream stream) {
  return rmsnorm_q8_launch(kind, x, w, h, xq, xs, xsum, d, eps, n, f16_scale, 0, 0, stream);
}

extern "C" int ill_rmsnorm_q8k_f16(ill_dptr x, ill_dptr w, ill_dptr h, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr xh, ill_dptr xe,
                                   int d, float eps, int64_t n, ill_stream stream) {
  if (!xh || !xe || (xh & 15) || (xe & 15)) return ILL_ERR_ARG;
  return rmsnorm_q8_launch(1, x, w, h, xq, xs, xsum, d, eps, n, 0, xh, xe, stream);
}

static int rmsnorm_q8_launch(int kind, ill_dptr x, ill_dptr w, ill_dptr h, ill_dptr xq, ill_dptr xs, ill_dptr xsum, int d, float eps,
                             int64_t n, int f16_scale, ill_dptr xh, ill_dptr xe, ill_stream stream) {
  const int bw = kind == 1 ? 256 : 32;
  if ((kind != 0 && kind != 1) || d <= 0 || d % bw || n < 0 || n > 65535 || !x || !w || !xq || !xs || (kind == 1 && !xsum))
    return ILL_ERR_ARG;
  if (d > 256 * RMS_MAX_GROUPS) return ILL_ERR_TOO_LARGE;
  if ((x & 3) || (w & 3) || (h & 3) || (xs & 3) || (xsum & (kind == 1 ? 1 : 3)) || (kind == 1 && (xq & 7))) return ILL_ERR_ALIGN;
  if (n == 0) return ILL_OK;
  const float* xp = (const float*)(uintptr_t)x;
  const float* wp = (const float*)(uintptr_t)w;
  float* hp = (float*)(uintptr_t)h;
  i8* qp = (i8*)(uintptr_t)xq;
  float* sp = (float*)(uintptr_t)xs;
  void* bp = (void*)(uintptr_t)xsum;
  __half *fhp = (__half*)(uintptr_t)xh, *fep = (__half*)(uintptr_t)xe;
  void* args[] = {&xp, &wp, &hp, &qp, &sp, &bp, &d, &eps, &f16_scale, &fhp, &fep};
  // a single row is spread over its blocks; many rows take a CTA each
  const int nb = d / bw;
  const unsigned slices = n == 1 ? (unsigned)((nb + 7) / 8) : 1u;
  const void* k = kind == 1 ? (xh ? (const void*)rmsnorm_q8_kernel<1, true> : (const void*)rmsnorm_q8_kernel<1, false>)
                            : (const void*)rmsnorm_q8_kernel<0, false>;
  return launch_kernel(k, dim3(slices, (unsigned)n), dim3(256), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_dequant_rows(int fmt, ill_dptr w, int cols, ill_dptr row_ids, int64_t first_row, int nrows,
                                ill_dptr out, ill_stream stream) {
  const int bw = fmt_block_weights(fmt);
  if (!bw || cols <= 0 || cols % bw || nrows < 0 || !w || !out || first_row < 0) return ILL_ERR_ARG;
  if ((out & 3) || (row_ids & 3)) return ILL_ERR_ALIGN;
  if (nrows == 0) return ILL_OK;
  const long long row_bytes = (long long)(cols / bw) * fmt_block_bytes(fmt);
  const u8* wp = (const u8*)(uintptr_t)w;
  const int* ids = (const int*)(uintptr_t)row_ids;
  float* op = (float*)(uintptr_t)out;
  dim3 grid(nrows, (cols + 2047) / 2048 > 0 ? (cols + 2047) / 2048 : 1);
  cudaStream_t st = (cudaStream_t)stream;
  switch (fmt) {
    case ILL_Q8_0: dequant_rows_kernel<ILL_Q8_0><<<grid, 256, 0, st>>>(wp, cols, row_bytes, ids, first_row, op); break;
    case ILL_Q4_K: dequant_rows_kernel<ILL_Q4_K><<<grid, 256, 0, st>>>(wp, cols, row_bytes, ids, first_row, op); break;
    case ILL_Q6_K: dequant_rows_kernel<ILL_Q6_K><<<grid, 256, 0, st>>>(wp, cols, row_bytes, ids, first_row, op); break;
    case ILL_Q2_K: dequant_rows_kernel<ILL_Q2_K><<<grid, 256, 0, st>>>(wp, cols, row_bytes, ids, first_row, op); break;
    case ILL_IQ2_XXS:
      dequant_rows_kernel<ILL_IQ2_XXS><<<grid, 256, 0, st>>>(wp, cols, row_bytes, ids, first_row, op);
      break;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}
