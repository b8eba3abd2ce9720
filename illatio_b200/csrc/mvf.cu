// mvf.cu -- small dense products with unquantized weights: the router's logits and the other F16 /
// BF16 / F32 tensors that sit between the quantized products (DK-MV16, src/cuda-ds4f.lisp:767-771:
// d4_mv_f16 src/cuda/ds4f.cu:145-165, g53_mv_bf16 src/cuda/glm53.cu:11, d41_mv_f32
// src/cuda/ds4f_v41.cu:204, and their several-token forms d4_mv_f16n / d41_mv_f32n).  The CPU path is
// F32MV! (src/ds4f.lisp:256-276) on the weights widened to float: a float dot a row.
//
// Pure bandwidth and small (the router of a 256-expert layer is 2 MB): a warp a row, 16-byte loads of
// the row, the tokens' activations from L1/L2, fp32 accumulate, one shuffle reduction a (row, token).
#include <cuda_bf16.h>

#include "common.cuh"
#include "host.h"

namespace ill {

template <int TYPE> struct DenseElt;
template <> struct DenseElt<ILL_F32> { static constexpr int BYTES = 4; };
template <> struct DenseElt<ILL_F16> { static constexpr int BYTES = 2; };
template <> struct DenseElt<ILL_BF16> { static constexpr int BYTES = 2; };

template <int TYPE>
__device__ __forceinline__ float dense_at(const u8* row, int j) {
  if constexpr (TYPE == ILL_F32) return ((const float*)row)[j];
  else if constexpr (TYPE == ILL_F16) return __half2float(((const __half*)row)[j]);
  else return __bfloat162float(((const __nv_bfloat16*)row)[j]);
}
// eight (four for F32) consecutive weights from a 16-byte load, as floats
template <int TYPE>
__device__ __forceinline__ void dense_vec(const uint4 v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if constexpr (TYPE == ILL_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(w[i]);
  } else if constexpr (TYPE == ILL_F16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*(const __half2*)&w[i]);
      f[2 * i] = p.x; f[2 * i + 1] = p.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // a bfloat16 is the top half of a float
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}

constexpr int MVF_MAXN = 16;

// Y[t * y_stride + r] = W[r] . X[t], r < rows, t < n: blockIdx.y takes the tokens sixteen at a time (a chunk's
// router logits: the matrix is small and stays in L2 between the token batches).  A warp takes RW rows against the
// batch's tokens: one row for a token or a few (more warps in flight), four for a chunk (an activation vector
// loaded once serves four rows).
template <int TYPE, int RW>
__global__ void __launch_bounds__(256) mv_dense_kernel(const u8* __restrict__ w, int rows, int cols, const float* __restrict__ x,
                                                       float* __restrict__ y, int n, long long y_stride, int vec_ok) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * RW;
  if (r0 >= rows) return;
  {
    const long long t0 = (long long)blockIdx.y * MVF_MAXN;
    x += t0 * cols;
    y += t0 * y_stride;
    n = min(n - (int)t0, MVF_MAXN);
  }
  constexpr int EB = DenseElt<TYPE>::BYTES, VE = 16 / EB;  // elements a 16-byte load
  const u8* row[RW];
#pragma unroll
  for (int q = 0; q < RW; ++q) row[q] = w + (long long)min(r0 + q, rows - 1) * cols * EB;  // rows past the end repeat the last: not stored
  float sum[RW][MVF_MAXN];
#pragma unroll
  for (int q = 0; q < RW; ++q)
#pragma unroll
    for (int t = 0; t < MVF_MAXN; ++t) sum[q][t] = 0.0f;
  int j0 = 0;
  if (vec_ok) {  // rows and activations 16-byte aligned, cols a whole number of vectors
    const int nv = cols / VE;
    for (int i = lane; i < nv; i += 32) {
      float f[RW][8];
#pragma unroll
      for (int q = 0; q < RW; ++q) dense_vec<TYPE>(__ldg((const uint4*)row[q] + i), f[q]);
#pragma unroll
      for (int t = 0; t < MVF_MAXN; ++t) {
        if (t < n) {
          const float4* xv = (const float4*)(x + (long long)t * cols + (long long)i * VE);
          const float4 a = xv[0];
          float4 b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if constexpr (VE == 8) b = xv[1];
#pragma unroll
          for (int q = 0; q < RW; ++q) {
            float s = sum[q][t];
            s = fmaf(f[q][0], a.x, s); s = fmaf(f[q][1], a.y, s); s = fmaf(f[q][2], a.z, s); s = fmaf(f[q][3], a.w, s);
            if constexpr (VE == 8) {
              s = fmaf(f[q][4], b.x, s); s = fmaf(f[q][5], b.y, s); s = fmaf(f[q][6], b.z, s); s = fmaf(f[q][7], b.w, s);
            }
            sum[q][t] = s;
          }
        }
      }
    }
    j0 = nv * VE;
  }
  for (int j = j0 + lane; j < cols; j += 32) {
#pragma unroll
    for (int q = 0; q < RW; ++q) {
      const float wv = dense_at<TYPE>(row[q], j);
#pragma unroll
      for (int t = 0; t < MVF_MAXN; ++t)
        if (t < n) sum[q][t] = fmaf(wv, x[(long long)t * cols + j], sum[q][t]);
    }
  }
#pragma unroll
  for (int q = 0; q < RW; ++q)
#pragma unroll
    for (int t = 0; t < MVF_MAXN; ++t) {
      if (t < n) {
        const float v = warp_sum(sum[q][t]);
        if (lane == 0 && r0 + q < rows) y[(long long)t * y_stride + r0 + q] = v;
      }
    }
}

template <int RW>
static const void* mv_dense_fn(int type) {
  return type == ILL_F32 ? (const void*)mv_dense_kernel<ILL_F32, RW>
         : type == ILL_F16 ? (const void*)mv_dense_kernel<ILL_F16, RW> : (const void*)mv_dense_kernel<ILL_BF16, RW>;
}

}  // namespace ill

using namespace ill;

extern "C" int ill_mv_dense(int type, ill_dptr w, int rows, int cols, ill_dptr x, ill_dptr y, int n, int64_t y_stride,
                            ill_stream stream) {
  if ((type != ILL_F32 && type != ILL_F16 && type != ILL_BF16) || rows <= 0 || cols <= 0 || n < 1 || n > 65535 * MVF_MAXN || !w || !x ||
      !y || y_stride < rows)
    return ILL_ERR_ARG;
  const int eb = type == ILL_F32 ? 4 : 2;
  if ((w & (eb - 1)) || (x & 3) || (y & 3)) return ILL_ERR_ALIGN;
  const int ve = 16 / eb;
  int vec_ok = !(w & 15) && !(x & 15) && cols % ve == 0 && ((long long)cols * eb) % 16 == 0 && ((long long)cols * 4) % 16 == 0;
  const u8* wp = (const u8*)(uintptr_t)w;
  const float* xp = (const float*)(uintptr_t)x;
  float* yp = (float*)(uintptr_t)y;
  long long ys = y_stride;
  void* args[] = {&wp, &rows, &cols, &xp, &yp, &n, &ys, &vec_ok};
  const int rw = n > MVF_MAXN ? 4 : 1;
  const void* k = rw == 4 ? mv_dense_fn<4>(type) : mv_dense_fn<1>(type);
  return launch_kernel(k, dim3((unsigned)((rows + 8 * rw - 1) / (8 * rw)), (unsigned)((n + MVF_MAXN - 1) / MVF_MAXN)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}
