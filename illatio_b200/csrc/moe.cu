// moe.cu -- the routed experts' small kernels: routing, grouping rows by expert,
// the gated middle, the sums in slot order; and the per-expert products of a
// decoded token, which are the matvec kernels (mv.cu) run over a table of expert
// addresses.
//
// Replaces d4_mv_iq2_xxs / d4_mv_q2_k / d4_swiglu_w / d4_moe_sum
// (src/cuda/ds4f.cu:645,769,837,902) and d4_route / d4_group_* / d4_gather_rows /
// d4_moe_sum_rows (src/cuda/ds4f_chunk.cu:393-508) of the reference.
#include <cuda.h>
#include <string.h>

#include "formats.cuh"
#include "host.h"
#include "quantdev.cuh"

namespace ill {

// D4-SIGMOID (src/ds4f.lisp:248-250), each step rounded as written.
// (One exponential and one division whatever the sign -- 1 / (1 + e^-x) for x >= 0, e^x / (1 + e^x) below, both with
// e = exp(-|x|) -- so that a warp whose lanes differ in sign does not run both branches one after the other.)
__device__ __forceinline__ float d4_sigmoid(float x) {
  const float e = expf(-fabsf(x));
  return __fdiv_rn(x >= 0.0f ? 1.0f : e, __fadd_rn(1.0f, e));
}

// MID[r*ff + j] = silu(min(G, c)) * clamp(U, +-c) * W[r]  (src/ds4f.lisp:1016-1019)
__global__ void __launch_bounds__(256) swiglu_w_kernel(long long n, int ff, float clamp, const float* __restrict__ g,
                                                       const float* __restrict__ u, const float* __restrict__ w,
                                                       float* __restrict__ mid) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gv = g[i], uv = u[i];
  if (clamp > 1e-6f) { gv = fminf(gv, clamp); uv = fmaxf(-clamp, fminf(uv, clamp)); }
  const float wv = w ? w[i / ff] : 1.0f;
  mid[i] = __fmul_rn(__fmul_rn(__fmul_rn(gv, d4_sigmoid(gv)), uv), wv);
}

// MOE[t*d + r] = sum over the token's NU slots, in slot order, of DOWN[row(t, s)*d + r], plus SHARED
// (src/ds4f.lisp:1031-1036, 1226-1231).  MAP gives row(t, s) (null: t*nu + s).
// With MAP2, row(t, s) = MAP2[MAP[t*nu + s]] (an expert-parallel chunk: the slot a row left in, then where that
// slot's result came back).  With FLAG_PEERS the ranks meet first (slot 1): DOWN then holds rows that peers stored,
// complete once every peer has said so; block 0 says it for this rank (the kernel before this one in the stream
// stored this rank's rows into its peers).  DOWN is read around L1 in that case.
__global__ void __launch_bounds__(256) moe_sum_kernel(int d, int nu, long long ntok, const float* __restrict__ down,
                                                      const unsigned* __restrict__ map, const unsigned* __restrict__ map2,
                                                      const float* __restrict__ shared_, float* __restrict__ moe,
                                                      const unsigned long long* flag_peers, unsigned* flags, int world, int rank,
                                                      unsigned epoch, unsigned long long wait_ns, unsigned* status,
                                                      const unsigned* ovf_epoch, unsigned* ovf_flag, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  // the chunk's overflow as 0 / 1: its dispatch and its plan raise OVF_EPOCH to the chunk's number
  if (ovf_flag && blockIdx.x == 0 && threadIdx.x == 0) *ovf_flag = *ovf_epoch == epoch ? 1u : 0u;
  if (flag_peers) {
    const bool ok = ep_meet(flag_peers, flags, world, rank, 1, epoch, blockIdx.x == 0, wait_ns, status);
    if (!__syncthreads_and(ok)) return;
  }
  // The blocks stride over the outputs (so that a block meets the ranks once, not once per 256 outputs); VEC: four
  // outputs a thread from 16-byte loads.  Every output is the same chain of additions in slot order either way.
  const long long nthr = (long long)gridDim.x * blockDim.x, tid0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    const int d4 = d / 4;
    for (long long gid = tid0; gid < ntok * d4; gid += nthr) {
      const long long t = gid / d4;
      const int r = (int)(gid - t * d4);
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int s = 0; s < nu; ++s) {
        long long row = map ? (long long)map[t * nu + s] : t * nu + s;
        if (map2) row = map2[row];
        const float4* src = (const float4*)(down + row * d) + r;
        const float4 v = flag_peers ? __ldcg(src) : *src;
        acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
      }
      if (shared_) {
        const float4 v = ((const float4*)shared_)[gid];
        acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
      }
      ((float4*)moe)[gid] = acc;
    }
    return;
  }
  for (long long gid = tid0; gid < ntok * d; gid += nthr) {
    const long long t = gid / d;
    const int r = (int)(gid - t * d);
    float acc = 0.0f;
    for (int s = 0; s < nu; ++s) {
      long long row = map ? (long long)map[t * nu + s] : t * nu + s;
      if (map2) row = map2[row];
      acc = __fadd_rn(acc, flag_peers ? __ldcg(down + row * d + r) : down[row * d + r]);
    }
    moe[gid] = shared_ ? __fadd_rn(acc, shared_[gid]) : acc;
  }
}

// ---- routing -----------------------------------------------------------------------
// A warp a token.  MODE 0: p = sqrt(softplus(logit)) (D4-ROUTE, src/ds4f.lisp:950-978);
// MODE 2: p = sigmoid(logit) (G53-ROUTE, src/glm53.lisp:360-379).  The NU largest of
// p + bias, the earlier expert first among equals; weights p / max(sum p, 6.103515625e-5) * scale.
constexpr int ROUTE_MAX_PER_LANE = 16;  // up to 512 experts

__global__ void __launch_bounds__(128) route_kernel(int ne, int nu, int mode, float scale, long long ntok,
                                                    const float* __restrict__ logits, const float* __restrict__ bias,
                                                    unsigned* __restrict__ sel, float* __restrict__ wout) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= ntok) return;
  float p[ROUTE_MAX_PER_LANE], sc[ROUTE_MAX_PER_LANE];
#pragma unroll
  for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    p[j] = 0.0f;
    sc[j] = -INFINITY;
    if (e < ne) {
      const float l = logits[t * ne + e];
      float pv;
      if (mode == 2) pv = d4_sigmoid(l);
      else {
        const float sp = l > 20.0f ? l : (l < -20.0f ? expf(l) : logf(__fadd_rn(1.0f, expf(l))));
        pv = sqrtf(sp);
      }
      p[j] = pv;
      sc[j] = bias ? __fadd_rn(pv, bias[e]) : pv;
    }
  }
  float sum = 0.0f, mine = 0.0f;
  unsigned mysel = 0;
  for (int k = 0; k < nu; ++k) {
    // this lane's best (lowest index among equals: j ascending, strict >)
    float bv = -INFINITY;
    int bj = 0;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j)
      if (sc[j] > bv) { bv = sc[j]; bj = j; }
    int be = bj * 32 + lane;
    float v = bv;
    int e = be;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oe = __shfl_xor_sync(0xffffffffu, e, o);
      if (ov > v || (ov == v && oe < e)) { v = ov; e = oe; }
    }
    // the winner's lane takes it out of the running and reports its probability
    float pw = 0.0f;
    if ((e & 31) == lane) {
#pragma unroll
      for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j)
        if (j == (e >> 5)) { pw = p[j]; sc[j] = -INFINITY; }
    }
    pw = __shfl_sync(0xffffffffu, pw, e & 31);
    sum = __fadd_rn(sum, pw);
    if (lane == k) { mine = pw; mysel = (unsigned)e; }
  }
  if (sum < 6.103515625e-5f) sum = 6.103515625e-5f;
  if (lane < nu) {
    sel[t * nu + lane] = mysel;
    wout[t * nu + lane] = __fmul_rn(__fdiv_rn(mine, sum), scale);
  }
}

// ---- grouping (token, slot) rows by expert: a stable counting sort -------------------
// Rows are taken in blocks of GROUP_BLOCK; within a block a row's rank among its
// expert's rows follows row order (so an expert's rows stay in token order and
// the result does not depend on scheduling).
constexpr int GROUP_BLOCK = 1024;

// pass 1: per block, each expert's count; each row's rank inside its block
// An expert number >= NE (the caller's SEL is not trusted) is left out of every count and recorded in the status word.
__global__ void __launch_bounds__(GROUP_BLOCK) group_count_kernel(long long rows, int ne, const unsigned* __restrict__ sel,
                                                                  unsigned* __restrict__ block_counts,
                                                                  unsigned* __restrict__ rank, unsigned* __restrict__ status) {
  extern __shared__ unsigned gsm[];  // ne counters, then 32 * ne per-warp counters
  pdl_launch_dependents();
  pdl_wait();
  unsigned* warp_counts = gsm;  // [32][ne]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < 32 * ne; i += GROUP_BLOCK) warp_counts[i] = 0;
  __syncthreads();
  const long long row = (long long)blockIdx.x * GROUP_BLOCK + tid;
  bool valid = row < rows;
  unsigned e = valid ? sel[row] : 0xffffffffu;
  if (valid && e >= (unsigned)ne) {
    if (status) atomicCAS(status, 0u, (unsigned)ST_GROUP_SEL);
    valid = false;
    e = 0xffffffffu;
  }
  // rank within the warp: lanes below with the same expert
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const unsigned below = same & ((1u << lane) - 1u);
  const unsigned r_in_warp = __popc(below);
  if (valid && r_in_warp == 0) warp_counts[warp * ne + e] = __popc(same);  // one writer per (warp, expert)
  __syncthreads();
  // exclusive scan over the warps, per expert
  for (int x = tid; x < ne; x += GROUP_BLOCK) {
    unsigned run = 0;
    for (int w = 0; w < 32; ++w) {
      const unsigned c = warp_counts[w * ne + x];
      warp_counts[w * ne + x] = run;
      run += c;
    }
    block_counts[(long long)blockIdx.x * ne + x] = run;
  }
  __syncthreads();
  if (valid) rank[row] = warp_counts[warp * ne + e] + r_in_warp;
}

// pass 2 (one CTA): blocks scanned per expert, experts scanned -> COUNTS, BASES, block bases
__global__ void __launch_bounds__(512) group_scan_kernel(int nblocks, int ne, unsigned* __restrict__ block_counts,
                                                         unsigned* __restrict__ counts, unsigned* __restrict__ bases) {
  __shared__ unsigned tot[512];
  pdl_launch_dependents();
  pdl_wait();
  const int e = threadIdx.x;
  unsigned run = 0;
  if (e < ne)
    for (int b = 0; b < nblocks; ++b) {
      const unsigned c = block_counts[(long long)b * ne + e];
      block_counts[(long long)b * ne + e] = run;  // rows of expert e in earlier blocks
      run += c;
    }
  tot[e] = e < ne ? run : 0;
  __syncthreads();
  if (e == 0) {
    unsigned acc = 0;
    for (int i = 0; i < ne; ++i) { const unsigned c = tot[i]; tot[i] = acc; acc += c; }
  }
  __syncthreads();
  if (e < ne) { counts[e] = run; bases[e] = tot[e]; }
}

// pass 3: each row to its place; RMAP[place] = token, SMAP[row] = place, WROW[place] = weight
__global__ void __launch_bounds__(256) group_scatter_kernel(long long rows, int ne, int nu, const unsigned* __restrict__ sel,
                                                            const unsigned* __restrict__ rank,
                                                            const unsigned* __restrict__ block_counts,
                                                            const unsigned* __restrict__ bases, const float* __restrict__ w,
                                                            unsigned* __restrict__ rmap, unsigned* __restrict__ smap,
                                                            float* __restrict__ wrow) {
  pdl_launch_dependents();
  pdl_wait();
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const unsigned e = sel[row];
  if (e >= (unsigned)ne) { smap[row] = 0; return; }  // not an expert (flagged by the counting pass): the row has no place
  const unsigned place = bases[e] + block_counts[(row / GROUP_BLOCK) * ne + e] + rank[row];
  rmap[place] = (unsigned)(row / nu);
  smap[row] = place;
  if (wrow) wrow[place] = w[row];
}

// X[r] = SRC[MAP[r]] for rows of ROW_BYTES bytes (a multiple of 16): gathers quantized activations
// or floats per expert.
__global__ void __launch_bounds__(256) gather_rows_kernel(long long rows, int row_vec, const uint4* __restrict__ src,
                                                          const unsigned* __restrict__ map, uint4* __restrict__ dst) {
  pdl_launch_dependents();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= rows * row_vec) return;
  const long long r = gid / row_vec;
  const int j = (int)(gid - r * row_vec);
  dst[gid] = src[(long long)map[r] * row_vec + j];
}

// d4_swiglu_w, the Q8_K quantizer and the conversion to the tensor cores' operands in one pass: a warp a
// 256-wide block of a row's middle values, lane l its elements 8l .. 8l+7.  Every step is the arithmetic of
// swiglu_w_kernel, quant_q8_k_kernel and act_f16_kernel in turn, so the results are theirs bit for bit; the
// middle values and their int8 form never go to memory.
__global__ void __launch_bounds__(256) swiglu_q8k_f16_kernel(long long nblocks, int ff, float clamp,
                                                             const float* __restrict__ g, const float* __restrict__ u,
                                                             const float* __restrict__ w, __half* __restrict__ mh,
                                                             __half* __restrict__ me, float* __restrict__ ms,
                                                             const unsigned* __restrict__ rows_dev) {
  pdl_launch_dependents();
  pdl_wait();
  const long long b = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  if (rows_dev && b >= (long long)*rows_dev * (ff / 256)) return;  // the rows in use, known on the device only
  const float wv = w ? w[b / (ff / 256)] : 1.0f;
  const float4 g0 = ((const float4*)(g + b * 256))[2 * lane], g1 = ((const float4*)(g + b * 256))[2 * lane + 1];
  const float4 u0 = ((const float4*)(u + b * 256))[2 * lane], u1 = ((const float4*)(u + b * 256))[2 * lane + 1];
  const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  const float us[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float gv = gs[j], uv = us[j];
    if (clamp > 1e-6f) { gv = fminf(gv, clamp); uv = fmaxf(-clamp, fminf(uv, clamp)); }
    v[j] = __fmul_rn(__fmul_rn(__fmul_rn(gv, d4_sigmoid(gv)), uv), wv);
  }
  // QUANTIZE-Q8K! (src/kquant.lisp:130-167), the quantizer kernels' own routine
  int q[8];
  float d;
  q8k_values(v, lane, q, d);
  uint32_t h[4];
  int s = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    s += q[2 * j] + q[2 * j + 1];
    const __half2 hh = __floats2half2_rn((float)q[2 * j], (float)q[2 * j + 1]);
    h[j] = *(const uint32_t*)&hh;
  }
  ((uint4*)(mh + b * 256))[lane] = make_uint4(h[0], h[1], h[2], h[3]);
  if (lane == 0) ms[b] = d;
  if (me) {
    // the block's sixteen sums of 16 as halves, then 48 zeros (the rest of the 64-wide K step of the mins' product)
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    __half* e = me + b * 64;
    if (!(lane & 1)) e[lane >> 1] = __float2half_rn((float)s);
    if (lane < 24) ((uint32_t*)(e + 16))[lane] = 0u;
  }
}

// the same for rows that are a whole number of 4-byte words only
__global__ void __launch_bounds__(256) gather_rows4_kernel(long long rows, int row_words, const uint32_t* __restrict__ src,
                                                           const unsigned* __restrict__ map, uint32_t* __restrict__ dst) {
  pdl_launch_dependents();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= rows * row_words) return;
  const long long r = gid / row_words;
  const int j = (int)(gid - r * row_words);
  dst[gid] = src[(long long)map[r] * row_words + j];
}

// ROW_PTRS[place] = PTRS[e] for every place of expert e (block e), so that the one-token kernels, which take an
// expert per row, run an expert's rows one after the other; block NE gives the places past the last expert's
// (rows the grouping left out) expert 0's matrix: their products are computed and never read.
__global__ void __launch_bounds__(128) row_ptrs_kernel(int ne, const unsigned long long* __restrict__ ptrs,
                                                       const unsigned* __restrict__ counts, const unsigned* __restrict__ bases,
                                                       long long total_rows, unsigned long long* __restrict__ row_ptrs) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x;
  if (e < ne) {
    const unsigned long long pe = ptrs[e];
    const long long b = bases[e], c = counts[e];
    for (long long i = threadIdx.x; i < c; i += blockDim.x)
      if (b + i < total_rows) row_ptrs[b + i] = pe;
  } else {
    const unsigned long long p0 = ptrs[0];
    for (long long i = (long long)bases[ne - 1] + counts[ne - 1] + threadIdx.x; i < total_rows; i += blockDim.x) row_ptrs[i] = p0;
  }
}

// One block a segment (rows of one expert from one source): arrival index <-> place of each row.
__global__ void __launch_bounds__(128) ep_plan_rows_kernel(const int* __restrict__ seg_arrival, const int* __restrict__ seg_place,
                                                           const int* __restrict__ seg_len, unsigned* __restrict__ p2r,
                                                           unsigned* __restrict__ r2p) {
  pdl_launch_dependents();
  pdl_wait();
  const int a = seg_arrival[blockIdx.x], pl = seg_place[blockIdx.x], n = seg_len[blockIdx.x];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    p2r[pl + i] = (unsigned)(a + i);
    r2p[a + i] = (unsigned)(pl + i);
  }
}

}  // namespace ill

using namespace ill;

static int check_ptr(ill_dptr p, unsigned align) { return p && !(p & (align - 1)); }

extern "C" int ill_moe_mv(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, int nz, ill_dptr xq, ill_dptr xs,
                          ill_dptr xsum, int x_per_expert, ill_dptr y, int64_t y_stride, ill_stream stream) {
  if (!ptrs || nz < 1 || (ptrs & 7) || (x_per_expert != 0 && x_per_expert != 1)) return ILL_ERR_ARG;
  const uint64_t ws[1] = {0}, ys[1] = {y};
  const int rs[1] = {nrows};
  return mv_common(fmt, MODE_PLAIN, 1, ws, rs, ncols, xq, xs, xsum, ys, nullptr, 0, 1, ptrs, nz, add, 0, x_per_expert,
                   y_stride, 0, 0.0f, stream);
}

extern "C" int ill_moe_glu(int fmt, int ncols, int nrows, int64_t gate_add, int64_t up_add, ill_dptr ptrs, int nz,
                           ill_dptr xq, ill_dptr xs, ill_dptr xsum, int x_per_expert, float clamp, ill_dptr weights,
                           ill_dptr mid, int64_t mid_stride, ill_stream stream) {
  if (!ptrs || nz < 1 || (ptrs & 7) || !weights || (weights & 3) || (x_per_expert != 0 && x_per_expert != 1))
    return ILL_ERR_ARG;
  const uint64_t ws[2] = {0, 0}, ys[2] = {mid, mid};
  const int rs[2] = {nrows, nrows};
  return mv_common(fmt, MODE_MOE_GLU, 2, ws, rs, ncols, xq, xs, xsum, ys, nullptr, 0, 1, ptrs, nz, gate_add,
                   up_add - gate_add, x_per_expert, mid_stride, weights, clamp, stream);
}

extern "C" int ill_swiglu_w(int64_t n, int ff, float clamp, ill_dptr g, ill_dptr u, ill_dptr w, ill_dptr mid,
                            ill_stream stream) {
  if (n < 0 || ff <= 0 || !check_ptr(g, 4) || !check_ptr(u, 4) || !check_ptr(mid, 4) || (w & 3)) return ILL_ERR_ARG;
  if (n == 0) return ILL_OK;
  long long nn = n;
  const float *gp = (const float*)(uintptr_t)g, *up = (const float*)(uintptr_t)u, *wp = (const float*)(uintptr_t)w;
  float* mp = (float*)(uintptr_t)mid;
  void* args[] = {&nn, &ff, &clamp, &gp, &up, &wp, &mp};
  return launch_kernel((const void*)swiglu_w_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

static int moe_sum_launch(int d, int nu, int64_t ntok, ill_dptr down, ill_dptr map, ill_dptr map2, ill_dptr shared_, ill_dptr moe,
                          ill_dptr flag_peers, ill_dptr flags, int world, int rank, uint32_t epoch, int64_t wait_ns,
                          ill_dptr ovf_epoch, ill_dptr ovf_flag, ill_stream stream) {
  if (d <= 0 || nu <= 0 || ntok < 0 || (ovf_epoch & 3) || (ovf_flag & 3) || (ovf_flag && !ovf_epoch) || !check_ptr(down, 4) || !check_ptr(moe, 4) || (map & 3) || (map2 & 3) || (shared_ & 3))
    return ILL_ERR_ARG;
  if (ntok == 0 && !flag_peers) return ILL_OK;
  long long nt = ntok;
  const float *dp = (const float*)(uintptr_t)down, *sp = (const float*)(uintptr_t)shared_;
  const unsigned *mp = (const unsigned*)(uintptr_t)map, *m2 = (const unsigned*)(uintptr_t)map2;
  float* op = (float*)(uintptr_t)moe;
  const unsigned long long* fp = (const unsigned long long*)(uintptr_t)flag_peers;
  unsigned* fl = (unsigned*)(uintptr_t)flags;
  unsigned long long wn = (unsigned long long)wait_ns;
  unsigned* stw = device_status_word();
  const unsigned* oe = (const unsigned*)(uintptr_t)ovf_epoch;
  unsigned* of = (unsigned*)(uintptr_t)ovf_flag;
  int vec = d % 4 == 0 && !(down & 15) && !(moe & 15) && !(shared_ & 15);
  void* args[] = {&d, &nu, &nt, &dp, &mp, &m2, &sp, &op, &fp, &fl, &world, &rank, &epoch, &wn, &stw, &oe, &of, &vec};
  long long blocks = (ntok * (vec ? d / 4 : d) + 255) / 256;
  if (blocks > 16 * 148) blocks = 16 * 148;  // the blocks stride over the rest
  if (blocks < 1) blocks = 1;  // a rank without tokens still meets the others
  return launch_kernel((const void*)moe_sum_kernel, dim3((unsigned)blocks), dim3(256), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_moe_sum(int d, int nu, int64_t ntok, ill_dptr down, ill_dptr map, ill_dptr shared_, ill_dptr moe,
                           ill_stream stream) {
  return moe_sum_launch(d, nu, ntok, down, map, 0, shared_, moe, 0, 0, 1, 0, 0, 0, 0, 0, stream);
}

extern "C" int ill_moe_sum_sync(int d, int nu, int64_t ntok, ill_dptr down, ill_dptr map, ill_dptr map2, ill_dptr shared_,
                                ill_dptr moe, ill_dptr flag_peers, ill_dptr flags, int world, int rank, uint32_t epoch,
                                int64_t wait_ns, ill_dptr ovf_epoch, ill_dptr ovf_flag, ill_stream stream) {
  if (!flag_peers || !flags || (flag_peers & 7) || (flags & 3) || world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world ||
      wait_ns < 0)
    return ILL_ERR_ARG;
  return moe_sum_launch(d, nu, ntok, down, map, map2, shared_, moe, flag_peers, flags, world, rank, epoch, wait_ns, ovf_epoch, ovf_flag,
                        stream);
}

// The ranks meet (slot SLOT of the flags), nothing else: one block.
__global__ void __launch_bounds__(64) ep_barrier_kernel(const unsigned long long* flag_peers, unsigned* flags, int world, int rank,
                                                        int slot, unsigned epoch, unsigned long long wait_ns, unsigned* status) {
  pdl_launch_dependents();
  pdl_wait();
  ep_meet(flag_peers, flags, world, rank, slot, epoch, true, wait_ns, status);
}

// ---- an all-gather by peer stores --------------------------------------------------------------
// Every CTA stores its share of SRC into every peer's buffer, fences, and takes a ticket; the CTA that takes the
// last one holds the meeting: its signal says that all of this rank's stores are out, and once every peer's
// signal is in, their blocks are complete in this rank's buffer.
__device__ unsigned g_put_ticket;  // CTAs of the running peer_put_kernel that have stored their share (one call at a time a device)

__global__ void __launch_bounds__(256) peer_put_kernel(const u8* __restrict__ src, long long nbytes, const unsigned long long* dst_peers,
                                                       long long dst_off, const unsigned long long* flag_peers, unsigned* flags,
                                                       int world, int rank, int slot, unsigned epoch, unsigned long long wait_ns,
                                                       int vec, unsigned* status) {
  pdl_launch_dependents();
  pdl_wait();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
  if (vec) {
    const long long nv = nbytes / 16;
    for (long long i = tid; i < nv; i += nthr) {
      const uint4 v = ((const uint4*)src)[i];
      for (int p = 0; p < world; ++p) {
        u8* dst = (u8*)(uintptr_t)dst_peers[p] + dst_off;
        if (dst != src) ((uint4*)dst)[i] = v;
      }
    }
    for (long long i = nv * 4 + tid; i < nbytes / 4; i += nthr) {
      const uint32_t v = ((const uint32_t*)src)[i];
      for (int p = 0; p < world; ++p) {
        u8* dst = (u8*)(uintptr_t)dst_peers[p] + dst_off;
        if (dst != src) ((uint32_t*)dst)[i] = v;
      }
    }
  } else {
    for (long long i = tid; i < nbytes / 4; i += nthr) {
      const uint32_t v = ((const uint32_t*)src)[i];
      for (int p = 0; p < world; ++p) {
        u8* dst = (u8*)(uintptr_t)dst_peers[p] + dst_off;
        if (dst != src) ((uint32_t*)dst)[i] = v;
      }
    }
  }
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = take_ticket(&g_put_ticket) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  if (threadIdx.x == 0) g_put_ticket = 0;
  ep_meet(flag_peers, flags, world, rank, slot, epoch, true, wait_ns, status);
}

extern "C" int ill_peer_put(ill_dptr src, int64_t nbytes, ill_dptr dst_peers, int64_t dst_off, ill_dptr flag_peers, ill_dptr flags,
                            int world, int rank, int slot, uint32_t epoch, int64_t wait_ns, ill_stream stream) {
  if (!src || nbytes <= 0 || !dst_peers || dst_off < 0 || !flag_peers || !flags || world < 1 || world > EP_MAX_RANKS || rank < 0 ||
      rank >= world || slot < 0 || slot >= EP_FLAG_SLOTS || wait_ns < 0)
    return ILL_ERR_ARG;
  if ((src & 3) || (nbytes & 3) || (dst_off & 3) || (dst_peers & 7) || (flag_peers & 7) || (flags & 3)) return ILL_ERR_ALIGN;
  const u8* sp = (const u8*)(uintptr_t)src;
  long long nb = nbytes, off = dst_off;
  const unsigned long long* dp = (const unsigned long long*)(uintptr_t)dst_peers;
  const unsigned long long* fp = (const unsigned long long*)(uintptr_t)flag_peers;
  unsigned* fl = (unsigned*)(uintptr_t)flags;
  unsigned long long wn = (unsigned long long)wait_ns;
  int vec = !(src & 15) && !(dst_off & 15);  // the peers' buffers are assumed 16-byte aligned when the offset is
  unsigned* stw = device_status_word();
  int grid = (int)((nbytes / 16 + 255) / 256);
  grid = grid < 1 ? 1 : grid > 512 ? 512 : grid;  // grid-stride loops: a few CTAs an SM are enough to fill the links
  void* args[] = {&sp, &nb, &dp, &off, &fp, &fl, &world, &rank, &slot, &epoch, &wn, &vec, &stw};
  return launch_kernel((const void*)peer_put_kernel, dim3(grid), dim3(256), 0, args, (cudaStream_t)stream);
}

extern "C" int64_t ill_ep_flags_bytes(void) { return (int64_t)EP_MAX_RANKS * EP_FLAG_SLOTS * 4; }

extern "C" int ill_ep_barrier(ill_dptr flag_peers, ill_dptr flags, int world, int rank, int slot, uint32_t epoch, int64_t wait_ns,
                              ill_stream stream) {
  if (!flag_peers || !flags || (flag_peers & 7) || (flags & 3) || world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world ||
      slot < 0 || slot >= EP_FLAG_SLOTS || wait_ns < 0)
    return ILL_ERR_ARG;
  const unsigned long long* fp = (const unsigned long long*)(uintptr_t)flag_peers;
  unsigned* fl = (unsigned*)(uintptr_t)flags;
  unsigned long long wn = (unsigned long long)wait_ns;
  unsigned* stw = device_status_word();
  void* args[] = {&fp, &fl, &world, &rank, &slot, &epoch, &wn, &stw};
  return launch_kernel((const void*)ep_barrier_kernel, dim3(1), dim3(64), 0, args, (cudaStream_t)stream);
}

// ---- peer mappings for hosts that drive the ranks as processes ----------------------------------
typedef CUresult (*AddrRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

extern "C" int ill_ep_ipc_export(ill_dptr buf, unsigned char* handle, int64_t* offset) {
  if (!buf || !handle || !offset) return ILL_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == ILL_EP_IPC_HANDLE_BYTES, "the handle is 64 bytes");
  static AddrRangeFn range = nullptr;
  if (!range) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return cuda_fail(cudaErrorNotSupported);
    range = (AddrRangeFn)p;
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, (CUdeviceptr)buf) != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base);
  if (e != cudaSuccess) return cuda_fail(e);
  memcpy(handle, &h, sizeof h);
  *offset = (int64_t)(buf - (ill_dptr)base);
  return ILL_OK;
}

extern "C" int ill_ep_ipc_open(const unsigned char* handle, int64_t offset, ill_dptr* out) {
  if (!handle || !out || offset < 0) return ILL_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e);
  *out = (ill_dptr)(uintptr_t)p + (ill_dptr)offset;
  return ILL_OK;
}

extern "C" int ill_ep_ipc_close(ill_dptr mapped, int64_t offset) {
  if (!mapped || offset < 0) return ILL_ERR_ARG;
  const cudaError_t e = cudaIpcCloseMemHandle((void*)(uintptr_t)(mapped - (ill_dptr)offset));
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}

extern "C" int ill_moe_route(int ne, int nu, int mode, float scale, int64_t ntok, ill_dptr logits, ill_dptr bias,
                             ill_dptr sel, ill_dptr weights, ill_stream stream) {
  if (ne <= 0 || ne > 32 * ROUTE_MAX_PER_LANE || nu <= 0 || nu > 32 || nu > ne || (mode != 0 && mode != 2) || ntok < 0)
    return ILL_ERR_ARG;
  if (!check_ptr(logits, 4) || !check_ptr(sel, 4) || !check_ptr(weights, 4) || (bias & 3)) return ILL_ERR_ARG;
  if (ntok == 0) return ILL_OK;
  long long nt = ntok;
  const float *lp = (const float*)(uintptr_t)logits, *bp = (const float*)(uintptr_t)bias;
  unsigned* sp = (unsigned*)(uintptr_t)sel;
  float* wp = (float*)(uintptr_t)weights;
  void* args[] = {&ne, &nu, &mode, &scale, &nt, &lp, &bp, &sp, &wp};
  return launch_kernel((const void*)route_kernel, dim3((unsigned)((ntok + 3) / 4)), dim3(128), 0, args,
                       (cudaStream_t)stream);
}

extern "C" int64_t ill_moe_group_scratch_bytes(int64_t rows, int ne) {
  if (rows < 0 || ne <= 0) return 0;
  const int64_t nblocks = (rows + GROUP_BLOCK - 1) / GROUP_BLOCK;
  return 4 * (rows + nblocks * ne);  // rank per row, counts per (block, expert)
}

extern "C" int ill_moe_group(int64_t rows, int ne, int nu, ill_dptr sel, ill_dptr w, ill_dptr scratch, ill_dptr counts,
                             ill_dptr bases, ill_dptr rmap, ill_dptr smap, ill_dptr wrow, ill_stream stream) {
  if (rows < 0 || ne <= 0 || ne > 512 || nu <= 0) return ILL_ERR_ARG;
  if (!check_ptr(sel, 4) || !check_ptr(scratch, 4) || !check_ptr(counts, 4) || !check_ptr(bases, 4) ||
      !check_ptr(rmap, 4) || !check_ptr(smap, 4) || (wrow & 3) || (wrow && !check_ptr(w, 4)))
    return ILL_ERR_ARG;
  long long nrows = rows;
  int nblocks = (int)((rows + GROUP_BLOCK - 1) / GROUP_BLOCK);
  if (nblocks < 1) nblocks = 1;
  unsigned* rank = (unsigned*)(uintptr_t)scratch;
  unsigned* block_counts = rank + rows;
  const unsigned* selp = (const unsigned*)(uintptr_t)sel;
  unsigned *cp = (unsigned*)(uintptr_t)counts, *bp = (unsigned*)(uintptr_t)bases, *rp = (unsigned*)(uintptr_t)rmap,
           *sp = (unsigned*)(uintptr_t)smap;
  const float* wp = (const float*)(uintptr_t)w;
  float* wr = (float*)(uintptr_t)wrow;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)32 * ne * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(group_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  {
    unsigned* stw = device_status_word();
    void* args[] = {&nrows, &ne, &selp, &block_counts, &rank, &stw};
    int rc = launch_kernel((const void*)group_count_kernel, dim3(nblocks), dim3(GROUP_BLOCK), smem, args, st);
    if (rc) return rc;
  }
  {
    void* args[] = {&nblocks, &ne, &block_counts, &cp, &bp};
    int rc = launch_kernel((const void*)group_scan_kernel, dim3(1), dim3(512), 0, args, st);
    if (rc) return rc;
  }
  if (rows == 0) return ILL_OK;
  const unsigned* rk = rank;
  const unsigned* bc = block_counts;
  const unsigned* bs = bp;
  void* args[] = {&nrows, &ne, &nu, &selp, &rk, &bc, &bs, &wp, &rp, &sp, &wr};
  return launch_kernel((const void*)group_scatter_kernel, dim3((unsigned)((rows + 255) / 256)), dim3(256), 0, args, st);
}

// ---- grouping without any allocation ------------------------------------------------------
// Scratch for ill_moe_group_static: a fixed array in the library's own device image, so a
// caller that may not allocate needs to provide none.  Sized for ILL_GROUP_STATIC_MAX_ROWS
// (token, slot) rows and ILL_GROUP_STATIC_MAX_EXPERTS experts: 4 bytes a row for the ranks plus
// 4 bytes per (block of 1024 rows, expert) for the counts -- 384 KB, held by every GPU that
// loads the library until the process exits.
constexpr long long GROUP_STATIC_WORDS =
    ILL_GROUP_STATIC_MAX_ROWS + (ILL_GROUP_STATIC_MAX_ROWS / GROUP_BLOCK) * ILL_GROUP_STATIC_MAX_EXPERTS;
static __device__ __align__(256) unsigned g_group_scratch[GROUP_STATIC_WORDS];

// The array's device address, looked up once per device (the name above is only a host-side
// handle for the symbol; kernels must be given the address cudaGetSymbolAddress returns).
static unsigned* group_scratch_address(int* rc) {
  constexpr int MAX_DEV = 64;
  static unsigned* addr[MAX_DEV] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEV) { *rc = cuda_fail(e == cudaSuccess ? cudaErrorInvalidDevice : e); return nullptr; }
  unsigned* p = __atomic_load_n(&addr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    e = cudaGetSymbolAddress((void**)&p, g_group_scratch);  // with DEV current: that device's copy
    if (e != cudaSuccess || !p) { *rc = cuda_fail(e == cudaSuccess ? cudaErrorInvalidSymbol : e); return nullptr; }
    __atomic_store_n(&addr[dev], p, __ATOMIC_RELEASE);
  }
  *rc = ILL_OK;
  return p;
}

extern "C" int ill_moe_group_static(int64_t rows, int ne, int nu, ill_dptr sel, ill_dptr w, ill_dptr counts, ill_dptr bases,
                                    ill_dptr rmap, ill_dptr smap, ill_dptr wrow, ill_stream stream) {
  if (rows < 0 || ne <= 0 || nu <= 0) return ILL_ERR_ARG;
  if (rows > ILL_GROUP_STATIC_MAX_ROWS || ne > ILL_GROUP_STATIC_MAX_EXPERTS) return ILL_ERR_TOO_LARGE;
  if (!check_ptr(sel, 4) || !check_ptr(counts, 4) || !check_ptr(bases, 4) || !check_ptr(rmap, 4) || !check_ptr(smap, 4) ||
      (wrow & 3) || (wrow && !check_ptr(w, 4)))
    return ILL_ERR_ARG;
  int rc = ILL_OK;
  unsigned* scratch = group_scratch_address(&rc);
  if (!scratch) return rc;
  long long nrows = rows;
  int nblocks = (int)((rows + GROUP_BLOCK - 1) / GROUP_BLOCK);
  if (nblocks < 1) nblocks = 1;
  // every word the passes read is written first by an earlier pass of this same call (ranks
  // for all ROWS, counts for all NBLOCKS x NE), so nothing left by a previous call is seen
  unsigned* rank = scratch;
  unsigned* block_counts = scratch + ILL_GROUP_STATIC_MAX_ROWS;
  const unsigned* selp = (const unsigned*)(uintptr_t)sel;
  unsigned *cp = (unsigned*)(uintptr_t)counts, *bp = (unsigned*)(uintptr_t)bases, *rp = (unsigned*)(uintptr_t)rmap,
           *sp = (unsigned*)(uintptr_t)smap;
  const float* wp = (const float*)(uintptr_t)w;
  float* wr = (float*)(uintptr_t)wrow;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)32 * ne * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(group_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  {
    unsigned* stw = device_status_word();
    void* args[] = {&nrows, &ne, &selp, &block_counts, &rank, &stw};
    rc = launch_kernel((const void*)group_count_kernel, dim3(nblocks), dim3(GROUP_BLOCK), smem, args, st);
    if (rc) return rc;
  }
  {
    void* args[] = {&nblocks, &ne, &block_counts, &cp, &bp};
    rc = launch_kernel((const void*)group_scan_kernel, dim3(1), dim3(512), 0, args, st);
    if (rc) return rc;
  }
  if (rows == 0) return ILL_OK;
  const unsigned* rk = rank;
  const unsigned* bc = block_counts;
  const unsigned* bs = bp;
  void* args[] = {&nrows, &ne, &nu, &selp, &rk, &bc, &bs, &wp, &rp, &sp, &wr};
  return launch_kernel((const void*)group_scatter_kernel, dim3((unsigned)((rows + 255) / 256)), dim3(256), 0, args, st);
}

extern "C" int ill_swiglu_q8k_f16(int64_t rows, int ff, float clamp, ill_dptr g, ill_dptr u, ill_dptr w, ill_dptr mh,
                                  ill_dptr me, ill_dptr ms, ill_dptr rows_dev, ill_stream stream) {
  if (rows < 0 || ff <= 0 || ff % 256 || !g || !u || !mh || !ms) return ILL_ERR_ARG;
  if ((g & 15) || (u & 15) || (w & 3) || (mh & 15) || (me & 15) || (ms & 3) || (rows_dev & 3)) return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  long long nb = rows * (ff / 256);
  const float* gp = (const float*)(uintptr_t)g;
  const float* up = (const float*)(uintptr_t)u;
  const float* wp = (const float*)(uintptr_t)w;
  __half* hp = (__half*)(uintptr_t)mh;
  __half* ep = (__half*)(uintptr_t)me;
  float* sp = (float*)(uintptr_t)ms;
  const unsigned* rd = (const unsigned*)(uintptr_t)rows_dev;
  void* args[] = {&nb, &ff, &clamp, &gp, &up, &wp, &hp, &ep, &sp, &rd};
  return launch_kernel((const void*)swiglu_q8k_f16_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

extern "C" int ill_moe_row_ptrs(int ne, ill_dptr ptrs, ill_dptr counts, ill_dptr bases, int64_t total_rows, ill_dptr row_ptrs,
                                ill_stream stream) {
  if (ne < 1 || ne > 65535 || total_rows < 0 || !check_ptr(ptrs, 8) || !check_ptr(counts, 4) || !check_ptr(bases, 4) ||
      !check_ptr(row_ptrs, 8))
    return ILL_ERR_ARG;
  if (total_rows == 0) return ILL_OK;
  const unsigned long long* pp = (const unsigned long long*)(uintptr_t)ptrs;
  const unsigned* cp = (const unsigned*)(uintptr_t)counts;
  const unsigned* bp = (const unsigned*)(uintptr_t)bases;
  long long tr = total_rows;
  unsigned long long* rp = (unsigned long long*)(uintptr_t)row_ptrs;
  void* args[] = {&ne, &pp, &cp, &bp, &tr, &rp};
  return launch_kernel((const void*)row_ptrs_kernel, dim3((unsigned)ne + 1), dim3(128), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_gather_rows(int64_t rows, int64_t row_bytes, ill_dptr src, ill_dptr map, ill_dptr dst,
                               ill_stream stream) {
  if (rows < 0 || row_bytes <= 0 || (row_bytes & 3) || !check_ptr(map, 4)) return ILL_ERR_ARG;
  const unsigned align = (row_bytes & 15) ? 4 : 16;
  if (!check_ptr(src, align) || !check_ptr(dst, align)) return ILL_ERR_ARG;
  if (rows == 0) return ILL_OK;
  long long nrows = rows;
  const unsigned* mp = (const unsigned*)(uintptr_t)map;
  if (align == 4) {
    int row_words = (int)(row_bytes / 4);
    const uint32_t* sp = (const uint32_t*)(uintptr_t)src;
    uint32_t* dp = (uint32_t*)(uintptr_t)dst;
    void* args[] = {&nrows, &row_words, &sp, &mp, &dp};
    return launch_kernel((const void*)gather_rows4_kernel, dim3((unsigned)((rows * row_words + 255) / 256)), dim3(256), 0,
                         args, (cudaStream_t)stream);
  }
  int row_vec = (int)(row_bytes / 16);
  const uint4* sp = (const uint4*)(uintptr_t)src;
  uint4* dp = (uint4*)(uintptr_t)dst;
  void* args[] = {&nrows, &row_vec, &sp, &mp, &dp};
  return launch_kernel((const void*)gather_rows_kernel, dim3((unsigned)((rows * row_vec + 255) / 256)), dim3(256), 0,
                       args, (cudaStream_t)stream);
}

extern "C" int ill_ep_plan_rows(int nseg, ill_dptr seg_arrival, ill_dptr seg_place, ill_dptr seg_len, ill_dptr p2r,
                                ill_dptr r2p, ill_stream stream) {
  if (nseg < 0 || !check_ptr(seg_arrival, 4) || !check_ptr(seg_place, 4) || !check_ptr(seg_len, 4) || !check_ptr(p2r, 4) ||
      !check_ptr(r2p, 4))
    return ILL_ERR_ARG;
  if (nseg == 0) return ILL_OK;
  const int* sa = (const int*)(uintptr_t)seg_arrival;
  const int* sp = (const int*)(uintptr_t)seg_place;
  const int* sl = (const int*)(uintptr_t)seg_len;
  unsigned* pp = (unsigned*)(uintptr_t)p2r;
  unsigned* rp = (unsigned*)(uintptr_t)r2p;
  void* args[] = {&sa, &sp, &sl, &pp, &rp};
  return launch_kernel((const void*)ep_plan_rows_kernel, dim3((unsigned)nseg), dim3(128), 0, args, (cudaStream_t)stream);
}
