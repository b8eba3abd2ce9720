// decode.cu -- a decoded token's whole chain of quantized products in ONE launch.
//
// The reference issues a kernel per product (CUDA-FORWARD-N, src/cuda-dense.lisp:380-432: about
// 1,700 launches a token, TODO.md:16-21); at one token every product moves 1-30 MB, i.e. 0.3-5 us of
// HBM time, and a dependent launch costs about as much again.  Here a persistent grid (one CTA per
// SM, launched cooperatively so that all of them are resident) walks a list of products:
//
//   * The weights never depend on earlier products, so every warp streams the tiles it will
//     multiply -- of this product and of the ones after it -- through its own ring in shared memory
//     with bulk asynchronous copies, as far ahead as the ring has room.  HBM keeps streaming across
//     the boundaries between products.
//   * Where a product reads what an earlier one wrote (AFTER), the CTAs meet at a barrier in global
//     memory (one arrival a CTA, a generation counter; the wait is bounded and ends in a status code).
//   * The activation quantizer -- and the RMSNorm before it -- runs in the consumer's prologue: every
//     CTA quantizes the vector it is about to multiply (at most 40 KB, from L2) into its own shared
//     memory, bit for bit as ill_quant_q8_0 / ill_quant_q8_k / ill_rmsnorm_q8 do.  No quantize launches.
//   * A row's arithmetic is the one-token product's (mv.cu): the same lanes a row, units a lane and
//     order of additions, so the results are the same bits as ill_mv / ill_mv_glu give.
//
// The ring is allocated by bytes, not by slots: a tile takes the 16-byte aligned span of its rows (a
// gated product's tile is its gate rows and its up rows), so the bytes in flight stay near the ring's
// size whatever the tile size, and up to DEC_NBAR tiles (an mbarrier each) are outstanding per warp.
#include "formats.cuh"
#include "iq2xxs_tables.cuh"
#include "quantdev.cuh"
#include "host.h"

#include <vector>

namespace ill {

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_NBAR = 8;          // tiles in flight per warp, at most
constexpr int DEC_MAX_OPS = 1024;
constexpr int DEC_MAX_COLS = 32768;  // activations staged in shared memory: 1.25 bytes a column

// One product as the kernel reads it (global memory, 128 bytes).
struct __align__(16) DecOp {
  const u8* w;
  const u8* w2;            // the "up" matrix of a gated product, else null
  float* y;
  const float* bias;
  const float* x;          // the activations as floats
  const float* norm_w;     // RMSNorm weights, or null
  float eps;
  int fmt, acc, f16_scale;
  int rows, cols, row_bytes, units;
  int lanes, upt, tr;      // lanes a row, units a lane, rows a tile
  int tile0, ntiles;       // the product's tiles among all the list's tiles
  int after, restage;      // meet the other CTAs first; quantize X into shared memory first
  int pad[4];
};
static_assert(sizeof(DecOp) == 128, "DecOp is 128 bytes");

// What the issuing lane needs of a product, in shared memory.
struct DecSrc {
  const u8* w;
  const u8* w2;
  int tile0, ntiles, rows, tr, row_bytes, pad;
};

struct DecParams {
  const DecOp* ops;
  int nops;
  unsigned* bar;           // [0] arrivals, [1] generation
  int total_tiles;
  int ring_bytes;          // per warp
  int max_cols;            // the staged activations' capacity
  int has_iq;
  unsigned* status;
};

// What every warp of the CTA shares, written once at the start (shared memory).
struct DecShared {
  const DecSrc* srcs;      // [nops] in shared memory
  unsigned* status;
  int total_tiles, ring_bytes, gstep, pad;
  const i8* xq;            // the staged activations
  const float* xs;
  const int16_t* bs;
  const uint2* iq_grid;
  const uint2* iq_smask;
};

// A warp's state (shared memory): the product it is on, and its ring of tiles.  C counts the tiles consumed; the
// fields after it belong to the issuing lane.  The ring's bytes lie elsewhere (RING of the functions below).
struct __align__(16) DecWarp {
  DecOp op;
  uint64_t bars[DEC_NBAR];
  int offs[DEC_NBAR];      // where tile i % DEC_NBAR starts in the ring
  int c;
  int issued, head;
  int iss_t, iss_op;
  int pad[3];
};

// bytes of the 16-byte aligned span that covers [SRC, SRC + LEN)
__device__ __forceinline__ uint32_t span16(const u8* src, uint32_t len) {
  const uintptr_t a0 = (uintptr_t)src & ~(uintptr_t)15;
  return (uint32_t)((((uintptr_t)src + len + 15) & ~(uintptr_t)15) - a0);
}

// Lane 0: issue this warp's next tiles while a barrier and contiguous room in the ring are free.
__device__ __forceinline__ void dec_issue(DecWarp* cw, u8* ring, const DecShared* sh) {
  const DecSrc* srcs = sh->srcs;
  const int total_tiles = sh->total_tiles, gstep = sh->gstep, ring_bytes = sh->ring_bytes;
  int issued = cw->issued, head = cw->head, iss_t = cw->iss_t, iss_op = cw->iss_op;
  const int c = cw->c;
  while (iss_t < total_tiles && issued - c < DEC_NBAR) {
    while (iss_t >= srcs[iss_op].tile0 + srcs[iss_op].ntiles) ++iss_op;
    const DecSrc o = srcs[iss_op];
    const long long row0 = (long long)(iss_t - o.tile0) * o.tr;
    const int nrows = min(o.tr, o.rows - (int)row0);
    const uint32_t len = (uint32_t)nrows * (uint32_t)o.row_bytes;
    const u8* s0 = o.w + row0 * o.row_bytes;
    const uint32_t b0 = span16(s0, len);
    const u8* s1 = o.w2 ? o.w2 + row0 * o.row_bytes : nullptr;
    const uint32_t b1 = s1 ? span16(s1, len) : 0u;
    const int need = (int)(b0 + b1);
    int off;
    if (issued == c) off = 0;  // nothing outstanding: start over at the ring's base
    else {
      const int tail = cw->offs[c % DEC_NBAR];  // the oldest tile not yet consumed
      if (head > tail) {
        if (head + need <= ring_bytes) off = head;
        else if (need <= tail) off = 0;
        else break;
      } else {
        if (head + need <= tail) off = head;
        else break;
      }
    }
    const int b = issued % DEC_NBAR;
    cw->offs[b] = off;
    mbar_expect_tx(&cw->bars[b], (uint32_t)need);
    bulk_g2s(ring + off, (const void*)((uintptr_t)s0 & ~(uintptr_t)15), b0, &cw->bars[b]);
    if (s1) bulk_g2s(ring + off + b0, (const void*)((uintptr_t)s1 & ~(uintptr_t)15), b1, &cw->bars[b]);
    ++issued;
    head = off + need;
    iss_t += gstep;
  }
  cw->issued = issued; cw->head = head; cw->iss_t = iss_t; cw->iss_op = iss_op;
}

// The CTAs meet (thread 0 of each, between two __syncthreads).  False after a bounded wait.
__device__ __forceinline__ bool dec_grid_barrier(unsigned* bar, unsigned nctas, unsigned* status) {
  volatile unsigned* gen = bar + 1;
  const unsigned g = *gen;  // read before arriving: the generation cannot move until this CTA has arrived
  __threadfence();
  const unsigned old = atomicAdd(bar, 1u);
  if (old == nctas - 1) {
    atomicExch(bar, 0u);
    __threadfence();
    atomicAdd(bar + 1, 1u);
  } else {
    unsigned long long t0 = 0;
    for (unsigned it = 1; *gen == g; ++it) {
      if ((it & 1023u) == 0) {
        const unsigned long long now = global_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > ILL_WAIT_NS) {
          if (status) atomicCAS(status, 0u, (unsigned)ST_BARRIER_WAIT);
          return false;
        }
      }
    }
  }
  __threadfence();
  return true;
}

// Every CTA quantizes the product's activations into its own shared memory (all threads; ends with a
// __syncthreads).  The arithmetic and its order are rmsnorm_q8_kernel's and the quantizer kernels' (quant.cu).
// X is read around L1 (ld.cg): an earlier product of this same launch may have written it.
__device__ __forceinline__ void dec_stage_x(const DecOp& op, i8* xq, float* xs, int16_t* bs, double* part, float* scale_s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = op.x;
  float sc = 1.0f;
  if (op.norm_w) {
    double acc = 0.0;
    if (tid < 256)
      for (int i = tid; i < op.cols; i += 256) {
        const float v = __ldcg(x + i);
        acc += (double)__fmul_rn(v, v);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0 && warp < 8) part[warp] = acc;
    __syncthreads();
    if (tid == 0) {
      double t = 0.0;
      for (int i = 0; i < 8; ++i) t += part[i];
      *scale_s = __fdiv_rn(1.0f, __fsqrt_rn((float)(t / (double)op.cols + (double)op.eps)));
    }
    __syncthreads();
    sc = *scale_s;
  }
  if (op.fmt != ILL_Q8_0) {
    for (int b = warp; b < op.cols / 256; b += DEC_WARPS) {
      const float4 v0 = __ldcg((const float4*)(x + b * 256) + 2 * lane), v1 = __ldcg((const float4*)(x + b * 256) + 2 * lane + 1);
      float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      if (op.norm_w) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], sc), op.norm_w[b * 256 + 8 * lane + j]);
      }
      quant_block_q8_k(v, lane, b, xq, xs, bs);
    }
  } else {
    for (int b = warp; b < op.cols / 32; b += DEC_WARPS) {
      float v = __ldcg(x + b * 32 + lane);
      if (op.norm_w) v = __fmul_rn(__fmul_rn(v, sc), op.norm_w[b * 32 + lane]);
      quant_block_q8_0(v, lane, b, xq, xs, nullptr, op.f16_scale);
    }
  }
  __syncthreads();
}

// This warp's tiles T_FIRST, T_FIRST + GSTEP, ... of the product in CW->OP.  False when a copy never landed.
// A function of its own per variant (not inlined): each gets the registers it needs, not the sum of them all.
template <int FMT, bool GLU, int UPT, int AL>
__device__ __noinline__ bool dec_run(DecWarp* cw, u8* ring, const DecShared* sh, int t_first) {
  const int lane = threadIdx.x & 31;
  const int L = cw->op.lanes, units = cw->op.units, tr = cw->op.tr, rows = cw->op.rows, row_bytes = cw->op.row_bytes;
  const int tile0 = cw->op.tile0, tend = tile0 + cw->op.ntiles, gstep = sh->gstep, acc = cw->op.acc;
  const u8* const wg = cw->op.w;
  const u8* const wu = cw->op.w2;
  float* const y = cw->op.y;
  const float* const bias = cw->op.bias;
  const int sub = lane / L, sl = lane - sub * L, nsub = 32 / L;
  IqTables iqt;
  iqt.grid = sh->iq_grid + (threadIdx.x & (IQ_COPIES - 1));
  iqt.smask = sh->iq_smask + (threadIdx.x & (IQ_COPIES - 1));
  XReg<FMT> x[UPT];
  UPos<FMT> up[UPT];
  {
    ActS xa;
    xa.q = sh->xq; xa.s = sh->xs; xa.bs = sh->bs;
#pragma unroll
    for (int k = 0; k < UPT; ++k) {
      const int u = sl + k * L;
      unit_pos(up[k], u);
      if (u < units) load_x(x[k], xa, u);
    }
  }
  int c = cw->c;
  bool all_ok = true;
  for (int t = t_first; t < tend; t += gstep) {
    const int b = c % DEC_NBAR;
    bool ok = mbar_wait(&cw->bars[b], (uint32_t)(c / DEC_NBAR) & 1u, sh->status, ST_MV_WAIT + 0x10 + FMT);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) { all_ok = false; break; }
    const int off = cw->offs[b];  // written by lane 0 before it issued the copy this wait has just seen land
    const long long row0 = (long long)(t - tile0) * tr;
    const int nrows = min(tr, rows - (int)row0);
    const u8* s0 = wg + row0 * row_bytes;
    const u8* rows_g = ring + off + ((uintptr_t)s0 & 15);
    const u8* rows_u = nullptr;
    if constexpr (GLU) {
      const u8* s1 = wu + row0 * row_bytes;
      rows_u = ring + off + span16(s0, (uint32_t)nrows * (uint32_t)row_bytes) + ((uintptr_t)s1 & 15);
    }
#pragma unroll 1
    for (int r0 = 0; r0 < nrows; r0 += nsub) {
      const int rr = r0 + sub;
      const bool valid = rr < nrows;
      float sum = 0.0f, sum2 = 0.0f;
      if (valid) {
        const u8* rowp = rows_g + (size_t)rr * row_bytes;
#pragma unroll
        for (int k = 0; k < UPT; ++k) {
          const int u = sl + k * L;
          if (k < UPT - 1 || u < units) {
            WReg<FMT> w;
            load_w<AL>(w, rowp, up[k], iqt);
            sum = __fadd_rn(sum, dot(w, x[k]));
          }
        }
        if constexpr (GLU) {
          const u8* rowu = rows_u + (size_t)rr * row_bytes;
#pragma unroll
          for (int k = 0; k < UPT; ++k) {
            const int u = sl + k * L;
            if (k < UPT - 1 || u < units) {
              WReg<FMT> w;
              load_w<AL>(w, rowu, up[k], iqt);
              sum2 = __fadd_rn(sum2, dot(w, x[k]));
            }
          }
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if constexpr (GLU) sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
      }
      if (valid && sl == 0) {
        const long long row = row0 + rr;
        if constexpr (GLU) {
          y[row] = (sum / (1.0f + expf(-sum))) * sum2;
        } else {
          float v = sum;
          if (bias) v += bias[row];
          y[row] = acc ? __ldcg(y + row) + v : v;
        }
      }
    }
    __syncwarp();  // every lane is done with the tile
    ++c;
    if (lane == 0) {
      cw->c = c;
      dec_issue(cw, ring, sh);
    }
  }
  __syncwarp();  // lane 0's state is the warp's
  return all_ok;
}

// The variant for a product, as a pointer: the kernel then has one call site (a call site each would give every
// one of them its own save area in the kernel's stack frame).
typedef bool (*DecFn)(DecWarp*, u8*, const DecShared*, int);

template <int FMT, bool GLU, int AL>
__device__ __forceinline__ DecFn dec_pick_u(int upt) {
  switch (upt) {
    case 1: return dec_run<FMT, GLU, 1, AL>;
    case 2: return dec_run<FMT, GLU, 2, AL>;
    case 3: return dec_run<FMT, GLU, 3, AL>;
    case 4: return dec_run<FMT, GLU, 4, AL>;
    case 5: return dec_run<FMT, GLU, 5, AL>;
    case 6: if constexpr (FMT == ILL_Q8_0) return dec_run<FMT, GLU, 6, AL>; break;
    case 7: if constexpr (FMT == ILL_Q8_0) return dec_run<FMT, GLU, 7, AL>; break;
  }
  return nullptr;  // not reached: the plan only holds 1..5 (Q8_0: ..7)
}

template <int FMT, int AL>
__device__ __forceinline__ DecFn dec_pick_f(bool glu, int upt) {
  return glu ? dec_pick_u<FMT, true, AL>(upt) : dec_pick_u<FMT, false, AL>(upt);
}

__global__ void __launch_bounds__(DEC_THREADS, 1) decode_kernel(const DecParams p) {
  extern __shared__ __align__(128) u8 smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // [rings][staged activations: quants, scales, sums of 16][IQ2_XXS tables][the products' sources][warps' state][misc]
  u8* at = smem + (size_t)DEC_WARPS * p.ring_bytes;
  i8* xq_s = (i8*)at;                      at += p.max_cols;
  float* xs_s = (float*)at;                at += p.max_cols / 32 * 4;
  int16_t* bs_s = (int16_t*)at;            at += p.max_cols / 16 * 2;
  uint2* iq_grid = (uint2*)at;
  uint2* iq_smask = iq_grid + IQ_COPIES * 256;
  if (p.has_iq) at += IQ_TABLE_BYTES;
  DecSrc* srcs = (DecSrc*)at;              at += (size_t)p.nops * sizeof(DecSrc);
  DecWarp* warps = (DecWarp*)at;           at += DEC_WARPS * sizeof(DecWarp);
  DecShared* sh = (DecShared*)at;          at += sizeof(DecShared);
  double* part = (double*)at;              at += 8 * 8;
  float* scale_s = (float*)at;
  DecWarp* cw = warps + warp;
  u8* ring = smem + (size_t)warp * p.ring_bytes;

  for (int i = tid; i < p.nops; i += DEC_THREADS) {
    const DecOp* o = p.ops + i;
    DecSrc s;
    s.w = o->w; s.w2 = o->w2; s.tile0 = o->tile0; s.ntiles = o->ntiles; s.rows = o->rows; s.tr = o->tr;
    s.row_bytes = o->row_bytes; s.pad = 0;
    srcs[i] = s;
  }
  const int gw = blockIdx.x * DEC_WARPS + warp, gstep = gridDim.x * DEC_WARPS;
  if (lane == 0) {
    for (int b = 0; b < DEC_NBAR; ++b) mbar_init(&cw->bars[b], 1);
    mbar_fence_init();
    cw->c = 0; cw->issued = 0; cw->head = 0; cw->iss_t = gw; cw->iss_op = 0;
  }
  if (tid == 0) {
    sh->srcs = srcs; sh->status = p.status; sh->total_tiles = p.total_tiles; sh->ring_bytes = p.ring_bytes; sh->gstep = gstep;
    sh->xq = xq_s; sh->xs = xs_s; sh->bs = bs_s; sh->iq_grid = iq_grid; sh->iq_smask = iq_smask;
  }
  if (p.has_iq) iq_tables_fill(iq_grid, iq_smask, ill_iq2xxs_grid, ill_ksigns_iq2xs);
  __syncthreads();
  if (lane == 0) dec_issue(cw, ring, sh);  // the weights depend on nothing: start streaming
  __syncwarp();

  // LOST: this warp gave up a wait.  It keeps walking the list (the CTA's barriers count on it) but does no more
  // work; the CTA learns of it at the next point where its warps meet and leaves the list there, all warps together.
  bool lost = false, broke = false;
  for (int oi = 0; oi < p.nops; ++oi) {
    // the warp's copy of the product: a lane a word
    __syncwarp();
    ((uint32_t*)&cw->op)[lane] = ((const uint32_t*)(p.ops + oi))[lane];
    __syncwarp();
    bool synced = false;
    if (cw->op.after) {
      __syncthreads();  // this CTA's part of everything before is written
      bool bad = false;
      if (tid == 0) bad = !dec_grid_barrier(p.bar, gridDim.x, p.status);
      if (__syncthreads_or(bad || lost)) { broke = true; break; }
      synced = true;
    }
    if (cw->op.restage) {
      // every warp has taken its registers from the activations staged before
      if (!synced && __syncthreads_or(lost)) { broke = true; break; }
      dec_stage_x(cw->op, xq_s, xs_s, bs_s, part, scale_s);
    }
    const int tile0 = cw->op.tile0;
    int d = (gw - tile0) % gstep;
    if (d < 0) d += gstep;
    const int t_first = tile0 + d;
    if (!lost && t_first < tile0 + cw->op.ntiles) {
      const bool glu = cw->op.w2 != nullptr;
      const int upt = cw->op.upt;
      DecFn fn = nullptr;
      switch (cw->op.fmt) {
        case ILL_Q8_0: fn = dec_pick_f<ILL_Q8_0, 1>(glu, upt); break;
        case ILL_Q4_K: fn = dec_pick_f<ILL_Q4_K, 16>(glu, upt); break;
        case ILL_Q6_K: fn = dec_pick_f<ILL_Q6_K, 1>(glu, upt); break;
        case ILL_Q2_K: fn = dec_pick_f<ILL_Q2_K, 4>(glu, upt); break;
        case ILL_IQ2_XXS: fn = dec_pick_f<ILL_IQ2_XXS, 1>(glu, upt); break;
      }
      const bool ok = fn ? fn(cw, ring, sh, t_first) : false;
      if (!ok) lost = true;
    }
  }
  if (__syncthreads_or(lost || broke)) {
    // copies still in flight into this warp's ring get a bounded time to land before shared memory is released
    // (a lost warp's own tile has had its time already)
    for (int k = cw->c + (lost ? 1 : 0); k < cw->issued; ++k)
      mbar_wait(&cw->bars[k % DEC_NBAR], (uint32_t)(k / DEC_NBAR) & 1u, nullptr, 0);
  }
}

static uint32_t up_to(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

}  // namespace ill

using namespace ill;

// launch[]: what ill_decode_plan hands to ill_decode_run
enum { DL_NOPS = 0, DL_GRID, DL_SMEM, DL_TILES, DL_RING, DL_MAXCOLS, DL_IQ, DL_MAGIC };
constexpr int DL_MAGIC_VALUE = 0x1d1ec0de;

extern "C" int64_t ill_decode_plan_bytes(int nops) {
  if (nops < 1 || nops > DEC_MAX_OPS) return 0;
  return 128 + (int64_t)nops * (int64_t)sizeof(DecOp);
}

extern "C" int ill_decode_plan(const ill_decode_op* ops, int nops, ill_dptr plan, int64_t plan_bytes, int32_t* launch,
                               ill_stream stream) {
  if (!ops || !launch || nops < 1 || nops > DEC_MAX_OPS || !plan) return ILL_ERR_ARG;
  if (plan & 127) return ILL_ERR_ALIGN;
  if (plan_bytes < ill_decode_plan_bytes(nops)) return ILL_ERR_TOO_LARGE;
  int dev = 0, sms = 0, smem_max = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  int max_cols = 0, has_iq = 0;
  for (int i = 0; i < nops; ++i) {
    const ill_decode_op& o = ops[i];
    const int bw = fmt_block_weights(o.fmt);
    if (!bw || (o.kind != ILL_OP_MV && o.kind != ILL_OP_GLU) || o.rows <= 0 || o.cols <= 0 || o.cols % (bw == 32 ? 32 : 256) ||
        o.cols > DEC_MAX_COLS || !o.w || !o.x || !o.y || (o.kind == ILL_OP_GLU && (!o.w2 || o.acc || o.bias)) ||
        (o.kind == ILL_OP_MV && o.w2))
      return ILL_ERR_ARG;
    if ((o.w & 15) || (o.w2 & 15) || (o.x & 15) || (o.norm_w & 3) || (o.y & 3) || (o.bias & 3)) return ILL_ERR_ALIGN;
    if (o.cols > max_cols) max_cols = o.cols;
    if (o.fmt == ILL_IQ2_XXS) has_iq = 1;
  }
  max_cols = (int)up_to((uint32_t)max_cols, 256);
  // shared memory: everything but the rings first, the rings get the rest
  const uint32_t fixed = (uint32_t)max_cols + (uint32_t)max_cols / 32 * 4 + (uint32_t)max_cols / 16 * 2 + (has_iq ? IQ_TABLE_BYTES : 0) +
                         (uint32_t)nops * (uint32_t)sizeof(DecSrc) + DEC_WARPS * (uint32_t)sizeof(DecWarp) + (uint32_t)sizeof(DecShared) + 64 + 16;
  const int budget = smem_max - 1024;
  if ((int)fixed + DEC_WARPS * 8192 > budget) return ILL_ERR_TOO_LARGE;
  const int ring = (int)((((uint32_t)budget - fixed) / DEC_WARPS) & ~127u);
  std::vector<DecOp> dev_ops((size_t)nops);
  long long tiles = 0;
  const long long gwarps = (long long)sms * DEC_WARPS;
  for (int i = 0; i < nops; ++i) {
    const ill_decode_op& o = ops[i];
    DecOp& d = dev_ops[(size_t)i];
    d = DecOp();
    const int bw = fmt_block_weights(o.fmt), uw = (o.fmt == ILL_Q8_0 || o.fmt == ILL_IQ2_XXS) ? 32 : 64;
    const bool glu = o.kind == ILL_OP_GLU;
    d.w = (const u8*)(uintptr_t)o.w;
    d.w2 = (const u8*)(uintptr_t)o.w2;
    d.y = (float*)(uintptr_t)o.y;
    d.bias = (const float*)(uintptr_t)o.bias;
    d.x = (const float*)(uintptr_t)o.x;
    d.norm_w = (const float*)(uintptr_t)o.norm_w;
    d.eps = o.eps;
    d.fmt = o.fmt;
    d.acc = o.acc ? 1 : 0;
    d.f16_scale = o.f16_scale ? 1 : 0;
    d.rows = o.rows;
    d.cols = o.cols;
    d.row_bytes = o.cols / bw * fmt_block_bytes(o.fmt);
    d.units = o.cols / uw;
    const bool big = (long long)o.rows * d.row_bytes >= (16ll << 20);
    if (!mv_pick_lanes(o.fmt, d.units, glu, big, &d.lanes, &d.upt)) return ILL_ERR_UNSUPPORTED;  // rows too long for registers
    // rows a tile: a multiple of the rows a warp has in progress; about 4 KB, cut finer when the product is
    // small (every warp should get a tile), and never more than a third of the ring
    const int nsub = 32 / d.lanes, parts = glu ? 2 : 1;
    long long target = (long long)o.rows * d.row_bytes * parts / (2 * gwarps);
    if (target > 4096) target = 4096;
    if (target < 1024) target = 1024;
    if (target > ring / 3) target = ring / 3;
    long long tr = target / ((long long)d.row_bytes * parts) / nsub * nsub;
    if (tr < nsub) tr = nsub;
    if (tr > o.rows) tr = (o.rows + nsub - 1) / nsub * nsub;
    if ((tr * d.row_bytes + 32) * parts > ring / 2) return ILL_ERR_UNSUPPORTED;  // a tile must leave room for the next
    d.tr = (int)tr;
    d.ntiles = (int)((o.rows + tr - 1) / tr);
    d.tile0 = (int)tiles;
    tiles += d.ntiles;
    if (tiles > 0x7fffffffll / 2) return ILL_ERR_TOO_LARGE;
    d.after = (i > 0 && o.after) ? 1 : 0;
    const ill_decode_op* pv = i ? &ops[i - 1] : nullptr;
    const bool k8 = o.fmt != ILL_Q8_0, pk8 = pv && pv->fmt != ILL_Q8_0;
    d.restage = (!pv || d.after || pv->x != o.x || pv->norm_w != o.norm_w || pv->eps != o.eps || pv->cols != o.cols || pk8 != k8 ||
                 (!k8 && (pv->f16_scale != 0) != (o.f16_scale != 0)))
                    ? 1 : 0;
  }
  unsigned char head[128] = {0};
  cudaStream_t st = (cudaStream_t)stream;
  e = cudaMemcpyAsync((void*)(uintptr_t)plan, head, sizeof head, cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync((void*)(uintptr_t)(plan + 128), dev_ops.data(), (size_t)nops * sizeof(DecOp), cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);  // the host copy of the list is released on return
  if (e != cudaSuccess) return cuda_fail(e);
  const uint32_t smem = fixed + (uint32_t)ring * DEC_WARPS;
  e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_kernel, DEC_THREADS, smem);
  if (e != cudaSuccess) return cuda_fail(e);
  if (per_sm < 1) return ILL_ERR_UNSUPPORTED;
  launch[DL_NOPS] = nops;
  launch[DL_GRID] = sms;
  launch[DL_SMEM] = (int)smem;
  launch[DL_TILES] = (int)tiles;
  launch[DL_RING] = ring;
  launch[DL_MAXCOLS] = max_cols;
  launch[DL_IQ] = has_iq;
  launch[DL_MAGIC] = DL_MAGIC_VALUE;
  return ILL_OK;
}

extern "C" int ill_decode_run(ill_dptr plan, const int32_t* launch, ill_stream stream) {
  if (!plan || !launch || launch[DL_MAGIC] != DL_MAGIC_VALUE || launch[DL_NOPS] < 1 || launch[DL_GRID] < 1) return ILL_ERR_ARG;
  if (plan & 127) return ILL_ERR_ALIGN;
  DecParams p;
  p.ops = (const DecOp*)(uintptr_t)(plan + 128);
  p.nops = launch[DL_NOPS];
  p.bar = (unsigned*)(uintptr_t)plan;
  p.total_tiles = launch[DL_TILES];
  p.ring_bytes = launch[DL_RING];
  p.max_cols = launch[DL_MAXCOLS];
  p.has_iq = launch[DL_IQ];
  p.status = device_status_word();
  cudaError_t e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, launch[DL_SMEM]);
  if (e != cudaSuccess) return cuda_fail(e);
  // cooperative: the launch fails rather than starts if the CTAs cannot all be resident, so the barrier
  // between them cannot wait for a CTA that has not begun
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)launch[DL_GRID], 1, 1);
  cfg.blockDim = dim3(DEC_THREADS, 1, 1);
  cfg.dynamicSmemBytes = (size_t)launch[DL_SMEM];
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  void* args[] = {&p};
  e = cudaLaunchKernelExC(&cfg, (const void*)decode_kernel, args);
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}
