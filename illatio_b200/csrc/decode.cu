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
//     the boundaries between products.  A tile is a few whole rows, or, for rows too long for that,
//     one row's next run of columns (the row's sum is carried from tile to tile).
//   * Where a product reads what an earlier one wrote (AFTER), the CTAs meet at a barrier in global
//     memory (one arrival a CTA, a generation counter; the wait is bounded and ends in a status code).
//   * The activation quantizer -- and the RMSNorm before it -- runs in the consumer's prologue: every
//     CTA quantizes the vector it is about to multiply (at most 40 KB, from L2) into its own shared
//     memory, bit for bit as ill_quant_q8_0 / ill_quant_q8_k / ill_rmsnorm_q8 do.  No quantize launches.
//   * The quantized activations stay in shared memory (in planes, so that the lanes' 16-byte reads do
//     not share banks) and are read from there unit by unit: no per-product preload into registers,
//     which at one token would cost a warp as much as the one or two rows it multiplies.
//   * A row's arithmetic is the one-token product's (mv.cu): the same lanes a row, units a lane and
//     order of additions, so the results are the same bits as ill_mv / ill_mv_glu give (for rows
//     those keep in registers).
//
// The ring is allocated by bytes, not by slots: a tile takes the 16-byte aligned span of its bytes, so
// the bytes in flight stay near the ring's size whatever the tile size, and up to DEC_NBAR tiles (an
// mbarrier each) are outstanding per warp.
#include "formats.cuh"
#include "iq2xxs_tables.cuh"
#include "quantdev.cuh"
#include "host.h"

#include <vector>

namespace ill {

#ifndef DEC_WARPS
#define DEC_WARPS 11   // 352 threads: three warps a scheduler (two on one), up to 184 registers a thread
#endif
constexpr int DEC_THREADS = 32 * DEC_WARPS;
constexpr int DEC_NBAR = 8;          // tiles in flight per warp, at most
constexpr int DEC_MAX_OPS = 1024;
constexpr int DEC_MAX_COLS = 32768;  // activations staged in shared memory: 1.25 bytes a column

// One product as the kernel reads it: global memory, copied to shared memory when the kernel starts (112 bytes).
// Its rows are taken in groups of TR (a warp's unit of work); a group is NCH tiles for each of the product's one or
// two matrices: whole rows (NCH = 1), or a single row in NCH runs of CU units.
struct __align__(16) DecOp {
  const u8* w;
  const u8* w2;            // the "up" matrix of a gated product, else null
  float* y;
  const float* bias;
  const float* x;          // the activations as floats
  const float* norm_w;     // RMSNorm weights, or null
  float eps;
  int rows, cols, row_bytes, units;
  int tr;                  // rows a group
  int g0, ng;              // the product's groups among all the list's groups
  int nch, cu, chunk_bytes;
  u8 fmt, acc, f16_scale, lanes, kc;   // lanes a row; units a lane in a tile
  u8 after, restage;       // meet the other CTAs first; quantize X into shared memory first
  u8 pad[9];
};
static_assert(sizeof(DecOp) == 112, "DecOp is 112 bytes");

struct DecParams {
  const DecOp* ops;
  int nops;
  unsigned* bar;           // arrivals at the barrier between CTAs, counted up for ever
  unsigned bar_base;       // its value when this launch began
  int ring_bytes;          // per warp
  int max_cols;            // the staged activations' capacity
  int has_iq;
  unsigned* status;
};

// What every warp of the CTA shares, written once at the start (shared memory).
struct __align__(16) DecShared {
  const DecOp* ops;        // [nops] in shared memory
  unsigned* status;
  int nops, ring_bytes, gstep, pad;
  const u8* xq;            // the staged activations: planes of quants, scales, planes of sums
  const float* xs;
  const int16_t* bs;
  const uint2* iq_grid;
  const uint2* iq_smask;
};

// A warp's ring (shared memory).  C counts the tiles consumed; the fields after it are the issuing lane's: the next
// tile to issue is sub-tile ISS_S of group ISS_G (of product ISS_OP).  The ring's bytes lie elsewhere.
struct __align__(16) DecWarp {
  uint64_t bars[DEC_NBAR];
  int offs[DEC_NBAR];      // where tile i % DEC_NBAR starts in the ring
  int c;
  int issued, head;
  int iss_g, iss_s, iss_op;
  int pad[2];
};
static_assert(sizeof(DecWarp) == 128, "DecWarp is 128 bytes");

// bytes of the 16-byte aligned span that covers [SRC, SRC + LEN)
__device__ __forceinline__ uint32_t span16(const u8* src, uint32_t len) {
  const uintptr_t a0 = (uintptr_t)src & ~(uintptr_t)15;
  return (uint32_t)((((uintptr_t)src + len + 15) & ~(uintptr_t)15) - a0);
}

// where sub-tile S of group G of product O lies, and how long it is
__device__ __forceinline__ const u8* dec_tile_src(const DecOp& o, int g, int s, uint32_t& len) {
  const long long row0 = (long long)(g - o.g0) * o.tr;
  if (o.nch == 1) {
    len = (uint32_t)min(o.tr, o.rows - (int)row0) * (uint32_t)o.row_bytes;
    return (s ? o.w2 : o.w) + row0 * o.row_bytes;
  }
  const int part = s >= o.nch ? 1 : 0, ch = s - part * o.nch;
  len = (uint32_t)min(o.chunk_bytes, o.row_bytes - ch * o.chunk_bytes);
  return (part ? o.w2 : o.w) + row0 * o.row_bytes + (long long)ch * o.chunk_bytes;
}

// Lane 0: issue this warp's next tiles while a barrier and contiguous room in the ring are free.
__device__ __forceinline__ void dec_issue(DecWarp* cw, u8* ring, const DecShared* sh, int c) {
  const DecOp* ops = sh->ops;
  const int nops = sh->nops, gstep = sh->gstep, ring_bytes = sh->ring_bytes;
  int issued = cw->issued, head = cw->head, g = cw->iss_g, s = cw->iss_s, io = cw->iss_op;
  while (issued - c < DEC_NBAR) {
    while (io < nops && g >= ops[io].g0 + ops[io].ng) ++io;
    if (io >= nops) break;
    const DecOp& o = ops[io];
    uint32_t len;
    const u8* src = dec_tile_src(o, g, s, len);
    const int need = (int)span16(src, len);
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
    bulk_g2s(ring + off, (const void*)((uintptr_t)src & ~(uintptr_t)15), (uint32_t)need, &cw->bars[b]);
    ++issued;
    head = off + need;
    if (++s == (o.w2 ? 2 : 1) * o.nch) { s = 0; g += gstep; }
  }
  cw->issued = issued; cw->head = head; cw->iss_g = g; cw->iss_s = s; cw->iss_op = io;
}

// The CTAs meet: thread 0 of each, between two barriers of its CTA.  Arrivals are counted up for ever; the K-th
// meeting of a launch is complete when the count has reached BASE + K * NCTAS.  False after a bounded wait.
__device__ __forceinline__ bool dec_grid_barrier(unsigned* bar, unsigned target, unsigned* status) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
  unsigned long long t0 = 0;
  for (unsigned it = 1;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
    if ((int)(v - target) >= 0) return true;
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

// ---- the activations, quantized into planes in shared memory ---------------------------------
// Where piece P (the token's quants 16 P .. 16 P + 15) lies in FMT's planes of U units (formats.cuh: piece j of
// unit u at (j U + u) 16): the inverse of plane_src.
template <int FMT>
__device__ __forceinline__ int plane_dst(int p, int U) {
  if constexpr (FMT == ILL_Q6_K || FMT == ILL_Q2_K) {
    const int rem = p & 15, u = 4 * (p >> 4) + 2 * (rem >> 3) + (rem & 1), j = (rem & 7) >> 1;
    return (j * U + u) * 16;
  } else {
    constexpr int PPU = PlaneGeom<FMT>::PPU;
    return ((p % PPU) * U + p / PPU) * 16;
  }
}

// One Q8_K super-block B of the row (lane l holds values 8l .. 8l+7) into FMT's planes.
template <int FMT>
__device__ __forceinline__ void stage_block_q8k(const float (&v)[8], int lane, int b, int U, u8* xq, float* xs, int16_t* bs) {
  int q[8];
  float d;
  q8k_values(v, lane, q, d);
  uint32_t w0, w1;
  int s = q8k_pack(q, w0, w1);
  *(uint2*)(xq + plane_dst<FMT>(16 * b + (lane >> 1), U) + 8 * (lane & 1)) = make_uint2(w0, w1);
  if (lane == 0) xs[b] = d;
  s += __shfl_xor_sync(0xffffffffu, s, 1);  // the sum of 16: number m = lane / 2 of the block's sixteen
  if constexpr (FMT == ILL_Q6_K || FMT == ILL_Q2_K) {
    const int m = lane >> 1, u = 4 * b + 2 * (m >> 3) + (m & 1), g = (m & 7) >> 1;
    if (!(lane & 1)) bs[g * U + u] = (int16_t)s;
  } else if constexpr (FMT == ILL_Q4_K) {
    // unit k of the block = its sums 4k .. 4k+3 (lanes 8k .. 8k+7), packed as two sums of 32
    int s32 = s + __shfl_xor_sync(0xffffffffu, s, 2);
    const int hi = __shfl_down_sync(0xffffffffu, s32, 4);
    if (!(lane & 7)) ((int*)bs)[4 * b + (lane >> 3)] = (s32 & 0xffff) | (hi << 16);
  }
}

// Every CTA quantizes the product's activations into its own shared memory, in the planes the product's format
// reads (all threads; ends with a __syncthreads).  The arithmetic is rmsnorm_q8_kernel's and the quantizer
// kernels' (quant.cu, quantdev.cuh), the sum of squares in the order quantdev.cuh fixes.  X is read around L1
// (ld.cg): an earlier product of this same launch may have written it.  The loads of all the blocks a warp handles
// are issued before any is used (the vector comes from L2: one latency, not one per block); rows longer than HOLD
// blocks a warp take them in rounds.
constexpr int DEC_HOLD8 = 4;    // 256-wide groups a warp keeps in registers at a time (32 values a lane)
constexpr int DEC_HOLD0 = 16;   // Q8_0 blocks a warp keeps at a time (16 values a lane)

template <int FMT>
__device__ __noinline__ void dec_stage_fmt(const DecOp& op, u8* xq, float* xs, int16_t* bs, double* group_s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = op.x;
  const float* nw = op.norm_w;
  const int d = op.cols, ng = (d + 255) / 256, U = op.units;
  constexpr bool k8 = FMT != ILL_Q8_0;
  float sc = 1.0f;
  // Q8_K rows of up to HOLD8 groups a warp: the values loaded for the sum of squares are the ones quantized
  const bool held = k8 && ng <= DEC_HOLD8 * DEC_WARPS;
  float v[DEC_HOLD8][8];
  if (nw || held) {
    for (int g0 = 0; g0 < ng; g0 += DEC_HOLD8 * DEC_WARPS) {
#pragma unroll
      for (int j = 0; j < DEC_HOLD8; ++j) {
        const int g = g0 + warp + j * DEC_WARPS;
        if (g < ng) rms_load8<true>(x, d, g * 256 + 8 * lane, v[j]);
      }
      if (nw) {
#pragma unroll
        for (int j = 0; j < DEC_HOLD8; ++j) {
          const int g = g0 + warp + j * DEC_WARPS;
          if (g < ng) {
            const double s = rms_group_sum(v[j]);
            if (lane == 0) group_s[g] = s;
          }
        }
      }
    }
  }
  if (nw) {
    __syncthreads();
    sc = rms_scale(rms_total(group_s, ng, lane), d, op.eps);
  }
  if constexpr (k8) {
    for (int b0 = 0; b0 < ng; b0 += DEC_HOLD8 * DEC_WARPS) {
      if (!held) {
#pragma unroll
        for (int j = 0; j < DEC_HOLD8; ++j) {
          const int b = b0 + warp + j * DEC_WARPS;
          if (b < ng) rms_load8<true>(x, d, b * 256 + 8 * lane, v[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < DEC_HOLD8; ++j) {
        const int b = b0 + warp + j * DEC_WARPS;
        if (b < ng) {
          if (nw) {
            const float4 w0 = ((const float4*)(nw + b * 256))[2 * lane], w1 = ((const float4*)(nw + b * 256))[2 * lane + 1];
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = __fmul_rn(__fmul_rn(v[j][i], sc), ww[i]);
          }
          stage_block_q8k<FMT>(v[j], lane, b, U, xq, xs, bs);
        }
      }
    }
  } else {
    const int nb = d / 32;
    for (int b0 = 0; b0 < nb; b0 += DEC_HOLD0 * DEC_WARPS) {
      float u[DEC_HOLD0];
#pragma unroll
      for (int j = 0; j < DEC_HOLD0; ++j) {
        const int b = b0 + warp + j * DEC_WARPS;
        if (b < nb) u[j] = __ldcg(x + b * 32 + lane);
      }
#pragma unroll
      for (int j = 0; j < DEC_HOLD0; ++j) {
        const int b = b0 + warp + j * DEC_WARPS;
        if (b < nb) {
          float t = u[j];
          if (nw) t = __fmul_rn(__fmul_rn(t, sc), nw[b * 32 + lane]);
          float ds;
          const int q = q8_0_value(t, op.f16_scale, ds);
          xq[plane_dst<ILL_Q8_0>(2 * b + (lane >> 4), U) + (lane & 15)] = (u8)(i8)q;
          if (lane == 0) xs[b] = ds;
        }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void dec_stage_x(const DecOp& op, u8* xq, float* xs, int16_t* bs, double* group_s) {
  switch (op.fmt) {
    case ILL_Q8_0: dec_stage_fmt<ILL_Q8_0>(op, xq, xs, bs, group_s); break;
    case ILL_Q4_K: dec_stage_fmt<ILL_Q4_K>(op, xq, xs, bs, group_s); break;
    case ILL_Q6_K: dec_stage_fmt<ILL_Q6_K>(op, xq, xs, bs, group_s); break;
    case ILL_Q2_K: dec_stage_fmt<ILL_Q2_K>(op, xq, xs, bs, group_s); break;
    default: dec_stage_fmt<ILL_IQ2_XXS>(op, xq, xs, bs, group_s); break;
  }
}

// This warp's groups G_FIRST, G_FIRST + GSTEP, ... of the product OP.  False when a copy never landed.
// KC: units a lane multiplies in a tile (all of the lane's units when rows are taken whole).
template <int FMT, int KC, int AL>
__device__ __forceinline__ bool dec_run(const DecOp* op, DecWarp* cw, u8* ring, const DecShared* sh, int g_first) {
  const int lane = threadIdx.x & 31;
  const int L = op->lanes, units = op->units, tr = op->tr, rows = op->rows, row_bytes = op->row_bytes;
  const int g0 = op->g0, gend = g0 + op->ng, gstep = sh->gstep, acc = op->acc, nch = op->nch, cu = op->cu;
  const int chunk_bytes = op->chunk_bytes;
  const u8* const wg = op->w;
  const u8* const wu = op->w2;
  float* const y = op->y;
  const float* const bias = op->bias;
  const int sub = lane / L, sl = lane - sub * L, nsub = 32 / L;
  const int nparts = wu ? 2 : 1;
  IqTables iqt;
  iqt.grid = sh->iq_grid + (threadIdx.x & (IQ_COPIES - 1));
  iqt.smask = sh->iq_smask + (threadIdx.x & (IQ_COPIES - 1));
  ActP xa;
  xa.q = sh->xq; xa.s = sh->xs; xa.bs = sh->bs; xa.U = units;
  int c = cw->c;
  bool all_ok = true;
  for (int g = g_first; g < gend && all_ok; g += gstep) {
    const long long row0 = (long long)(g - g0) * tr;
    const int nrows = min(tr, rows - (int)row0);
    float car0 = 0.0f, car1 = 0.0f;  // a group taken in several tiles: the row's sums so far (gate, up)
    for (int s = 0; s < nparts * nch; ++s) {
      const int b = c % DEC_NBAR;
      bool ok = mbar_wait(&cw->bars[b], (uint32_t)(c / DEC_NBAR) & 1u, sh->status, ST_MV_WAIT + 0x10 + FMT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { all_ok = false; break; }
      const int off = cw->offs[b];  // written by lane 0 before it issued the copy this wait has just seen land
      const int part = s >= nch ? 1 : 0, ch = s - part * nch;
      const u8* src = (part ? wu : wg) + row0 * row_bytes + (nch > 1 ? (long long)ch * chunk_bytes : 0ll);
      // the tile's rows in the ring; a run of columns starts CH * CHUNK_BYTES into its row, and the unit offsets
      // below are taken from the row's start
      const u8* rows_s = ring + off + ((uintptr_t)src & 15) - (nch > 1 ? (size_t)ch * chunk_bytes : 0);
      const int ubase = ch * cu;
      const bool single = nparts * nch == 1;
#pragma unroll 1
      for (int r0 = 0; r0 < nrows; r0 += nsub) {
        const int rr = r0 + sub;
        const bool valid = rr < nrows;
        float sum = single ? 0.0f : (part ? car1 : car0);
        if (valid) {
          const u8* rowp = rows_s + (size_t)rr * row_bytes;
#pragma unroll
          for (int k = 0; k < KC; ++k) {
            const int u = ubase + sl + k * L;
            if (u < units && (nch == 1 || u < ubase + cu)) {
              UPos<FMT> up;
              unit_pos(up, u);
              XReg<FMT> x;
              load_x_planes<FMT>(x, xa, u);
              WReg<FMT> w;
              load_w<AL>(w, rowp, up, iqt);
              sum = __fadd_rn(sum, dot(w, x));
            }
          }
        }
        if (!single) { if (part) car1 = sum; else car0 = sum; }  // one row iteration a group then (the plan sees to it)
        if (single || s == nparts * nch - 1) {
          float v = single ? sum : car0, v2 = car1;
          for (int o = L >> 1; o > 0; o >>= 1) {
            v += __shfl_xor_sync(0xffffffffu, v, o);
            if (nparts == 2) v2 += __shfl_xor_sync(0xffffffffu, v2, o);
          }
          if (valid && sl == 0) {
            const long long row = row0 + rr;
            if (nparts == 2) {
              y[row] = (v / (1.0f + expf(-v))) * v2;
            } else {
              if (bias) v += bias[row];
              y[row] = acc ? __ldcg(y + row) + v : v;
            }
          }
        }
      }
      __syncwarp();  // every lane is done with the tile
      ++c;
      if (lane == 0) {
        cw->c = c;
        dec_issue(cw, ring, sh, c);
      }
    }
  }
  __syncwarp();
  return all_ok;
}

template <int FMT, int AL>
__device__ __forceinline__ bool dec_run_k(int kc, const DecOp* op, DecWarp* cw, u8* ring, const DecShared* sh, int g_first) {
  switch (kc) {
    case 1: return dec_run<FMT, 1, AL>(op, cw, ring, sh, g_first);
    case 2: return dec_run<FMT, 2, AL>(op, cw, ring, sh, g_first);
    case 3: return dec_run<FMT, 3, AL>(op, cw, ring, sh, g_first);
    case 4: return dec_run<FMT, 4, AL>(op, cw, ring, sh, g_first);
    case 5: return dec_run<FMT, 5, AL>(op, cw, ring, sh, g_first);
    case 6: if constexpr (FMT == ILL_Q8_0) return dec_run<FMT, 6, AL>(op, cw, ring, sh, g_first); break;
    case 7: if constexpr (FMT == ILL_Q8_0) return dec_run<FMT, 7, AL>(op, cw, ring, sh, g_first); break;
  }
  return false;  // not reached: the plan only holds 1..5 (Q8_0: ..7)
}

__global__ void __launch_bounds__(DEC_THREADS, 1) decode_kernel(const DecParams p) {
  extern __shared__ __align__(128) u8 smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // [rings][staged activations: planes of quants, scales, planes of sums][IQ2_XXS tables][the products][warps' state]
  // [misc]; every region is a multiple of 16 bytes
  u8* at = smem + (size_t)DEC_WARPS * p.ring_bytes;
  u8* xq_s = at;                           at += p.max_cols;
  float* xs_s = (float*)at;                at += p.max_cols / 32 * 4;
  int16_t* bs_s = (int16_t*)at;            at += p.max_cols / 16 * 2;
  uint2* iq_grid = (uint2*)at;
  uint2* iq_smask = iq_grid + IQ_COPIES * 256;
  if (p.has_iq) at += IQ_TABLE_BYTES;
  DecOp* ops_s = (DecOp*)at;               at += (size_t)p.nops * sizeof(DecOp);
  DecWarp* warps = (DecWarp*)at;           at += DEC_WARPS * sizeof(DecWarp);
  DecShared* sh = (DecShared*)at;          at += sizeof(DecShared);
  double* group_s = (double*)at;           // [RMS_MAX_GROUPS]

  for (int i = tid; i < p.nops * (int)(sizeof(DecOp) / 16); i += DEC_THREADS) ((uint4*)ops_s)[i] = ((const uint4*)p.ops)[i];
  const int gstep = gridDim.x * DEC_WARPS, gw = blockIdx.x * DEC_WARPS + warp;
  DecWarp* cw = warps + warp;
  u8* ring = smem + (size_t)warp * p.ring_bytes;
  if (lane == 0) {
    for (int b = 0; b < DEC_NBAR; ++b) mbar_init(&cw->bars[b], 1);
    mbar_fence_init();
    cw->c = 0; cw->issued = 0; cw->head = 0; cw->iss_g = gw; cw->iss_s = 0; cw->iss_op = 0;
  }
  if (tid == 0) {
    sh->ops = ops_s; sh->status = p.status; sh->nops = p.nops; sh->ring_bytes = p.ring_bytes; sh->gstep = gstep;
    sh->xq = xq_s; sh->xs = xs_s; sh->bs = bs_s; sh->iq_grid = iq_grid; sh->iq_smask = iq_smask;
  }
  if (p.has_iq) iq_tables_fill(iq_grid, iq_smask, ill_iq2xxs_grid, ill_ksigns_iq2xs);
  __syncthreads();
  if (lane == 0) dec_issue(cw, ring, sh, 0);  // the weights depend on nothing: start streaming
  __syncwarp();

  // LOST: this warp gave up a wait.  It keeps walking the list (the CTA's barriers count on it) but does no more
  // work; the CTA learns of it at the next point where its warps meet and leaves the list there, all warps together.
  bool lost = false, broke = false;
  unsigned meetings = 0;
  for (int oi = 0; oi < p.nops; ++oi) {
    const DecOp* op = ops_s + oi;
    bool synced = false;
    if (op->after) {
      __syncthreads();  // this CTA's part of everything before is written
      ++meetings;
      bool bad = false;
      if (tid == 0) bad = !dec_grid_barrier(p.bar, p.bar_base + meetings * gridDim.x, p.status);
      if (__syncthreads_or(bad || lost)) { broke = true; break; }
      synced = true;
    }
    if (op->restage) {
      // every warp is done with the activations staged before
      if (!synced && __syncthreads_or(lost)) { broke = true; break; }
      dec_stage_x(*op, xq_s, xs_s, bs_s, group_s);
    }
    const int g0 = op->g0;
    int d = (gw - g0) % gstep;
    if (d < 0) d += gstep;
    const int g_first = g0 + d;
    if (!lost && g_first < g0 + op->ng) {
      const int kc = op->kc;
      bool ok = false;
      switch (op->fmt) {
        case ILL_Q8_0: ok = dec_run_k<ILL_Q8_0, 1>(kc, op, cw, ring, sh, g_first); break;
        case ILL_Q4_K: ok = dec_run_k<ILL_Q4_K, 16>(kc, op, cw, ring, sh, g_first); break;
        case ILL_Q6_K: ok = dec_run_k<ILL_Q6_K, 1>(kc, op, cw, ring, sh, g_first); break;
        case ILL_Q2_K: ok = dec_run_k<ILL_Q2_K, 4>(kc, op, cw, ring, sh, g_first); break;
        case ILL_IQ2_XXS: ok = dec_run_k<ILL_IQ2_XXS, 1>(kc, op, cw, ring, sh, g_first); break;
      }
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
enum { DL_NOPS = 0, DL_GRID, DL_SMEM, DL_TILES, DL_RING, DL_MAXCOLS, DL_IQ, DL_MEETINGS, DL_EPOCH, DL_MAGIC, DL_WORDS };
constexpr int DL_MAGIC_VALUE = 0x1d1ec0de;
static_assert(DL_WORDS <= ILL_DECODE_LAUNCH_WORDS, "the caller's array holds the launch words");

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
    if ((o.w & 15) || (o.w2 & 15) || (o.x & 15) || (o.norm_w & 15) || (o.y & 3) || (o.bias & 3)) return ILL_ERR_ALIGN;
    if (o.cols > max_cols) max_cols = o.cols;
    if (o.fmt == ILL_IQ2_XXS) has_iq = 1;
  }
  max_cols = (int)up_to((uint32_t)max_cols, 256);
  // shared memory: everything but the rings first, the rings get the rest
  const uint32_t fixed = (uint32_t)max_cols + (uint32_t)max_cols / 32 * 4 + (uint32_t)max_cols / 16 * 2 + (has_iq ? IQ_TABLE_BYTES : 0) +
                         (uint32_t)nops * (uint32_t)sizeof(DecOp) + DEC_WARPS * (uint32_t)sizeof(DecWarp) + (uint32_t)sizeof(DecShared) +
                         RMS_MAX_GROUPS * 8;
  const int budget = smem_max - 1024;
  if ((int)fixed + DEC_WARPS * 8192 > budget) return ILL_ERR_TOO_LARGE;
  const int ring = (int)((((uint32_t)budget - fixed) / DEC_WARPS) & ~127u);
  const int limit = ring / 2 - 32;  // a tile's bytes at most: the next one fits beside it
  std::vector<DecOp> dev_ops((size_t)nops);
  long long groups = 0;
  int meetings = 0;
  const long long gwarps = (long long)sms * DEC_WARPS;
  for (int i = 0; i < nops; ++i) {
    const ill_decode_op& o = ops[i];
    DecOp& d = dev_ops[(size_t)i];
    d = DecOp();
    const int bw = fmt_block_weights(o.fmt), bb = fmt_block_bytes(o.fmt), uw = (o.fmt == ILL_Q8_0 || o.fmt == ILL_IQ2_XXS) ? 32 : 64;
    const bool glu = o.kind == ILL_OP_GLU;
    d.w = (const u8*)(uintptr_t)o.w;
    d.w2 = (const u8*)(uintptr_t)o.w2;
    d.y = (float*)(uintptr_t)o.y;
    d.bias = (const float*)(uintptr_t)o.bias;
    d.x = (const float*)(uintptr_t)o.x;
    d.norm_w = (const float*)(uintptr_t)o.norm_w;
    d.eps = o.eps;
    d.fmt = (u8)o.fmt;
    d.acc = o.acc ? 1 : 0;
    d.f16_scale = o.f16_scale ? 1 : 0;
    d.rows = o.rows;
    d.cols = o.cols;
    d.row_bytes = o.cols / bw * bb;
    d.units = o.cols / uw;
    // lanes a row and units a lane as the one-token product picks them (the order of a row's additions follows from
    // the pair); rows it would not keep in registers: 32 lanes, as many units a lane as it takes
    const bool big = (long long)o.rows * d.row_bytes >= (16ll << 20);
    int lanes = 0, upt = 0;
    if (!mv_pick_lanes(o.fmt, d.units, glu, big, &lanes, &upt)) { lanes = 32; upt = (d.units + 31) / 32; }
    int nsub = 32 / lanes;
    const int kmax = o.fmt == ILL_Q8_0 ? 7 : 5;
    if ((long long)nsub * d.row_bytes > limit && lanes < 32 && d.row_bytes > limit) { lanes = 32; upt = (d.units + 31) / 32; nsub = 1; }
    d.lanes = (u8)lanes;
    if (d.row_bytes <= limit && upt <= kmax) {
      // whole rows.  A gated product's group is one pass of the warp (its gate rows' sums are carried to its up
      // rows); a plain product's is about 4 KB, cut finer when the product is small (every warp should get some).
      // Rows that do not fit side by side: fewer a group, and the lanes past them idle.
      long long tr = nsub;
      if (!glu) {
        long long target = (long long)o.rows * d.row_bytes / (2 * gwarps);
        if (target > 4096) target = 4096;
        if (target < 1024) target = 1024;
        tr = target / d.row_bytes / nsub * nsub;
        if (tr < nsub) tr = nsub;
      }
      while (tr > 1 && tr * d.row_bytes > limit) tr = tr > nsub ? tr - nsub : tr - 1;
      if (tr > o.rows) tr = o.rows;
      d.tr = (int)tr;
      d.nch = 1;
      d.cu = d.units;
      d.kc = (u8)upt;
      d.chunk_bytes = d.row_bytes;
    } else {
      // a row at a time, in runs of KC * 32 units (whole blocks): about 4 KB a tile
      const int upb = bw / uw;  // units a block
      int kc = kmax < upt ? kmax : upt;
      while (kc > 1 && ((long long)kc * 32 / upb * bb > limit || (long long)kc * 32 / upb * bb > 4096)) --kc;
      if ((long long)kc * 32 / upb * bb > limit) return ILL_ERR_UNSUPPORTED;
      d.tr = 1;
      d.cu = kc * 32;
      d.kc = (u8)kc;
      d.nch = (d.units + d.cu - 1) / d.cu;
      d.chunk_bytes = d.cu / upb * bb;
    }
    d.ng = (int)((o.rows + d.tr - 1) / d.tr);
    d.g0 = (int)groups;
    groups += d.ng;
    if (groups > 0x7fffffffll / 2) return ILL_ERR_TOO_LARGE;
    d.after = (i > 0 && o.after) ? 1 : 0;
    meetings += d.after;
    // the activations are staged again when they change -- or the planes they are laid out in do
    const ill_decode_op* pv = i ? &ops[i - 1] : nullptr;
    d.restage = (!pv || d.after || pv->x != o.x || pv->norm_w != o.norm_w || pv->eps != o.eps || pv->cols != o.cols || pv->fmt != o.fmt ||
                 (o.fmt == ILL_Q8_0 && (pv->f16_scale != 0) != (o.f16_scale != 0)))
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
  launch[DL_TILES] = (int)groups;
  launch[DL_RING] = ring;
  launch[DL_MAXCOLS] = max_cols;
  launch[DL_IQ] = has_iq;
  launch[DL_MEETINGS] = meetings;
  launch[DL_EPOCH] = 0;   // arrivals at the barrier so far (the count in PLAN starts at 0 with it)
  launch[DL_MAGIC] = DL_MAGIC_VALUE;
  return ILL_OK;
}

extern "C" int ill_decode_run(ill_dptr plan, int32_t* launch, ill_stream stream) {
  if (!plan || !launch || launch[DL_MAGIC] != DL_MAGIC_VALUE || launch[DL_NOPS] < 1 || launch[DL_GRID] < 1) return ILL_ERR_ARG;
  if (plan & 127) return ILL_ERR_ALIGN;
  DecParams p;
  p.ops = (const DecOp*)(uintptr_t)(plan + 128);
  p.nops = launch[DL_NOPS];
  p.bar = (unsigned*)(uintptr_t)plan;
  p.bar_base = (unsigned)launch[DL_EPOCH];
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
  if (e != cudaSuccess) return cuda_fail(e);
  // this token's meetings are counted on from here: the next run's first target lies past them
  launch[DL_EPOCH] = (int32_t)((unsigned)launch[DL_EPOCH] + (unsigned)launch[DL_MEETINGS] * (unsigned)launch[DL_GRID]);
  return ILL_OK;
}
