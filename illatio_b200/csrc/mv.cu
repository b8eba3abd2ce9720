// mv.cu -- dequant-fused quantized matrix x vector products (decode path).
//
// HBM-bound: one pass over the raw GGUF bytes.  One token (mvw_kernel): every warp
// streams its own tiles of whole rows through its own ring of shared-memory stages
// with 1-D bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier per stage; no CTA-wide barrier in the loop), the lanes that share a row
// keep that row's activations in registers, unpack the blocks from shared memory,
// take exact integer dots with dp4a, scale in fp32 and meet with shuffles.  Several
// tokens (mvn_kernel): a CTA-wide ring, the activations in shared memory, each
// weight read once.  A copy covers the 16-byte aligned superset of the tile's byte
// range, so rows of any byte length and base alignment are read where they lie (no
// repacking or padding).
//
// Replaces mv_q8 / mv_q8_3 / mv_q8_glu (src/cuda/dense.cu:194-250), mv_k /
// mv_k_glu (src/cuda/kquant.cu:169-193), d4_mvq8 / d4_mvq8n (src/cuda/ds4f.cu:
// 50-107) and the per-expert d4_mv_iq2_xxs / d4_mv_q2_k (src/cuda/ds4f.cu:769,
// 837) of the reference.
#include "formats.cuh"
#include "iq2xxs_tables.cuh"
#include "host.h"

namespace ill {

constexpr int MV_THREADS = 256;
constexpr int MV_MAX_MATS = 3;
constexpr int MV_MAX_TOK = 16;



struct MvParams {
  // matrices (PLAIN: up to three sharing the activations; GLU: gate, up)
  const u8* w[MV_MAX_MATS];
  float* y[MV_MAX_MATS];
  const float* bias[MV_MAX_MATS];
  int rows[MV_MAX_MATS];
  int tile0[MV_MAX_MATS + 1];  // first tile of each matrix; tile0[nmat] = tiles per segment
  int nmat;
  int cols, row_bytes, units;  // units per row
  // activations (global): token t at xq + t*cols etc.
  const i8* xq;
  const float* xs;
  const int16_t* xsum;
  int n;                 // tokens
  int acc;
  int rows_per_tile, lanes_per_row;
  int nchunks;           // one-token kernel: column chunks a row is staged in (1: whole rows)
  int chunk_units;       // units per chunk
  uint32_t chunk_bytes;
  uint32_t stage_bytes;  // bytes of one stage (one matrix' part of it in GLU modes)
  int nstages;
  uint32_t x_bytes;      // shared bytes of the activation region
  uint32_t xs_off, bs_off;
  // segments (grid.y): expert z's weights at ptrs[z] + add (+ up_add for "up"),
  // its activations at token z*x_seg (0: shared), its output at y + z*y_seg
  const unsigned long long* ptrs;
  long long add, up_add;
  int x_seg;
  long long y_seg;
  const float* seg_w;    // MOE_GLU: weight of segment z
  float clamp;
  unsigned int* status;
  // the row-split head: the one-token product's results go to every rank's buffer (its own included) instead of
  // y[0], at y_peers[r] + 4 (y_peer_off + row), and the CTA that finishes last meets the other ranks
  const unsigned long long* y_peers;  // 0: off
  long long y_peer_off;
  const unsigned long long* flag_peers;
  unsigned* flags;
  int world, rank, slot;
  unsigned epoch;
  unsigned long long wait_ns;
};

__device__ unsigned g_mv_ticket;  // CTAs of the running peer-storing product that are through (one such call at a time a device)

__device__ __forceinline__ void store_to_peers(const MvParams& p, long long row, float v) {
  for (int r = 0; r < p.world; ++r) ((float*)(uintptr_t)p.y_peers[r])[p.y_peer_off + row] = v;
}

// The row r0 .. of one matrix that a tile covers, and where its bytes are.
struct TileRef {
  int m, row0, nrows;
  const u8* g;  // global address of the first row
};

__device__ __forceinline__ TileRef tile_ref(const MvParams& p, int tile, const u8* const* wbase) {
  TileRef t;
  int m = 0;
#pragma unroll
  for (int i = 1; i < MV_MAX_MATS; ++i)
    if (i < p.nmat && tile >= p.tile0[i]) m = i;
  t.m = m;
  t.row0 = (tile - p.tile0[m]) * p.rows_per_tile;
  t.nrows = min(p.rows_per_tile, p.rows[m] - t.row0);
  t.g = wbase[m] + (long long)t.row0 * p.row_bytes;
  return t;
}

template <int FMT, int MODE, int NT>
__global__ void __launch_bounds__(MV_THREADS) mvn_kernel(const MvParams p) {
  extern __shared__ __align__(128) u8 smem[];
  constexpr bool GLU = MODE != MODE_PLAIN;
  constexpr bool IQ = FMT == ILL_IQ2_XXS;
  const int tid = threadIdx.x;
  const int z = blockIdx.y;

  u8* xreg = smem;
  u8* stage0 = smem + p.x_bytes;
  const uint32_t stage_stride = p.stage_bytes * (GLU ? 2u : 1u);
  u8* after = stage0 + (size_t)stage_stride * p.nstages;
  uint2* iq_grid = (uint2*)after;
  uint2* iq_smask = iq_grid + IQ_COPIES * 256;
  uint64_t* full = (uint64_t*)(after + (IQ ? IQ_TABLE_BYTES : 0));

  // this segment's matrices
  const u8* wbase[MV_MAX_MATS];
  if (p.ptrs) {
    const u8* b = (const u8*)(uintptr_t)p.ptrs[z] + p.add;
    wbase[0] = b;
    wbase[1] = b + p.up_add;
    wbase[2] = b;
  } else {
#pragma unroll
    for (int i = 0; i < MV_MAX_MATS; ++i) wbase[i] = p.w[i];
  }
  const int ntiles = p.tile0[p.nmat];
  const int first = blockIdx.x, step = gridDim.x;

  auto issue = [&](int tile, int s) {
    const TileRef t = tile_ref(p, tile, wbase);
    const uint32_t len = (uint32_t)t.nrows * (uint32_t)p.row_bytes;
    u8* dst = stage0 + (size_t)s * stage_stride;
    const uintptr_t a0 = (uintptr_t)t.g & ~(uintptr_t)15;
    const uint32_t bytes = (uint32_t)((((uintptr_t)t.g + len + 15) & ~(uintptr_t)15) - a0);
    if (GLU) {
      const u8* g2 = wbase[1] + (long long)t.row0 * p.row_bytes;
      const uintptr_t b0 = (uintptr_t)g2 & ~(uintptr_t)15;
      const uint32_t bytes2 = (uint32_t)((((uintptr_t)g2 + len + 15) & ~(uintptr_t)15) - b0);
      mbar_expect_tx(&full[s], bytes + bytes2);
      bulk_g2s(dst, (const void*)a0, bytes, &full[s]);
      bulk_g2s(dst + p.stage_bytes, (const void*)b0, bytes2, &full[s]);
    } else {
      mbar_expect_tx(&full[s], bytes);
      bulk_g2s(dst, (const void*)a0, bytes, &full[s]);
    }
  };

  if (tid == 0) {
    for (int s = 0; s < p.nstages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    // weights do not depend on the previous kernel: start streaming them now
    for (int s = 0; s < p.nstages; ++s) {
      const int tile = first + s * step;
      if (tile < ntiles) issue(tile, s);
    }
  }
  if (IQ) iq_tables_fill(iq_grid, iq_smask, ill_iq2xxs_grid, ill_ksigns_iq2xs);
  pdl_launch_dependents();
  pdl_wait();  // activations may come from the previous kernel

  // activations -> shared memory
  {
    const int ntok_x = p.x_seg ? 1 : p.n;  // a segment with its own activations has one token
    const long long tok0 = (long long)z * p.x_seg;
    const int nsc = FMT == ILL_Q8_0 ? p.cols / 32 : p.cols / 256;
    const uint4* src = (const uint4*)(p.xq + tok0 * p.cols);
    uint4* dst = (uint4*)xreg;
    for (int i = tid; i < ntok_x * p.cols / 16; i += MV_THREADS) dst[i] = src[i];
    const float* ssrc = p.xs + tok0 * nsc;
    float* sdst = (float*)(xreg + p.xs_off);
    for (int i = tid; i < ntok_x * nsc; i += MV_THREADS) sdst[i] = ssrc[i];
    if (FMT != ILL_Q8_0 && FMT != ILL_IQ2_XXS) {
      const int16_t* bsrc = p.xsum + tok0 * (p.cols / 16);
      int16_t* bdst = (int16_t*)(xreg + p.bs_off);
      for (int i = tid; i < ntok_x * p.cols / 16; i += MV_THREADS) bdst[i] = bsrc[i];
    }
  }
  __syncthreads();

  const int L = p.lanes_per_row;
  const int group = tid / L, lane_in = tid % L, ngroups = MV_THREADS / L;
  const int nsc = FMT == ILL_Q8_0 ? p.cols / 32 : p.cols / 256;
  IqTables iqt;
  iqt.grid = iq_grid + (threadIdx.x & (IQ_COPIES - 1));
  iqt.smask = iq_smask + (threadIdx.x & (IQ_COPIES - 1));

  int it = 0;
  bool failed = false;
  for (int tile = first; tile < ntiles; tile += step, ++it) {
    const int s = it % p.nstages;
    const uint32_t parity = (uint32_t)(it / p.nstages) & 1u;
    const bool ok = mbar_wait(&full[s], parity, p.status, ST_MV_WAIT + FMT);
    if (__syncthreads_or(!ok)) { failed = true; break; }

    const TileRef t = tile_ref(p, tile, wbase);
    const u8* sbase = stage0 + (size_t)s * stage_stride;
    const u8* rows_s = sbase + ((uintptr_t)t.g & 15);
    const u8* rows_u = nullptr;
    if (GLU) rows_u = sbase + p.stage_bytes + ((uintptr_t)(wbase[1] + (long long)t.row0 * p.row_bytes) & 15);

    const int passes = (t.nrows + ngroups - 1) / ngroups;
    for (int ps = 0; ps < passes; ++ps) {
      const int r = ps * ngroups + group;
      const bool valid = r < t.nrows;
      float sum[NT], sum2[GLU ? NT : 1];
#pragma unroll
      for (int k = 0; k < NT; ++k) sum[k] = 0.0f;
      sum2[0] = 0.0f;
      if (valid) {
        const u8* rowp = rows_s + (size_t)r * p.row_bytes;
        for (int u = lane_in; u < p.units; u += L) {
          WReg<FMT> w;
          UPos<FMT> up;
          unit_pos(up, u);
          load_w(w, rowp, up, iqt);
          if constexpr (GLU) {
            WReg<FMT> w2;
            const u8* rowu = rows_u + (size_t)r * p.row_bytes;
            load_w(w2, rowu, up, iqt);
            ActS a;
            a.q = (const i8*)xreg;
            a.s = (const float*)(xreg + p.xs_off);
            a.bs = (const int16_t*)(xreg + p.bs_off);
            XReg<FMT> x;
            load_x(x, a, u);
            sum[0] = __fadd_rn(sum[0], dot(w, x));
            sum2[0] = __fadd_rn(sum2[0], dot(w2, x));
          } else {
#pragma unroll
            for (int k = 0; k < NT; ++k) {
              if (k < p.n) {
                ActS a;
                a.q = (const i8*)xreg + (size_t)k * p.cols;
                a.s = (const float*)(xreg + p.xs_off) + (size_t)k * nsc;
                a.bs = (const int16_t*)(xreg + p.bs_off) + (size_t)k * (p.cols / 16);
                XReg<FMT> x;
                load_x(x, a, u);
                sum[k] = __fadd_rn(sum[k], dot(w, x));
              }
            }
          }
        }
      }
      // lanes of a row meet
      for (int o = L >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int k = 0; k < NT; ++k) sum[k] += __shfl_xor_sync(0xffffffffu, sum[k], o);
        if (GLU) sum2[0] += __shfl_xor_sync(0xffffffffu, sum2[0], o);
      }
      if (valid && lane_in == 0) {
        const long long row = t.row0 + r;
        if constexpr (MODE == MODE_GLU) {
          const float g = sum[0];
          p.y[0][(long long)z * p.y_seg + row] = (g / (1.0f + expf(-g))) * sum2[0];
        } else if constexpr (MODE == MODE_MOE_GLU) {
          // D4-ROUTED!'s middle (src/ds4f.lisp:1016-1019): silu(min(g,c)) * clamp(u) * weight
          float g = sum[0], uu = sum2[0];
          if (p.clamp > 1e-6f) { g = fminf(g, p.clamp); uu = fmaxf(-p.clamp, fminf(uu, p.clamp)); }
          const float sg = g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : (expf(g) / (1.0f + expf(g)));
          p.y[0][(long long)z * p.y_seg + row] = ((g * sg) * uu) * p.seg_w[z];
        } else {
          float* y = p.y[t.m] + (long long)z * p.y_seg;
          const float* bias = p.bias[t.m];
#pragma unroll
          for (int k = 0; k < NT; ++k) {
            if (k < p.n) {
              float v = sum[k];
              if (bias) v += bias[row];
              const long long o = (long long)k * p.rows[t.m] + row;
              y[o] = p.acc ? y[o] + v : v;
            }
          }
        }
      }
    }
    __syncthreads();  // every lane is done with the stage
    if (tid == 0) {
      const int nt = tile + p.nstages * step;
      if (nt < ntiles) issue(nt, s);
    }
  }
  if (failed) {
    // give copies still in flight a bounded time to land before the CTA's
    // shared memory is released
    int it2 = it;
    for (int tile = first + it * step; tile < ntiles && it2 < it + p.nstages; tile += step, ++it2)
      mbar_wait(&full[it2 % p.nstages], (uint32_t)(it2 / p.nstages) & 1u, nullptr, 0);
  }
}

// ---- one token: a pipeline per warp ------------------------------------------------
//
// Each warp streams its own tiles through its own ring of stages: lane 0 issues
// the bulk copies, all lanes wait on the stage's mbarrier, and after a __syncwarp
// the stage is refilled -- no CTA-wide barrier in the loop.  A row is shared by L
// consecutive lanes (L = 8, 16 or 32, so 32/L rows are in progress per warp);
// lane sl of them owns units sl, sl+L, ... and keeps those units' activations in
// registers, loaded from global memory once.  A row's lanes meet with log2(L)
// shuffles.
//
// A warp's unit of work is a group of G stages whose sums it carries in
// registers: the gate rows and then the up rows of a gated product (G = 2), or,
// for rows too long to stage whole (XS), a row's column chunks one after another
// (G = chunks, or twice that when gated).  In XS mode the activations are staged
// in shared memory once per CTA and read from there.
constexpr int MV_MAXRI = 4;  // row iterations a warp tile may take when sums are carried

template <int FMT, int MODE, int UPT, int AL, bool XS>
__global__ void __launch_bounds__(MV_THREADS) mvw_kernel(const MvParams p) {
  extern __shared__ __align__(128) u8 smem[];
  constexpr bool GLU = MODE == MODE_GLU || MODE == MODE_MOE_GLU;
  constexpr bool IQ = FMT == ILL_IQ2_XXS;
  const int WARPS = blockDim.x >> 5;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int z = blockIdx.y;

  u8* wstage = smem + (size_t)warp * p.stage_bytes * p.nstages;
  u8* after = smem + (size_t)WARPS * p.stage_bytes * p.nstages;
  uint2* iq_grid = (uint2*)after;
  uint2* iq_smask = iq_grid + IQ_COPIES * 256;
  uint64_t* full = (uint64_t*)(after + (IQ ? IQ_TABLE_BYTES : 0)) + warp * p.nstages;
  u8* xsm = after + (IQ ? IQ_TABLE_BYTES : 0) + 8 * WARPS * p.nstages;  // XS: the activations (16-byte aligned)

  const u8* wbase[MV_MAX_MATS];
  if (p.ptrs) {
    const u8* b = (const u8*)(uintptr_t)p.ptrs[z] + p.add;
    wbase[0] = b;
    wbase[1] = b + p.up_add;
    wbase[2] = b;
  } else {
#pragma unroll
    for (int i = 0; i < MV_MAX_MATS; ++i) wbase[i] = p.w[i];
  }
  const int ngroups = p.tile0[p.nmat];
  const int NC = XS ? p.nchunks : 1;
  const int G = (GLU ? 2 : 1) * NC;
  const int first = blockIdx.x * WARPS + warp, step = gridDim.x * WARPS;

  // stage G of group GRP: which matrix (gate / up), which column chunk, where its bytes are
  auto locate = [&](int grp, int g, int& nrows, long long& row0, int& m) -> const u8* {
    const TileRef t = tile_ref(p, grp, wbase);
    nrows = t.nrows;
    row0 = t.row0;
    m = t.m;
    const int which = GLU ? g / NC : 0, c = g - which * NC;
    const u8* base = GLU ? (wbase[which] + (long long)t.row0 * p.row_bytes) : t.g;
    return base + (size_t)c * p.chunk_bytes;
  };
  auto issue = [&](int grp, int g, int s) {
    int nrows, m;
    long long row0;
    const u8* src = locate(grp, g, nrows, row0, m);
    uint32_t len = (uint32_t)nrows * (uint32_t)p.row_bytes;
    if (XS) {
      const int c = g % NC;
      len = min(p.chunk_bytes, (uint32_t)p.row_bytes - (uint32_t)c * p.chunk_bytes);
    }
    const uintptr_t a0 = (uintptr_t)src & ~(uintptr_t)15;
    const uint32_t bytes = (uint32_t)((((uintptr_t)src + len + 15) & ~(uintptr_t)15) - a0);
    mbar_expect_tx(&full[s], bytes);
    bulk_g2s(wstage + (size_t)s * p.stage_bytes, (const void*)a0, bytes, &full[s]);
  };

  // the warp's stages in order: (group, g) for i = 0, 1, ...
  int i_grp = first, i_g = 0;  // next stage to issue
  int n_issued = 0, n_done = 0;  // stages issued (lane 0 counts) and consumed by this warp
  auto issue_next = [&](int s) {
    if (i_grp < ngroups) {
      issue(i_grp, i_g, s);
      ++n_issued;
      if (++i_g == G) { i_g = 0; i_grp += step; }
    }
  };
  if (lane == 0) {
    for (int s = 0; s < p.nstages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    for (int s = 0; s < p.nstages; ++s) issue_next(s);  // weights do not depend on the previous kernel
  }
  if (IQ) iq_tables_fill(iq_grid, iq_smask, ill_iq2xxs_grid, ill_ksigns_iq2xs);
  pdl_launch_dependents();
  pdl_wait();  // the activations may come from the previous kernel

  const int L = p.lanes_per_row, sub = lane / L, sl = lane - sub * L, nsub = 32 / L;
  XReg<FMT> x[XS ? 1 : UPT];
  UPos<FMT> up[UPT];
  ActP xa;
  {
    const long long tok0 = (long long)z * p.x_seg;
    const int nsc = FMT == ILL_Q8_0 ? p.cols / 32 : p.cols / 256;
    ActS a;
    a.q = p.xq + tok0 * p.cols;
    a.s = p.xs + tok0 * nsc;
    a.bs = p.xsum + tok0 * (p.cols / 16);
    if constexpr (XS) planes_fill<FMT>(xsm, a, p.units, nsc, xa);
#pragma unroll
    for (int k = 0; k < UPT; ++k) {
      const int u = sl + k * L;
      unit_pos(up[k], u);
      if constexpr (!XS) {
        if (u < p.units) load_x(x[k], a, u);
      }
    }
  }
  if (IQ || XS) __syncthreads();  // tables / activations staged
  else __syncwarp();
  IqTables iqt;
  iqt.grid = iq_grid + (threadIdx.x & (IQ_COPIES - 1));
  iqt.smask = iq_smask + (threadIdx.x & (IQ_COPIES - 1));

  int s = 0;
  uint32_t parity = 0;
  bool dead = false;
  for (int grp = first; grp < ngroups && !dead; grp += step) {
    float acc[MV_MAXRI], acc2[MV_MAXRI];
#pragma unroll
    for (int i = 0; i < MV_MAXRI; ++i) acc[i] = acc2[i] = 0.0f;
    int nrows = 0, m = 0;
    long long row0 = 0;
    for (int g = 0; g < G; ++g) {
      bool ok = mbar_wait(&full[s], parity, p.status, ST_MV_WAIT + FMT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { dead = true; break; }  // the copy never landed: the status word says so; nothing is read
      const u8* src = locate(grp, g, nrows, row0, m);
      const u8* rows_s = wstage + (size_t)s * p.stage_bytes + ((uintptr_t)src & 15);
      const int which = GLU ? g / NC : 0, c = g - which * NC;
      const int ubase = XS ? c * p.chunk_units : 0;
      const int uend = XS ? min(p.units, ubase + p.chunk_units) : p.units;
      // plain, whole rows: the sums of a row iteration are written at once, so a tile may take any
      // number of them; carried sums (gated, chunked) are limited to MV_MAXRI iterations
#pragma unroll 1
      for (int r0 = 0, ri = 0; r0 < nrows; r0 += nsub, ++ri) {
        const int r = r0 + sub;
        const bool valid = r < nrows;
        float sum = 0.0f;
        if (valid) {
          const u8* rowp = rows_s + (size_t)r * p.row_bytes;
#pragma unroll
          for (int k = 0; k < UPT; ++k) {
            const int u = ubase + sl + k * L;
            if ((!XS && k < UPT - 1) || u < uend) {
              if constexpr (XS) load_x_planes<FMT>(x[0], xa, u);
              WReg<FMT> w;
              load_w<AL>(w, rowp, up[k], iqt);
              sum = __fadd_rn(sum, dot(w, x[XS ? 0 : k]));
            }
          }
        }
        if constexpr (!GLU && !XS) {
          for (int o = L >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
          if (valid && sl == 0) {
            const long long row = row0 + r;
            float* y = p.y[m] + (long long)z * p.y_seg;
            float v = sum;
            if (p.bias[m]) v += p.bias[m][row];
            if constexpr (MODE == MODE_PEERS) store_to_peers(p, row, v);
            else y[row] = p.acc ? y[row] + v : v;
          }
        } else {
          // ri < MV_MAXRI by the plan; the select chain keeps the sums in registers
#pragma unroll
          for (int i = 0; i < MV_MAXRI; ++i) {
            if (i == ri) { if (which == 0) acc[i] += sum; else acc2[i] += sum; }
          }
        }
      }
      __syncwarp();  // every lane is done with the stage
      if (lane == 0) issue_next(s);
      ++n_done;
      if (++s == p.nstages) { s = 0; parity ^= 1u; }
    }
    if constexpr (GLU || XS) {
      if (dead) break;
#pragma unroll
      for (int i = 0; i < MV_MAXRI; ++i) {
        const int r = i * nsub + sub;
        if (i * nsub >= nrows) break;
        float v = acc[i], v2 = acc2[i];
        for (int o = L >> 1; o > 0; o >>= 1) {
          v += __shfl_xor_sync(0xffffffffu, v, o);
          if constexpr (GLU) v2 += __shfl_xor_sync(0xffffffffu, v2, o);
        }
        if (r < nrows && sl == 0) {
          const long long row = row0 + r;
          if constexpr (MODE == MODE_GLU) {
            p.y[0][(long long)z * p.y_seg + row] = (v / (1.0f + expf(-v))) * v2;
          } else if constexpr (MODE == MODE_MOE_GLU) {
            // D4-ROUTED!'s middle (src/ds4f.lisp:1016-1019): silu(min(g,c)) * clamp(u) * weight
            float g = v, uu = v2;
            if (p.clamp > 1e-6f) { g = fminf(g, p.clamp); uu = fmaxf(-p.clamp, fminf(uu, p.clamp)); }
            float sg;
            if (g >= 0.0f) sg = __fdiv_rn(1.0f, 1.0f + expf(-g));
            else { const float e = expf(g); sg = __fdiv_rn(e, 1.0f + e); }
            p.y[0][(long long)z * p.y_seg + row] = __fmul_rn(__fmul_rn(__fmul_rn(g, sg), uu), p.seg_w[z]);
          } else {
            float* y = p.y[m] + (long long)z * p.y_seg;
            if (p.bias[m]) v += p.bias[m][row];
            if constexpr (MODE == MODE_PEERS) store_to_peers(p, row, v);
            else y[row] = p.acc ? y[row] + v : v;
          }
        }
      }
    }
  }
  if (dead) {
    // copies issued after the one that never landed may still be in flight into this warp's stages: give each a
    // bounded time to land before the CTA's shared memory is released
    const int issued = __shfl_sync(0xffffffffu, n_issued, 0);
    for (int k = n_done + 1; k < issued; ++k)
      mbar_wait(&full[k % p.nstages], (uint32_t)(k / p.nstages) & 1u, nullptr, 0);
  }
  if constexpr (MODE == MODE_PEERS) {
    // every CTA takes a ticket once its stores are issued; the last one signals the peers and waits for theirs
    __syncthreads();
    __shared__ int last;
    if (tid == 0) last = take_ticket(&g_mv_ticket) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (last) {
      if (tid == 0) g_mv_ticket = 0;
      ep_meet(p.flag_peers, p.flags, p.world, p.rank, p.slot, p.epoch, true, p.wait_ns, p.status);
    }
  }
}

// ---- host side ----------------------------------------------------------------

static unsigned int* status_ptr() {
  static thread_local int cached_dev = -1;
  static thread_local unsigned int* cached = nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    cached = device_status_word();
    cached_dev = dev;
  }
  return cached;
}

// SMs of the current device (looked up once per device and thread).
static int sm_count() {
  static thread_local int cached_dev = -1, cached = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    int n = 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

static uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
static int unit_weights(int fmt) { return (fmt == ILL_Q8_0 || fmt == ILL_IQ2_XXS) ? 32 : 64; }

struct MvPlan {
  bool one;  // the one-token kernel (activations in registers)
  bool xs;   // ... rows staged in column chunks, the activations read from shared memory
  int warps; // warps per CTA
  int nchunks, chunk_units;
  uint32_t chunk_bytes;
  int rows_per_tile, lanes, nstages, upt, tps, slots, al;
  uint32_t stage_bytes, x_bytes, xs_off, bs_off, smem;
};

// Tile size: small matrices are cut into many tiles so every SM gets several;
// large ones use stages of at most STAGE_CAP bytes.
static long long tile_target(long long total_bytes, uint32_t cap) {
  long long t = total_bytes / ((long long)sm_count() * 16);
  if (t > cap) t = cap;
  if (t < 2048) t = 2048;
  return t;
}

// Overrides of the plan for sweeps: lanes a row, rows a warp tile, stages, CTAs per SM (0 = planned).  They
// exist only in builds made with -DILL_TUNING (an entry point ill_set_tuning sets them); the shipped library has
// no mutable plan state.
#ifdef ILL_TUNING
static int g_env_L = 0, g_env_TR = 0, g_env_NST = 0, g_env_CTAS = 0, g_env_XS = 0;
#else
constexpr int g_env_L = 0, g_env_TR = 0, g_env_NST = 0, g_env_CTAS = 0, g_env_XS = 0;
#endif

// Lanes that share a row (L) and units a lane keeps in registers (UPT) for rows of UNITS units; false when the
// row is too long for registers.  The order in which a row's partial sums are added follows from the pair, so
// every kernel that wants the one-token product's bits picks it here.
bool mv_pick_lanes(int fmt, int units, bool glu, bool big, int* L_out, int* upt_out) {
  const int uw = unit_weights(fmt);
  // Units a lane keeps in registers, at most.  More of them lets fewer lanes share a row with none idle (80 units:
  // 16 lanes x 5 instead of 32 x 3 with five lanes idle) at the price of registers, i.e. of resident warps.
  // Measured on 151936-row matrices and the 4B model's shapes: five pays for Q6_K rows, for the gated Q4_K product
  // and for large Q4_K matrices (BIG: past 16 MB), three for the rest -- Q2_K too, which is bound by instructions
  // and at five units (154 registers) keeps one CTA resident where three units keep two (81 us against 62 on
  // 151936 x 5120); Q8_0's 32-wide units go up to seven, four lanes a row.
  const int upt_max = fmt == ILL_Q8_0 ? 7 : uw == 32 ? 5 : (fmt == ILL_Q4_K && !glu) ? (big ? 5 : 3) : (fmt == ILL_Q6_K && !glu) || (fmt == ILL_Q4_K && glu) ? 5 : 3;
  int bestL = 0, bestU = 0;
  double best = -1.0;
  for (int L = 32; L >= (fmt == ILL_Q8_0 ? 4 : 8); L >>= 1) {
    const int upt = (units + L - 1) / L;
    if (upt > upt_max) continue;
    const double eff = (double)units / ((double)L * upt) + (L == 16 ? 0.02 : L == 32 ? 0.01 : 0.0);  // ties: 16, then 32
    if (eff > best) { best = eff; bestL = L; bestU = upt; }
  }
  // a row too long for that many units still beats staging it in column chunks if 32 lanes x 5 units hold it
  if (!bestL && uw == 64 && (units + 31) / 32 <= 5) { bestL = 32; bestU = (units + 31) / 32; }
  *L_out = bestL;
  *upt_out = bestU;
  return bestL != 0;
}

// One-token plan.  Whole rows: L lanes a row and UPT units a lane in registers,
// chosen for the fewest idle lanes; a warp's stage holds (32/L) * k rows, about
// 3 KB.  Rows too long for that (or FORCE_XS): 32 lanes a row, the row staged in
// column chunks of whole blocks, the activations in shared memory.
static int plan_one(int fmt, long long total_rows, int cols, int nseg, bool glu, MvPlan* pl) {
  const int bb = fmt_block_bytes(fmt), bw = fmt_block_weights(fmt), uw = unit_weights(fmt);
  const long long row_bytes = (long long)(cols / bw) * bb;
  const int units = cols / uw;
  const bool big = total_rows * row_bytes * nseg >= (16ll << 20);
  int bestL = 0, bestU = 0;
  if (!mv_pick_lanes(fmt, units, glu, big, &bestL, &bestU) || g_env_XS) bestL = 0;
  if (g_env_L && (units + g_env_L - 1) / g_env_L <= 7) { bestL = g_env_L; bestU = (units + g_env_L - 1) / g_env_L; }
  pl->one = true;
  pl->xs = false;
  pl->nchunks = 1;
  pl->chunk_units = units;
  pl->chunk_bytes = (uint32_t)row_bytes;
  long long tr;
  if (!bestL) {
    // blocks per chunk: a multiple that makes the chunk's units a multiple of 32, near 3 KB
    const int upb = bw / uw;                  // units per block
    int bpc = 32 / upb > 0 ? 32 / upb : 1;    // 32 units
    while ((long long)bpc * 2 * bb <= 3400 && bpc * 2 * upb <= 128) bpc *= 2;
    const int blocks = cols / bw;
    if (bpc > blocks) bpc = blocks;
    pl->xs = true;
    pl->nchunks = (blocks + bpc - 1) / bpc;
    pl->chunk_units = bpc * upb;
    pl->chunk_bytes = (uint32_t)bpc * bb;
    bestL = 32;
    bestU = (pl->chunk_units + 31) / 32;
    if (bestU > 4) return ILL_ERR_UNSUPPORTED;
    tr = 1;
  } else {
    const int nsub = 32 / bestL;
    // rows per warp tile: about 3 KB a stage (small stages keep more CTAs resident, which is what
    // hides the copy latency), and small matrices are cut finer so that every warp gets some
    const long long warps = (long long)sm_count() * 16;
    // (Q2_K is bound by instructions, not by HBM: twice the stage halves what a tile costs it in waits, address
    // arithmetic and copies issued; IQ2_XXS, with 48 KB of tables a CTA, does better with two small CTAs resident)
    tr = (fmt == ILL_Q2_K ? 6144 : 3072) / row_bytes;
    const long long share = (total_rows * nseg + warps - 1) / warps;
    if (tr > share) tr = share;
    if (g_env_TR) tr = g_env_TR;
    tr = tr / nsub * nsub;
    if (tr < nsub) tr = nsub;
    if (glu && tr > (long long)MV_MAXRI * nsub) tr = (long long)MV_MAXRI * nsub;
  }
  pl->warps = MV_THREADS / 32;
  {  // few groups: smaller CTAs, so that the warps spread over every SM
    const long long groups = (total_rows * nseg + tr - 1) / tr;
    while (pl->warps > 1 && groups < (long long)sm_count() * 2 * pl->warps) pl->warps >>= 1;
  }
  pl->upt = bestU;
  pl->lanes = bestL;
  pl->rows_per_tile = (int)tr;
  pl->stage_bytes = align_up((pl->xs ? pl->chunk_bytes : (uint32_t)(tr * row_bytes)) + 32, 128);
  pl->x_bytes = pl->xs_off = pl->bs_off = 0;
  if (pl->xs) {
    const int nsc = fmt == ILL_Q8_0 ? cols / 32 : cols / 256;
    switch (fmt) {
      case ILL_Q8_0: pl->x_bytes = plane_bytes<ILL_Q8_0>(units, nsc); break;
      case ILL_Q4_K: pl->x_bytes = plane_bytes<ILL_Q4_K>(units, nsc); break;
      case ILL_Q6_K: pl->x_bytes = plane_bytes<ILL_Q6_K>(units, nsc); break;
      case ILL_Q2_K: pl->x_bytes = plane_bytes<ILL_Q2_K>(units, nsc); break;
      default: pl->x_bytes = plane_bytes<ILL_IQ2_XXS>(units, nsc); break;
    }
  }
  // stages: four if two CTAs still fit an SM, else three or two with two CTAs, else three or two with one
  const uint32_t fixed = (fmt == ILL_IQ2_XXS ? IQ_TABLE_BYTES : 0) + 8 * 8 * pl->warps + pl->x_bytes + 64 + 1024;
  const uint32_t per_stage = pl->stage_bytes * pl->warps;
  const uint32_t two = 113 * 1024;  // half an SM's shared memory
  // (plain products: two CTAs with two stages each beat one CTA with three, residency hides more latency than
  // depth; a gated product's group is two stages, so it needs the third to fetch ahead at all)
  pl->nstages = per_stage * 4 + fixed <= two ? 4 : per_stage * 3 + fixed <= two ? 3 : (!glu && per_stage * 2 + fixed <= two) ? 2
                : per_stage * 3 + fixed <= 200 * 1024 ? 3 : 2;
  if (g_env_NST) pl->nstages = g_env_NST;
  pl->smem = pl->stage_bytes * pl->nstages * pl->warps + (fmt == ILL_IQ2_XXS ? IQ_TABLE_BYTES : 0) + 8 * pl->nstages * pl->warps +
             pl->x_bytes + 64;
  return pl->smem > 220 * 1024 ? ILL_ERR_UNSUPPORTED : ILL_OK;
}

static int plan_many(int fmt, long long total_rows, int cols, int ntok, int nseg, MvPlan* pl) {
  const long long row_bytes = (long long)(cols / fmt_block_weights(fmt)) * fmt_block_bytes(fmt);
  if (row_bytes + 32 > 49152) return ILL_ERR_UNSUPPORTED;
  long long rpt = tile_target(total_rows * row_bytes * nseg, 16384) / row_bytes;
  if (rpt < 1) rpt = 1;
  if (rpt > total_rows) rpt = total_rows;
  pl->one = false;
  pl->xs = false;
  pl->warps = MV_THREADS / 32;
  pl->upt = 0;
  pl->nchunks = 1;
  pl->chunk_units = 0;
  pl->chunk_bytes = 0;
  pl->al = 1;
  pl->rows_per_tile = (int)rpt;
  pl->stage_bytes = align_up((uint32_t)(rpt * row_bytes) + 32, 128);
  pl->nstages = 4;
  const int units = cols / unit_weights(fmt);
  int L = 32;
  while (L > 1 && (L / 2) * rpt >= MV_THREADS) L >>= 1;  // enough rows to fill the CTA with fewer lanes a row
  while (L > 1 && L / 2 >= units) L >>= 1;
  pl->lanes = L;
  const int nsc = fmt == ILL_Q8_0 ? cols / 32 : cols / 256;
  pl->xs_off = align_up((uint32_t)ntok * cols, 16);
  pl->bs_off = align_up(pl->xs_off + 4u * ntok * nsc, 16);
  pl->x_bytes = align_up(pl->bs_off + 2u * ntok * (cols / 16), 128);
  pl->smem = pl->x_bytes + pl->stage_bytes * pl->nstages + (fmt == ILL_IQ2_XXS ? IQ_TABLE_BYTES : 0) + 64;
  return pl->smem > 227 * 1024 ? ILL_ERR_UNSUPPORTED : ILL_OK;
}

template <typename K>
static int launch_k(K k, const MvParams& p, const MvPlan& pl, int gx, int gy, cudaStream_t st) {
  if (pl.smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  MvParams pp = p;
  void* args[] = {&pp};
  return launch_kernel((const void*)k, dim3(gx, gy, 1), dim3(32 * pl.warps, 1, 1), pl.smem, args, st);
}

template <int FMT, int MODE, int AL>
static int launch_one_u(const MvParams& p, const MvPlan& pl, int gx, int gy, cudaStream_t st) {
  constexpr int UMAX = 5;
  if (pl.xs) {
    if constexpr (MODE != MODE_PEERS) {
      switch (pl.upt) {
        case 1: return launch_k(mvw_kernel<FMT, MODE, 1, AL, true>, p, pl, gx, gy, st);
        case 2: return launch_k(mvw_kernel<FMT, MODE, 2, AL, true>, p, pl, gx, gy, st);
        case 3: return launch_k(mvw_kernel<FMT, MODE, 3, AL, true>, p, pl, gx, gy, st);
        case 4: return launch_k(mvw_kernel<FMT, MODE, 4, AL, true>, p, pl, gx, gy, st);
      }
    }
    return ILL_ERR_UNSUPPORTED;
  }
  switch (pl.upt) {
    case 1: return launch_k(mvw_kernel<FMT, MODE, 1, AL, false>, p, pl, gx, gy, st);
    case 2: return launch_k(mvw_kernel<FMT, MODE, 2, AL, false>, p, pl, gx, gy, st);
    case 3: return launch_k(mvw_kernel<FMT, MODE, 3, AL, false>, p, pl, gx, gy, st);
    case 4: if constexpr (UMAX >= 4) return launch_k(mvw_kernel<FMT, MODE, 4, AL, false>, p, pl, gx, gy, st); break;
    case 5: if constexpr (UMAX >= 5) return launch_k(mvw_kernel<FMT, MODE, 5, AL, false>, p, pl, gx, gy, st); break;
    case 6: if constexpr (FMT == ILL_Q8_0) return launch_k(mvw_kernel<FMT, MODE, 6, AL, false>, p, pl, gx, gy, st); break;
    case 7: if constexpr (FMT == ILL_Q8_0) return launch_k(mvw_kernel<FMT, MODE, 7, AL, false>, p, pl, gx, gy, st); break;
  }
  return ILL_ERR_UNSUPPORTED;
}

template <int FMT, int MODE>
static int launch_one_a(const MvParams& p, const MvPlan& pl, int gx, int gy, cudaStream_t st) {
  if constexpr (FMT == ILL_Q4_K) {
    if (pl.al >= 16) return launch_one_u<FMT, MODE, 16>(p, pl, gx, gy, st);
  }
  if constexpr (FMT == ILL_Q2_K) {
    if (pl.al >= 4) return launch_one_u<FMT, MODE, 4>(p, pl, gx, gy, st);
  }
  return launch_one_u<FMT, MODE, 1>(p, pl, gx, gy, st);
}

template <int FMT>
static int launch_fmt(int mode, const MvParams& p, const MvPlan& pl, int gx, int gy, cudaStream_t st) {
  if (pl.one) {
    if (mode == MODE_GLU) return launch_one_a<FMT, MODE_GLU>(p, pl, gx, gy, st);
    if (mode == MODE_MOE_GLU) {
      if constexpr (FMT == ILL_IQ2_XXS || FMT == ILL_Q2_K) return launch_one_a<FMT, MODE_MOE_GLU>(p, pl, gx, gy, st);
      return ILL_ERR_UNSUPPORTED;
    }
    if (mode == MODE_PEERS) return pl.xs ? ILL_ERR_UNSUPPORTED : launch_one_a<FMT, MODE_PEERS>(p, pl, gx, gy, st);
    return launch_one_a<FMT, MODE_PLAIN>(p, pl, gx, gy, st);
  }
  if (mode != MODE_PLAIN) return ILL_ERR_UNSUPPORTED;
  if (p.n == 1) return launch_k(mvn_kernel<FMT, MODE_PLAIN, 1>, p, pl, gx, gy, st);
  if (p.n <= 4) return launch_k(mvn_kernel<FMT, MODE_PLAIN, 4>, p, pl, gx, gy, st);
  if (p.n <= 8) return launch_k(mvn_kernel<FMT, MODE_PLAIN, 8>, p, pl, gx, gy, st);
  return launch_k(mvn_kernel<FMT, MODE_PLAIN, 16>, p, pl, gx, gy, st);
}

static int launch_mv(int fmt, int mode, const MvParams& p, const MvPlan& pl, int gx, int gy, cudaStream_t st) {
  switch (fmt) {
    case ILL_Q8_0: return launch_fmt<ILL_Q8_0>(mode, p, pl, gx, gy, st);
    case ILL_Q4_K: return launch_fmt<ILL_Q4_K>(mode, p, pl, gx, gy, st);
    case ILL_Q6_K: return launch_fmt<ILL_Q6_K>(mode, p, pl, gx, gy, st);
    case ILL_Q2_K: return launch_fmt<ILL_Q2_K>(mode, p, pl, gx, gy, st);
    case ILL_IQ2_XXS: return launch_fmt<ILL_IQ2_XXS>(mode, p, pl, gx, gy, st);
  }
  return ILL_ERR_ARG;
}

static bool needs_bsums(int fmt) { return fmt == ILL_Q4_K || fmt == ILL_Q6_K || fmt == ILL_Q2_K; }

// Common entry: NMAT matrices of one format sharing the activations, NSEG
// segments (experts) of them.
// What ill_mv_peers asks of the one-token kernel on top of the product (set around its call of mv_common).
struct MvPeer {
  ill_dptr y_peers, flag_peers, flags;
  long long y_off;
  int world, rank, slot;
  unsigned epoch;
  unsigned long long wait_ns;
};
static thread_local const MvPeer* t_peer = nullptr;

int mv_common(int fmt, int mode, int nmat, const ill_dptr* w, const int* rows, int cols, ill_dptr xq, ill_dptr xs,
              ill_dptr xsum, const ill_dptr* y, const ill_dptr* bias, int acc, int n, ill_dptr ptrs, int nseg,
              long long add, long long up_add, int x_seg, long long y_seg, ill_dptr seg_w, float clamp,
              ill_stream stream) {
  const int bw = fmt_block_weights(fmt);
  if (!bw || nmat < 1 || nmat > MV_MAX_MATS || cols <= 0 || cols % (bw == 32 ? 32 : 256)) return ILL_ERR_ARG;
  if (n < 1 || nseg < 1 || nseg > 65535) return ILL_ERR_ARG;
  if (!xq || !xs || (needs_bsums(fmt) && !xsum)) return ILL_ERR_ARG;
  if (xq & 15 || xs & 3 || xsum & 7) return ILL_ERR_ALIGN;
  long long total_rows = 0;
  uint64_t align_bits = (uint64_t)add | (uint64_t)up_add;
  for (int i = 0; i < nmat; ++i) {
    if (rows[i] <= 0 || !y[i] || (!ptrs && !w[i])) return ILL_ERR_ARG;
    if (y[i] & 3) return ILL_ERR_ALIGN;
    total_rows += rows[i];
    if (!ptrs) align_bits |= w[i];
  }
  const bool glu = mode == MODE_GLU || mode == MODE_MOE_GLU;
  if ((glu || mode == MODE_PEERS) && n != 1) return ILL_ERR_ARG;
  if (n >= 2 && !glu && nmat == 1 && !ptrs && !x_seg) {
    // several tokens: the tensor cores' int8 path where it is written (Q8_0, Q4_K, Q6_K; up to 16 tokens with the
    // activations resident, chunks with them streamed), else the token loop below
    int rc_t = ILL_ERR_UNSUPPORTED;
    if (n <= 16) rc_t = mvt_try(fmt, w[0], rows[0], cols, xq, xs, xsum, y[0], bias ? bias[0] : 0, acc, n, stream);
    // a few tokens of rows too long for their activations to stay in shared memory
    if (rc_t == ILL_ERR_UNSUPPORTED && n <= 16) rc_t = mmk_try(fmt, w[0], rows[0], cols, xq, xs, xsum, y[0], bias ? bias[0] : 0, acc, n, stream);
    // a chunk
    if (rc_t == ILL_ERR_UNSUPPORTED) rc_t = mmd_try(fmt, w[0], rows[0], cols, xq, xs, xsum, y[0], bias ? bias[0] : 0, acc, n, stream);
    if (rc_t != ILL_ERR_UNSUPPORTED) return rc_t;
  }
  if (n > MV_MAX_TOK) return ILL_ERR_UNSUPPORTED;  // the token loop below takes 16 at most: the caller splits the chunk
  MvPlan pl;
  int rc = ILL_ERR_UNSUPPORTED;
  if (n == 1) rc = plan_one(fmt, glu ? rows[0] : total_rows, cols, nseg, glu, &pl);
  if (rc == ILL_ERR_UNSUPPORTED && !glu && !t_peer) rc = plan_many(fmt, total_rows, cols, x_seg ? 1 : n, nseg, &pl);
  if (rc) return rc;
  pl.al = (align_bits & 15) == 0 ? 16 : (align_bits & 3) == 0 ? 4 : 1;
  MvParams p = {};
  p.nmat = glu ? 1 : nmat;
  int tiles = 0;
  for (int i = 0; i < MV_MAX_MATS; ++i) {
    p.w[i] = i < nmat ? (const u8*)(uintptr_t)w[i] : nullptr;
    p.y[i] = i < nmat ? (float*)(uintptr_t)y[i] : nullptr;
    p.bias[i] = (i < nmat && bias) ? (const float*)(uintptr_t)bias[i] : nullptr;
    p.rows[i] = i < nmat ? rows[i] : 0;
    p.tile0[i] = tiles;
    if (i < p.nmat) tiles += (rows[i] + pl.rows_per_tile - 1) / pl.rows_per_tile;
  }
  p.tile0[p.nmat] = tiles;
  for (int i = p.nmat + 1; i <= MV_MAX_MATS; ++i) p.tile0[i] = tiles;
  p.cols = cols;
  p.row_bytes = cols / bw * fmt_block_bytes(fmt);
  p.units = cols / unit_weights(fmt);
  p.xq = (const i8*)(uintptr_t)xq;
  p.xs = (const float*)(uintptr_t)xs;
  p.xsum = (const int16_t*)(uintptr_t)xsum;
  p.n = n;
  p.acc = acc;
  p.rows_per_tile = pl.rows_per_tile;
  p.lanes_per_row = pl.lanes;
  p.nchunks = pl.nchunks;
  p.chunk_units = pl.chunk_units;
  p.chunk_bytes = pl.chunk_bytes;
  p.stage_bytes = pl.stage_bytes;
  p.nstages = pl.nstages;
  p.x_bytes = pl.x_bytes;
  p.xs_off = pl.xs_off;
  p.bs_off = pl.bs_off;
  p.ptrs = (const unsigned long long*)(uintptr_t)ptrs;
  p.add = add;
  p.up_add = up_add;
  p.x_seg = x_seg;
  p.y_seg = y_seg;
  p.seg_w = (const float*)(uintptr_t)seg_w;
  p.clamp = clamp;
  p.status = status_ptr();
  if (t_peer) {
    p.y_peers = (const unsigned long long*)(uintptr_t)t_peer->y_peers;
    p.y_peer_off = t_peer->y_off;
    p.flag_peers = (const unsigned long long*)(uintptr_t)t_peer->flag_peers;
    p.flags = (unsigned*)(uintptr_t)t_peer->flags;
    p.world = t_peer->world;
    p.rank = t_peer->rank;
    p.slot = t_peer->slot;
    p.epoch = t_peer->epoch;
    p.wait_ns = t_peer->wait_ns;
  }
  // persistent grid: as many CTAs as can be resident, split over the segments
  int per_sm = (int)((227u * 1024u) / (pl.smem + 1024u));
  const int per_sm_cap = pl.one ? 16 / pl.warps * 2 : 6;  // up to 32 warps an SM
  per_sm = per_sm < 1 ? 1 : (per_sm > per_sm_cap ? per_sm_cap : per_sm);
  if (g_env_CTAS) per_sm = g_env_CTAS;
  int gx = (sm_count() * per_sm + nseg - 1) / nseg;
  const int work = pl.one ? (tiles + pl.warps - 1) / pl.warps : tiles;  // a warp a tile, or a CTA a tile
  if (gx > work) gx = work;
  if (gx < 1) gx = 1;
  return launch_mv(fmt, mode, p, pl, gx, nseg, (cudaStream_t)stream);
}

}  // namespace ill

using namespace ill;

#ifdef ILL_TUNING
extern "C" __attribute__((visibility("default"))) int ill_set_tuning(int lanes, int tile_rows, int stages, int ctas_per_sm) {
  g_env_XS = 0;
  if (lanes == 1) { g_env_XS = 1; lanes = 0; }  // 1: stage rows in column chunks whatever their length
  if (lanes && lanes != 8 && lanes != 16 && lanes != 32) return ILL_ERR_ARG;
  if (tile_rows < 0 || stages < 0 || stages > 8 || ctas_per_sm < 0 || ctas_per_sm > 16) return ILL_ERR_ARG;
  g_env_L = lanes;
  g_env_TR = tile_rows;
  g_env_NST = stages;
  g_env_CTAS = ctas_per_sm;
  return ILL_OK;
}
#endif

extern "C" int ill_mv(int fmt, ill_dptr w, int rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr y,
                      ill_dptr bias, int acc, int n, ill_stream stream) {
  const ill_dptr ws[1] = {w}, ys[1] = {y}, bs[1] = {bias};
  const int rs[1] = {rows};
  return mv_common(fmt, MODE_PLAIN, 1, ws, rs, cols, xq, xs, xsum, ys, bs, acc, n, 0, 1, 0, 0, 0, 0, 0, 0.0f, stream);
}

extern "C" int ill_mv_peers(int fmt, ill_dptr w, int rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr y_peers,
                            int64_t y_off, ill_dptr bias, ill_dptr flag_peers, ill_dptr flags, int world, int rank, int slot,
                            uint32_t epoch, int64_t wait_ns, ill_stream stream) {
  if (!y_peers || y_off < 0 || !flag_peers || !flags || world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || slot < 0 ||
      slot >= EP_FLAG_SLOTS || wait_ns < 0)
    return ILL_ERR_ARG;
  if ((y_peers & 7) || (flag_peers & 7) || (flags & 3)) return ILL_ERR_ALIGN;
  const MvPeer peer = {y_peers, flag_peers, flags, (long long)y_off, world, rank, slot, epoch, (unsigned long long)wait_ns};
  const ill_dptr ws[1] = {w}, ys[1] = {flags /* stands for Y in the checks: the kernel stores through Y_PEERS */}, bs[1] = {bias};
  const int rs[1] = {rows};
  t_peer = &peer;
  const int rc = mv_common(fmt, MODE_PEERS, 1, ws, rs, cols, xq, xs, xsum, ys, bs, 0, 1, 0, 1, 0, 0, 0, 0, 0, 0.0f, stream);
  t_peer = nullptr;
  return rc;
}

extern "C" int ill_mv_3(int fmt, ill_dptr w0, ill_dptr w1, ill_dptr w2, int rows0, int rows1, int rows2, int cols,
                        ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr y0, ill_dptr y1, ill_dptr y2, ill_dptr b0,
                        ill_dptr b1, ill_dptr b2, ill_stream stream) {
  const ill_dptr ws[3] = {w0, w1, w2}, ys[3] = {y0, y1, y2}, bs[3] = {b0, b1, b2};
  const int rs[3] = {rows0, rows1, rows2};
  const int nmat = (rows2 == 0 && !w2) ? 2 : 3;
  return mv_common(fmt, MODE_PLAIN, nmat, ws, rs, cols, xq, xs, xsum, ys, bs, 0, 1, 0, 1, 0, 0, 0, 0, 0, 0.0f, stream);
}

extern "C" int ill_mv_glu(int fmt, ill_dptr wg, ill_dptr wu, int rows, int cols, ill_dptr xq, ill_dptr xs,
                          ill_dptr xsum, ill_dptr y, ill_stream stream) {
  const ill_dptr ws[2] = {wg, wu}, ys[2] = {y, y};
  const int rs[2] = {rows, rows};
  if (!wu) return ILL_ERR_ARG;
  return mv_common(fmt, MODE_GLU, 2, ws, rs, cols, xq, xs, xsum, ys, nullptr, 0, 1, 0, 1, 0, 0, 0, 0, 0, 0.0f, stream);
}
