// mm_id.cu -- the routed experts' product for a chunk of tokens, on the 5th-generation
// tensor cores (tcgen05, accumulators in tensor memory).
//
//   Y[place, n] = sum_k X[place, k] * W_e[n, k]      for every expert e and every row
//                                                    `place` in [bases[e], bases[e] + counts[e])
//
// X is the chunk's activations already grouped by expert (ill_moe_group), as fp16
// (ill_act_f16: the Q8_K quants times their block scale, i.e. exactly the values the
// reference's CPU kernels multiply, rounded once to fp16).  W_e is expert e's matrix
// of raw IQ2_XXS or Q2_K blocks at ptrs[e] + add.
//
// One CTA computes a 128 (rows of X) x 128 (rows of W_e) tile, K in steps of 64:
//   warp 0      one lane issues the TMA loads of the X tile (128-byte swizzle)
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128x128x16, fp16 in,
//               fp32 accumulate) and commits each stage back to the producers
//   warps 2-5   dequantize W_e's blocks straight into the swizzled shared-memory operand
//               tile (one weight row per thread), then read the accumulators back
//               (tcgen05.ld) and store the tile's valid rows
// Every mbarrier wait is bounded; on a time-out the kernel records a code in the status
// word, skips what depends on the wait, frees its tensor memory and returns.
//
// Replaces d4_mm_id_iq2_xxs / d4_mm_id_q2_k (src/cuda/ds4f_mm.cu:229-257: mma.sync
// m16n8k16, 64x64 tiles) behind DK-FFN-ROUTED-CHUNK (src/cuda-ds4f-prefill.lisp:315-356).
#include <cuda.h>

#include "formats.cuh"
#include "iq2xxs_tables.cuh"
#include "host.h"

namespace ill {

constexpr int MM_BM = 128, MM_BN = 128, MM_BK = 64, MM_STAGES = 3;  // 3 stages: two CTAs fit an SM
constexpr int MM_THREADS = 192;
constexpr uint32_t MM_TILE_BYTES = MM_BM * MM_BK * 2;  // 16 KB, A or B
constexpr uint32_t MM_TMEM_COLS = 128;

struct MmParams {
  int ncols, nrows;            // K and N of every expert matrix
  int row_bytes;
  long long add;
  const unsigned long long* ptrs;
  const unsigned* counts;
  const unsigned* bases;
  float* y;
  long long y_stride;          // floats between rows of Y
  int ne;
  int max_mtiles;
  unsigned int* status;
};

// ---- tcgen05 / TMA wrappers ---------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, 128 x 128 x 16, fp16 operands, fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// arrive on BAR once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
  const uint64_t addr = (uint64_t)(smem_u32(tile) >> 4) & 0x3fffu;
  return addr | (1ull << 16) /* leading offset: 16 B, unused with a swizzle */ | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) /* descriptor version of sm_100 */ | (2ull << 61) /* SWIZZLE_128B */;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *(const uint32_t*)&h;
}

// ---- dequantization of 64 weights of one row into the swizzled B tile ----------------
// ROW is the thread's weight row (0..127) in the tile; the 64 weights are 8 chunks of 8
// halves; chunk c goes to 16-byte slot c ^ (row % 8) of the row's 128 bytes.
__device__ __forceinline__ void store_chunk(u8* tile, int row, int c, uint4 v) {
  *(uint4*)(tile + (row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4)) = v;
}

// words [first, first+N) of the block at P (any 2-byte alignment), from global memory
template <int N>
__device__ __forceinline__ void ldg_words(const u8* p, uint32_t (&out)[N]) {
  const uint32_t mis = (uint32_t)(uintptr_t)p & 3u;
  const uint32_t* b = (const uint32_t*)(p - mis);
  const uint32_t sh = mis * 8u;
  uint32_t prev = __ldg(b);
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const uint32_t next = __ldg(b + i + 1);
    out[i] = __funnelshift_r(prev, next, sh);
    prev = next;
  }
}

// IQ2_XXS: K step KS (0..3) of the block at BLK: sub-blocks 2*ks, 2*ks+1.  Values as
// IQ2XXS-ROW-FLOATS! computes them (src/iquant.lisp:161-175), then rounded to fp16.
__device__ __forceinline__ void dequant64_iq2xxs(const u8* blk, int ks, u8* tile, int row, const uint2* grid,
                                                 const u8* signs) {
  uint32_t v[4];
  ldg_words<4>(blk + 2 + 16 * ks, v);
  const float d = h2f((uint32_t)__ldg((const u16*)blk));
#pragma unroll
  for (int sb = 0; sb < 2; ++sb) {
    const uint32_t idx = v[2 * sb], aux = v[2 * sb + 1];
    const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(aux >> 28))), 0.25f);
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint2 g = grid[(idx >> (8 * l)) & 0xff];
      const uint32_t s = signs[(aux >> (7 * l)) & 127];
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float mag = (float)(((j < 4 ? g.x : g.y) >> (8 * (j & 3))) & 0xff);
        f[j] = __fmul_rn(db, mag);
        if ((s >> j) & 1) f[j] = -f[j];
      }
      store_chunk(tile, row, 4 * sb + l,
                  make_uint4(pack_h2(f[0], f[1]), pack_h2(f[2], f[3]), pack_h2(f[4], f[5]), pack_h2(f[6], f[7])));
    }
  }
}

// Q2_K: K step KS of the block at BLK: weights 64*ks .. 64*ks+63 = half h = ks/2, shifts
// k = 2*(ks%2), 2*(ks%2)+1.  Values as Q2K-ROW-FLOATS! (src/iquant.lisp:217-230), to fp16.
__device__ __forceinline__ void dequant64_q2k(const u8* blk, int ks, u8* tile, int row) {
  const int h = ks >> 1, k0 = 2 * (ks & 1);
  const uint32_t* q32 = (const uint32_t*)(blk + 16 + 32 * h);  // 32 bytes of quants, 4-byte aligned
  uint32_t q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = __ldg(q32 + i);
  const uint32_t dd = __ldg((const uint32_t*)(blk + 80));
  const float d = h2f(dd & 0xffff), dmin = h2f(dd >> 16);
  const uint32_t sc4 = __ldg((const uint32_t*)(blk + 8 * h + 4 * (ks & 1)));  // scale bytes 8h + 2k + half, k = k0, k0+1
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t sb = (sc4 >> (8 * (2 * kk + half))) & 0xff;
      const float dl = __fmul_rn(d, (float)(sb & 15)), ml = __fmul_rn(dmin, (float)(sb >> 4));
      // 16 weights: bytes 16*half .. 16*half+15 of the 32, shifted by 2*(k0+kk)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int byte = 16 * half + 8 * c + j;
          const uint32_t qv = (q[byte >> 2] >> (8 * (byte & 3) + 2 * (k0 + kk))) & 3u;
          f[j] = __fsub_rn(__fmul_rn(dl, (float)qv), ml);
        }
        store_chunk(tile, row, 4 * kk + 2 * half + c,
                    make_uint4(pack_h2(f[0], f[1]), pack_h2(f[2], f[3]), pack_h2(f[4], f[5]), pack_h2(f[6], f[7])));
      }
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(MM_THREADS) mm_id_kernel(const __grid_constant__ CUtensorMap xmap, const MmParams p) {
  extern __shared__ __align__(1024) u8 smem_raw[];
  // [A stages][B stages] (each tile 1024-byte aligned, as the 128-byte swizzle needs), then barriers, tables
  u8* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  u8* a_tiles = smem;
  u8* b_tiles = smem + MM_STAGES * MM_TILE_BYTES;
  u8* tail = smem + 2 * MM_STAGES * MM_TILE_BYTES;
  uint64_t* full_a = (uint64_t*)tail;            // TMA bytes landed
  uint64_t* full_b = full_a + MM_STAGES;         // 4 dequant warps arrived
  uint64_t* empty = full_b + MM_STAGES;          // the MMAs that read the stage completed
  uint64_t* acc_full = empty + MM_STAGES;        // all MMAs of the tile completed
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  int* tile_info = (int*)(tmem_slot + 1);        // expert, row0, nrows valid
  uint2* iq_grid = (uint2*)(tail + 256);
  u8* iq_signs = (u8*)(iq_grid + 256);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt = blockIdx.x;   // tile along the weights' rows
  const int mt = blockIdx.y;   // running index of 128-row tiles over all experts

  // which expert does this row tile belong to?  (warp 0 scans the counts)
  if (warp == 0) {
    int before = 0, found = -1, row0 = 0, nvalid = 0;
    for (int e0 = 0; e0 < p.ne && found < 0; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < p.ne ? (int)p.counts[e] : 0;
      const int tiles = (c + MM_BM - 1) / MM_BM;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int excl = before + incl - tiles;
      const bool mine = mt >= excl && mt < excl + tiles;
      const unsigned who = __ballot_sync(0xffffffffu, mine);
      if (who) {
        const int src = __ffs(who) - 1;
        found = __shfl_sync(0xffffffffu, e, src);
        const int m_in = mt - __shfl_sync(0xffffffffu, excl, src);
        const int cnt = __shfl_sync(0xffffffffu, c, src);
        row0 = (int)p.bases[found] + m_in * MM_BM;
        nvalid = min(MM_BM, cnt - m_in * MM_BM);
      }
      before += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) { tile_info[0] = found; tile_info[1] = row0; tile_info[2] = nvalid; }
  }
  if (tid == 32) {
    for (int s = 0; s < MM_STAGES; ++s) { mbar_init(&full_a[s], 1); mbar_init(&full_b[s], 4); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (FMT == ILL_IQ2_XXS) {
    for (int i = tid; i < 256; i += MM_THREADS) {
      const uint64_t g = ill_iq2xxs_grid[i];
      iq_grid[i] = make_uint2((uint32_t)g, (uint32_t)(g >> 32));
    }
    for (int i = tid; i < 128; i += MM_THREADS) iq_signs[i] = ill_ksigns_iq2xs[i];
  }
  __syncthreads();
  const int expert = tile_info[0], row0 = tile_info[1], nvalid = tile_info[2];
  if (expert < 0) return;  // past the last row tile: nothing allocated, nothing in flight
  if (warp == 1) tmem_alloc(tmem_slot, MM_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int ksteps = p.ncols / MM_BK;
  const u8* wexp = (const u8*)(uintptr_t)p.ptrs[expert] + p.add;
  bool ok = true;

  if (warp == 0) {
    // ---- TMA producer of the X tile
    if (lane == 0) {
      for (int ks = 0; ks < ksteps; ++ks) {
        const int s = ks % MM_STAGES, use = ks / MM_STAGES;
        if (use > 0 && !mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(&full_a[s], MM_TILE_BYTES);
        tma_load_2d(a_tiles + s * MM_TILE_BYTES, &xmap, ks * MM_BK, row0, &full_a[s]);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      // fp32 accumulate, fp16 A and B, both K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(MM_BN >> 3) << 17) | ((uint32_t)(MM_BM >> 4) << 24);
      for (int ks = 0; ks < ksteps; ++ks) {
        const int s = ks % MM_STAGES;
        const uint32_t par = (uint32_t)(ks / MM_STAGES) & 1u;
        if (!mbar_wait(&full_a[s], par, p.status, ST_MM_WAIT_FULL) ||
            !mbar_wait(&full_b[s], par, p.status, ST_MM_WAIT_FULL + 1)) { ok = false; break; }
        tc_fence_after();
        const uint64_t ad = umma_desc(a_tiles + s * MM_TILE_BYTES), bd = umma_desc(b_tiles + s * MM_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < MM_BK / 16; ++k)  // 32 bytes further along K inside the swizzle atom each time
          umma_f16(tmem_base, ad + 2 * k, bd + 2 * k, idesc, (ks | k) ? 1u : 0u);
        umma_commit(&empty[s]);  // frees the stage when these MMAs are done
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ---- dequantizing producers of the W tile (warps 2..5), then the epilogue
    const int row = (warp - 2) * 32 + lane;        // weight row in the tile
    const int n = nt * MM_BN + row;
    const bool has_row = n < p.nrows;
    const u8* wrow = wexp + (long long)(has_row ? n : 0) * p.row_bytes;
    constexpr int BB = FMT == ILL_IQ2_XXS ? 66 : 84;
    for (int ks = 0; ks < ksteps; ++ks) {
      const int s = ks % MM_STAGES, use = ks / MM_STAGES;
      if (use > 0) {
        bool w_ok = mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 1);
        w_ok = __all_sync(0xffffffffu, w_ok);
        if (!w_ok) { ok = false; break; }
      }
      u8* tile = b_tiles + s * MM_TILE_BYTES;
      const u8* blk = wrow + (ks >> 2) * BB;
      if (has_row) {
        if constexpr (FMT == ILL_IQ2_XXS) dequant64_iq2xxs(blk, ks & 3, tile, row, iq_grid, iq_signs);
        else dequant64_q2k(blk, ks & 3, tile, row);
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) store_chunk(tile, row, c, make_uint4(0, 0, 0, 0));
      }
      fence_async_smem();  // the tensor core reads the tile through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_b[s]);
    }
    // ---- epilogue: this warp reads the 32 accumulator rows it may access
    if (ok) {
      bool e_ok = mbar_wait(acc_full, 0, p.status, ST_MM_WAIT_ACC);
      e_ok = __all_sync(0xffffffffu, e_ok);
      if (e_ok) {
        tc_fence_after();
        const int q = warp & 3;                   // TMEM lanes 32q .. 32q+31
        const int r = q * 32 + lane;              // row of the tile
        float* yrow = p.y + (long long)(row0 + r) * p.y_stride + (long long)nt * MM_BN;
#pragma unroll 1
        for (int c0 = 0; c0 < MM_BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
          if (r < nvalid) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (nt * MM_BN + c0 + j + 3 < p.nrows) {
                *(float4*)(yrow + c0 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                        __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              } else {
                for (int jj = 0; jj < 4; ++jj)
                  if (nt * MM_BN + c0 + j + jj < p.nrows) yrow[c0 + j + jj] = __uint_as_float(v[j + jj]);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, MM_TMEM_COLS);
}

// X (tokens' Q8_K quants) -> fp16 rows in expert order: XH[place, k] = fp16(q[t, k] * d[t, k/256]),
// t = MAP[place] (or place when MAP is null).
__global__ void __launch_bounds__(256) act_f16_kernel(long long rows, int cols, const i8* __restrict__ xq,
                                                      const float* __restrict__ xd, const unsigned* __restrict__ map,
                                                      __half* __restrict__ xh) {
  pdl_launch_dependents();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread: 16 values
  const int per_row = cols / 16;
  if (gid >= rows * per_row) return;
  const long long place = gid / per_row;
  const int j = (int)(gid - place * per_row);
  const long long t = map ? (long long)map[place] : place;
  const uint4 q = *(const uint4*)(xq + t * cols + 16 * j);
  const float d = xd[t * (cols / 256) + (16 * j) / 256];
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int b0 = (int)(signed char)((w[i >> 1] >> (16 * (i & 1))) & 0xff);
    const int b1 = (int)(signed char)((w[i >> 1] >> (16 * (i & 1) + 8)) & 0xff);
    h[i] = pack_h2(__fmul_rn((float)b0, d), __fmul_rn((float)b1, d));
  }
  uint4* dst = (uint4*)(xh + place * cols + 16 * j);
  dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
  dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

}  // namespace ill

using namespace ill;

extern "C" int ill_act_f16(int64_t rows, int cols, ill_dptr xq, ill_dptr xd, ill_dptr map, ill_dptr xh,
                           ill_stream stream) {
  if (rows < 0 || cols <= 0 || cols % 256 || !xq || !xd || !xh) return ILL_ERR_ARG;
  if ((xq & 15) || (xd & 3) || (map & 3) || (xh & 15)) return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  long long nrows = rows;
  const i8* qp = (const i8*)(uintptr_t)xq;
  const float* dp = (const float*)(uintptr_t)xd;
  const unsigned* mp = (const unsigned*)(uintptr_t)map;
  __half* hp = (__half*)(uintptr_t)xh;
  void* args[] = {&nrows, &cols, &qp, &dp, &mp, &hp};
  const long long threads = rows * (cols / 16);
  return launch_kernel((const void*)act_f16_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

extern "C" int ill_moe_mm_id(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases,
                             int ne, int64_t total_rows, ill_dptr xh, ill_dptr y, int64_t y_stride, ill_stream stream) {
  if (fmt != ILL_IQ2_XXS && fmt != ILL_Q2_K) return ILL_ERR_UNSUPPORTED;
  if (ncols <= 0 || ncols % 256 || nrows <= 0 || ne <= 0 || ne > 65535 || total_rows < 0 || y_stride < nrows)
    return ILL_ERR_ARG;
  if (!ptrs || !counts || !bases || !xh || !y) return ILL_ERR_ARG;
  if ((ptrs & 7) || (counts & 3) || (bases & 3) || (xh & 15) || (y & 15) || (y_stride & 3) || (add & 3))
    return ILL_ERR_ALIGN;
  if (total_rows == 0) return ILL_OK;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cuda_fail(cudaErrorNotSupported);
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)ncols, (cuuint64_t)total_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ncols * 2};
  const cuuint32_t box[2] = {MM_BK, MM_BM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)(uintptr_t)xh, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  MmParams p;
  p.ncols = ncols;
  p.nrows = nrows;
  p.row_bytes = ncols / 256 * fmt_block_bytes(fmt);
  p.add = add;
  p.ptrs = (const unsigned long long*)(uintptr_t)ptrs;
  p.counts = (const unsigned*)(uintptr_t)counts;
  p.bases = (const unsigned*)(uintptr_t)bases;
  p.y = (float*)(uintptr_t)y;
  p.y_stride = y_stride;
  p.ne = ne;
  p.max_mtiles = (int)((total_rows + MM_BM - 1) / MM_BM) + ne;  // every expert may end with a partial tile
  p.status = device_status_word();
  const size_t smem = 2 * MM_STAGES * MM_TILE_BYTES + 256 + 2048 + 128 + 1024;
  const void* k = fmt == ILL_IQ2_XXS ? (const void*)mm_id_kernel<ILL_IQ2_XXS> : (const void*)mm_id_kernel<ILL_Q2_K>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  void* args[] = {&map, &p};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((nrows + MM_BN - 1) / MM_BN, p.max_mtiles, 1);
  cfg.blockDim = dim3(MM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  e = cudaLaunchKernelExC(&cfg, k, args);
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}
