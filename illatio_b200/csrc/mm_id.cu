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
// A persistent grid (a CTA per SM) walks 128 (rows of X) x 128 (rows of W_e) tiles, K in steps of 64:
//   warp 0      one lane issues the TMA loads of the X tile (128-byte swizzle)
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128x128x16, fp16 in,
//               fp32 accumulate) and commits each stage back to the producers
//   warps 2-17  turn W_e's blocks into the swizzled shared-memory operand tile (four threads a
//               weight row, one K step each), and drain the accumulators block by block
//               (tcgen05.ld), scaling each block's sum; then store the tile's valid rows
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

constexpr int MM_BM = 128, MM_BN = 128, MM_BK = 64, MM_STAGES = 6;
constexpr int MM_THREADS = 576;                        // TMA warp, MMA warp, 16 dequantize / drain warps
constexpr int MM_DQ_WARPS = 16;
constexpr uint32_t MM_TILE_BYTES = MM_BM * MM_BK * 2;  // 16 KB, A or B

struct MmParams {
  int ncols, nrows;            // K and N of every expert matrix
  int row_bytes;
  long long add;
  const unsigned long long* ptrs;
  const unsigned* counts;
  const unsigned* bases;
  const float* xd;             // the activations' block scales, [token][K/256]
  const unsigned* map;         // token of each row of X (null: the row itself)
  long long total_rows;
  float* y;
  long long y_stride;          // floats between rows of Y
  int ne;
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

// ---- the weights' integer parts into the swizzled B tile ---------------------------------
// A thread owns half of a weight row's 64-wide K step: 32 weights = 4 chunks of 8 halves;
// chunk c of the row goes to 16-byte slot c ^ (row % 8) of the row's 128 bytes.
__device__ __forceinline__ void store_chunk(u8* tile, int row, int c, uint4 v) {
  *(uint4*)(tile + (row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4)) = v;
}

// N words at P (any alignment), from global memory
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

// two unsigned bytes (byte positions B0, B1 of V) as the halves 1024 + byte
__device__ __forceinline__ uint32_t bytes_to_h2_1024(uint32_t v, uint32_t sel) {
  return __byte_perm(v, 0x64646464u, sel);
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t h2_of(float a) {
  const __half2 h = __float2half2_rn(a);
  return *(const uint32_t*)&h;
}

// A thread's raw share of one block, prefetched a block ahead.  Thread (row, j) makes K step j
// (64 columns) of its row: IQ2_XXS sub-blocks 2j and 2j+1 (16 bytes); Q2_K the 32 quant bytes of
// half j/2, the four scale bytes of shifts 2(j&1) and 2(j&1)+1, and (j < 2) the eight scale
// bytes of half j for the mins; and the block's fp16 scale(s).
struct RawBlk { uint32_t w[8]; uint32_t s; uint32_t m[2]; uint32_t dd; };

template <int FMT>
__device__ __forceinline__ void load_raw(RawBlk& r, const u8* blk, int j) {
  if constexpr (FMT == ILL_IQ2_XXS) {
    uint32_t v[4];
    ldg_words<4>(blk + 2 + 16 * j, v);
    r.w[0] = v[0]; r.w[1] = v[1]; r.w[2] = v[2]; r.w[3] = v[3];
    r.dd = __ldg((const u16*)blk);
  } else {
    const uint32_t* q32 = (const uint32_t*)(blk + 16 + 32 * (j >> 1));  // a block is 4-byte aligned
#pragma unroll
    for (int i = 0; i < 8; ++i) r.w[i] = __ldg(q32 + i);
    r.s = __ldg((const uint32_t*)(blk + 8 * (j >> 1) + 4 * (j & 1)));
    if (j < 2) { r.m[0] = __ldg((const uint32_t*)(blk + 8 * j)); r.m[1] = __ldg((const uint32_t*)(blk + 8 * j + 4)); }
    r.dd = __ldg((const uint32_t*)(blk + 80));
  }
}

// The four lanes of a row write the same row of four different tiles; each starts ROT = 2j chunks
// further round the row, so that at any moment they touch different banks.
//
// IQ2_XXS: the K step's 64 integers grid * sign * (2 LS + 1) (at most 43 * 31: exact in fp16).  The
// block's float part is d / 8 (src/avx2.lisp:77-110 takes the products this way).  GRID and SMASK
// point at this lane's copy of the tables (eight interleaved copies: entry e of copy c at [8 e + c]).
__device__ __forceinline__ void b_iq2xxs(const RawBlk& r, int rot, u8* tile, int row, const uint2* grid,
                                         const uint2* smask) {
  const float ls0 = (float)(2 * (r.w[1] >> 28) + 1), ls1 = (float)(2 * (r.w[3] >> 28) + 1);
  // (1024 + (b + 128)) * s - 1152 s = b * s
  const uint32_t s20 = h2_of(ls0), bias0 = h2_of(-1152.0f * ls0), s21 = h2_of(ls1), bias1 = h2_of(-1152.0f * ls1);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = (i + rot) & 7, sb = c >> 2, l = c & 3;
    const uint32_t idx = sb ? r.w[2] : r.w[0], aux = sb ? r.w[3] : r.w[1];
    const uint32_t s2 = sb ? s21 : s20, bias = sb ? bias1 : bias0;
    const uint2 g = grid[8 * ((idx >> (8 * l)) & 0xff)];
    const uint2 m = smask[8 * ((aux >> (7 * l)) & 127)];
    // signed bytes: (g ^ m) - m per byte; then + 128 to make them unsigned for the conversion
    const uint32_t lo = ((g.x ^ m.x) + (m.x & 0x01010101u)) ^ 0x80808080u;
    const uint32_t hi = ((g.y ^ m.y) + (m.y & 0x01010101u)) ^ 0x80808080u;
    store_chunk(tile, row, c,
                make_uint4(hfma2(bytes_to_h2_1024(lo, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(lo, 0x4342), s2, bias),
                           hfma2(bytes_to_h2_1024(hi, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(hi, 0x4342), s2, bias)));
  }
}

// Q2_K: K step j of the block: shifts k = 2(j&1) + kk, kk = 0, 1; the 64 integers (scale & 15) * q
// (at most 45); chunk 4 kk + 2 half + c holds bytes 16 half + 8 c .. +7 of the 32 at shift k.
__device__ __forceinline__ void b_q2k(const RawBlk& r, int j, u8* tile, int row) {
#pragma unroll
  for (int pi = 0; pi < 4; ++pi) {
    const int cp = (pi + j) & 3, kk = cp >> 1, half = cp & 1;  // pairs of chunks, rotated by j
    const int k = 2 * (j & 1) + kk;
    const float sc = (float)((r.s >> (8 * (2 * kk + half))) & 15u);
    const uint32_t s2 = h2_of(sc), bias = h2_of(-1024.0f * sc);
    const uint32_t q0 = half ? r.w[4] : r.w[0], q1 = half ? r.w[5] : r.w[1], q2 = half ? r.w[6] : r.w[2],
                   q3 = half ? r.w[7] : r.w[3];
    const uint32_t w0 = (q0 >> (2 * k)) & 0x03030303u, w1 = (q1 >> (2 * k)) & 0x03030303u;
    const uint32_t w2 = (q2 >> (2 * k)) & 0x03030303u, w3 = (q3 >> (2 * k)) & 0x03030303u;
    store_chunk(tile, row, 2 * cp,
                make_uint4(hfma2(bytes_to_h2_1024(w0, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(w0, 0x4342), s2, bias),
                           hfma2(bytes_to_h2_1024(w1, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(w1, 0x4342), s2, bias)));
    store_chunk(tile, row, 2 * cp + 1,
                make_uint4(hfma2(bytes_to_h2_1024(w2, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(w2, 0x4342), s2, bias),
                           hfma2(bytes_to_h2_1024(w3, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(w3, 0x4342), s2, bias)));
  }
}
// Q2_K: half H's eight mins (scale >> 4) as chunk H of the "mins" tile
__device__ __forceinline__ void b_q2k_mins(const RawBlk& r, int h, u8* tile, int row) {
  const uint32_t lo = (r.m[0] >> 4) & 0x0f0f0f0fu, hi = (r.m[1] >> 4) & 0x0f0f0f0fu;
  const uint32_t k1024 = 0xe400e400u;  // -1024 twice
  uint32_t v[4];
  v[0] = bytes_to_h2_1024(lo, 0x4140); v[1] = bytes_to_h2_1024(lo, 0x4342);
  v[2] = bytes_to_h2_1024(hi, 0x4140); v[3] = bytes_to_h2_1024(hi, 0x4342);
#pragma unroll
  for (int i = 0; i < 4; ++i) asm("add.rn.f16x2 %0, %0, %1;" : "+r"(v[i]) : "r"(k1024));
  store_chunk(tile, row, h, make_uint4(v[0], v[1], v[2], v[3]));
}

// K steps per 256-wide block: four of the quants; for Q2_K a fifth whose A tile holds the
// activations' sums of 16 and whose B tile holds the mins (one K = 16 MMA into a second
// accumulator).
template <int FMT> struct MmGeom { static constexpr int SPB = FMT == ILL_Q2_K ? 5 : 4, ACCS = FMT == ILL_Q2_K ? 2 : 1; };

template <int FMT>
__global__ void __launch_bounds__(MM_THREADS) mm_id_kernel(const __grid_constant__ CUtensorMap xmap,
                                                           const __grid_constant__ CUtensorMap emap, const MmParams p) {
  constexpr int SPB = MmGeom<FMT>::SPB, ACCS = MmGeom<FMT>::ACCS;
  constexpr uint32_t TMEM_COLS = 2 * ACCS * MM_BN;  // two buffers of accumulators
  extern __shared__ __align__(1024) u8 smem_raw[];
  // [A stages][B stages] (each tile 1024-byte aligned, as the 128-byte swizzle needs), then barriers, tables
  u8* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  u8* a_tiles = smem;
  u8* b_tiles = smem + MM_STAGES * MM_TILE_BYTES;
  u8* tail = smem + 2 * MM_STAGES * MM_TILE_BYTES;
  uint64_t* full_a = (uint64_t*)tail;            // TMA bytes landed
  uint64_t* full_b = full_a + MM_STAGES;         // 8 dequantizing warps arrived
  uint64_t* empty = full_b + MM_STAGES;          // the MMAs that read the stage completed
  uint64_t* acc_full = empty + MM_STAGES;        // [2] a block's MMAs completed
  uint64_t* acc_free = acc_full + 2;             // [2] the 8 drain warps read the buffer
  uint32_t* tmem_slot = (uint32_t*)(acc_free + 2);
  float* wsc = (float*)(tail + 256);             // [2 buffers][2: d, dmin][128 rows] of the block
  int* tile_first = (int*)(tail + 256 + 2048);   // [ne + 1] first row tile of each expert; the total
  uint2* iq_grid = (uint2*)(tail + 256 + 2048 + 2304);  // eight interleaved copies
  uint2* iq_smask = iq_grid + 8 * 256;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- once per CTA: the experts' row tiles counted (first tile of each expert, in shared memory),
  // barriers, tables, tensor memory.  The CTA then walks tiles blockIdx.x, + gridDim.x, ...
  if (warp == 0) {
    int before = 0;
    for (int e0 = 0; e0 < p.ne; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < p.ne ? (int)p.counts[e] : 0;
      const int tiles = (c + MM_BM - 1) / MM_BM;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (e < p.ne) tile_first[e] = before + incl - tiles;
      before += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) tile_first[p.ne] = before;  // row tiles in all
  }
  if (tid == 32) {
    for (int s = 0; s < MM_STAGES; ++s) { mbar_init(&full_a[s], 1); mbar_init(&full_b[s], MM_DQ_WARPS); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_free[b], MM_DQ_WARPS); }
    mbar_fence_init();
  }
  if (FMT == ILL_IQ2_XXS) {
    for (int i = tid; i < 8 * 256; i += MM_THREADS) {
      const uint64_t g = ill_iq2xxs_grid[i >> 3];
      iq_grid[i] = make_uint2((uint32_t)g, (uint32_t)(g >> 32));
    }
    for (int i = tid; i < 8 * 128; i += MM_THREADS) {
      const uint32_t sg = ill_ksigns_iq2xs[i >> 3];
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if ((sg >> j) & 1) lo |= 0xffu << (8 * j);
        if ((sg >> (4 + j)) & 1) hi |= 0xffu << (8 * j);
      }
      iq_smask[i] = make_uint2(lo, hi);
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nkb = p.ncols / 256;
  const int ntn = (p.nrows + MM_BN - 1) / MM_BN;
  const int ntiles = tile_first[p.ne] * ntn;  // weight-row tiles vary fastest: CTAs running together share X
  bool ok = true;

  // tile index -> expert, first row of X, valid rows, weight-row tile
  auto locate = [&](int tile, int& expert, int& row0, int& nvalid, int& nt) {
    const int mt = tile / ntn;
    nt = tile - mt * ntn;
    int lo = 0, hi = p.ne - 1;  // the last expert whose first tile is <= mt and that has tiles
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (tile_first[mid] <= mt) lo = mid; else hi = mid - 1;
    }
    expert = lo;
    const int m_in = mt - tile_first[lo];
    row0 = (int)p.bases[lo] + m_in * MM_BM;
    nvalid = min(MM_BM, (int)p.counts[lo] - m_in * MM_BM);
  };

  if (warp == 0) {
    // ---- TMA producer of the X tiles
    if (lane == 0) {
      int g_st = 0;  // stages issued so far by this CTA
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int expert, row0, nvalid, nt;
        locate(tile, expert, row0, nvalid, nt);
        for (int st = 0; st < nkb * SPB; ++st, ++g_st) {
          const int s = g_st % MM_STAGES, use = g_st / MM_STAGES;
          if (use > 0 && !mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY)) { ok = false; break; }
          const int kb = st / SPB, j = st - kb * SPB;
          mbar_expect_tx(&full_a[s], MM_TILE_BYTES);
          if (j < 4) tma_load_2d(a_tiles + s * MM_TILE_BYTES, &xmap, kb * 256 + j * MM_BK, row0, &full_a[s]);
          else tma_load_2d(a_tiles + s * MM_TILE_BYTES, &emap, kb * MM_BK, row0, &full_a[s]);  // the sums of 16
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      // fp32 accumulate, fp16 A and B, both K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(MM_BN >> 3) << 17) | ((uint32_t)(MM_BM >> 4) << 24);
      int g_st = 0, g_kb = 0;  // stages and blocks consumed so far by this CTA
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < nkb && ok; ++kb, ++g_kb) {
          const int b = g_kb & 1;
          if (g_kb >= 2 && !mbar_wait(&acc_free[b], (uint32_t)(g_kb / 2 - 1) & 1u, p.status, ST_MM_WAIT_EPI)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d1 = tmem_base + (uint32_t)(b * ACCS * MM_BN);
          for (int j = 0; j < SPB; ++j, ++g_st) {
            const int s = g_st % MM_STAGES;
            const uint32_t par = (uint32_t)(g_st / MM_STAGES) & 1u;
            if (!mbar_wait(&full_a[s], par, p.status, ST_MM_WAIT_FULL) ||
                !mbar_wait(&full_b[s], par, p.status, ST_MM_WAIT_FULL + 1)) { ok = false; break; }
            tc_fence_after();
            const uint64_t ad = umma_desc(a_tiles + s * MM_TILE_BYTES), bd = umma_desc(b_tiles + s * MM_TILE_BYTES);
            if (j < 4) {
#pragma unroll
              for (int k = 0; k < MM_BK / 16; ++k)  // 32 bytes further along K inside the swizzle atom each time
                umma_f16(d1, ad + 2 * k, bd + 2 * k, idesc, (j | k) ? 1u : 0u);
            } else {
              umma_f16(d1 + MM_BN, ad, bd, idesc, 0u);  // mins x sums of 16: one K = 16 product
            }
            umma_commit(&empty[s]);  // frees the stage when these MMAs are done
          }
          if (ok) umma_commit(&acc_full[b]);
        }
      }
    }
  } else {
    // ---- warps 2..17: the weights' integer parts into the B tiles; the accumulators drained block by
    // block with the block's float scales; the tile's store
    const int t = tid - 64;                        // 0..511
    const int row = t >> 2, j = t & 3;             // weight row in the tile, K step of each block
    constexpr int BB = FMT == ILL_IQ2_XXS ? 66 : 84;
    const int q = warp & 3;                        // TMEM lanes 32q .. 32q+31 are this warp's
    const int m = q * 32 + lane;                   // accumulator row
    const int cq = (warp - 2) >> 2;                // columns 32*cq .. +31
    int g_st = 0, g_kb = 0;                        // stages / blocks produced so far by this CTA
    int d_kb = 0;                                  // blocks drained so far
    // per tile
    bool has_row = false;
    const u8* wrow = nullptr;
    int nvalid = 0;
    long long tok = -1;
    float out[32];

    // Block KB's B tiles from CUR (its raw words, loaded a block ago); NXT gets the next block's.
    auto produce = [&](int kb, const RawBlk& cur, RawBlk& nxt) -> bool {
      const int b = g_kb & 1;
      if (kb + 1 < nkb && has_row) load_raw<FMT>(nxt, wrow + (long long)(kb + 1) * BB, j);
      if (g_kb >= 2) {  // the scales two blocks back have been read by every drain warp
        bool w_ok = mbar_wait(&acc_free[b], (uint32_t)(g_kb / 2 - 1) & 1u, p.status, ST_MM_WAIT_EPI + 1);
        if (!__all_sync(0xffffffffu, w_ok)) return false;
      }
      if (j == 0) {
        float d = 0.0f, dmin = 0.0f;
        if (has_row) { d = h2f(cur.dd & 0xffff); dmin = h2f(cur.dd >> 16); }
        wsc[b * 256 + row] = d;
        wsc[b * 256 + 128 + row] = dmin;
      }
      {
        const int st = g_st + j, s = st % MM_STAGES, use = st / MM_STAGES;
        bool w_ok = true;
        if (use > 0) w_ok = mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 1);
        if (!__all_sync(0xffffffffu, w_ok)) return false;
        u8* tile = b_tiles + s * MM_TILE_BYTES;
        if (has_row) {
          if constexpr (FMT == ILL_IQ2_XXS) b_iq2xxs(cur, 2 * j, tile, row, iq_grid + (lane & 7), iq_smask + (lane & 7));
          else b_q2k(cur, j, tile, row);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) store_chunk(tile, row, (c + 2 * j) & 7, make_uint4(0, 0, 0, 0));
        }
        fence_async_smem();  // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane < 4) mbar_arrive(&full_b[s]);  // lane j for the stage the K-step-j lanes wrote
      }
      if constexpr (SPB == 5) {
        const int st = g_st + 4, s = st % MM_STAGES, use = st / MM_STAGES;
        bool w_ok = true;
        if (use > 0) w_ok = mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 1);
        if (!__all_sync(0xffffffffu, w_ok)) return false;
        u8* tile = b_tiles + s * MM_TILE_BYTES;
        if (j < 2) {
          if (has_row) b_q2k_mins(cur, j, tile, row);
          else store_chunk(tile, row, j, make_uint4(0, 0, 0, 0));
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_b[s]);
      }
      g_st += SPB;
      ++g_kb;
      return true;
    };
    // Block KB of the current tile (the D_KB-th block of this CTA) out of tensor memory into OUT.
    auto drain = [&](int kb) -> bool {
      const int b = d_kb & 1;
      bool e_ok = mbar_wait(&acc_full[b], (uint32_t)(d_kb / 2) & 1u, p.status, ST_MM_WAIT_ACC);
      if (!__all_sync(0xffffffffu, e_ok)) return false;
      tc_fence_after();
      if (32 * q < nvalid) {  // a quarter of the tile with no valid row is not read
        const float dx = tok >= 0 ? p.xd[tok * nkb + kb] : 0.0f;
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * ACCS * MM_BN + 32 * cq);
        const float4* wd = (const float4*)(wsc + b * 256 + 32 * cq);
        uint32_t v[32];
        tmem_ld32(t0, v);
        if constexpr (FMT == ILL_IQ2_XXS) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 dw = wd[i >> 2];
            // IQ2XXS-DOT-AVX2 (src/avx2.lisp:107-110): total += d * y.d * sum; the 1/8 at the end
            out[i] = fmaf(__fmul_rn(dw.x, dx), __uint_as_float(v[i]), out[i]);
            out[i + 1] = fmaf(__fmul_rn(dw.y, dx), __uint_as_float(v[i + 1]), out[i + 1]);
            out[i + 2] = fmaf(__fmul_rn(dw.z, dx), __uint_as_float(v[i + 2]), out[i + 2]);
            out[i + 3] = fmaf(__fmul_rn(dw.w, dx), __uint_as_float(v[i + 3]), out[i + 3]);
          }
        } else {
          // Q2K-DOT-AVX2 (src/avx2.lisp:147-150): y.d * d * sum - y.d * dmin * mins; the sums first,
          // then the mins through the same registers
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 dw = wd[i >> 2];
            out[i] = fmaf(__fmul_rn(dx, dw.x), __uint_as_float(v[i]), out[i]);
            out[i + 1] = fmaf(__fmul_rn(dx, dw.y), __uint_as_float(v[i + 1]), out[i + 1]);
            out[i + 2] = fmaf(__fmul_rn(dx, dw.z), __uint_as_float(v[i + 2]), out[i + 2]);
            out[i + 3] = fmaf(__fmul_rn(dx, dw.w), __uint_as_float(v[i + 3]), out[i + 3]);
          }
          tmem_ld32(t0 + MM_BN, v);
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 dm = wd[32 + (i >> 2)];
            out[i] = fmaf(-__fmul_rn(dx, dm.x), __uint_as_float(v[i]), out[i]);
            out[i + 1] = fmaf(-__fmul_rn(dx, dm.y), __uint_as_float(v[i + 1]), out[i + 1]);
            out[i + 2] = fmaf(-__fmul_rn(dx, dm.z), __uint_as_float(v[i + 2]), out[i + 2]);
            out[i + 3] = fmaf(-__fmul_rn(dx, dm.w), __uint_as_float(v[i + 3]), out[i + 3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[b]);
      ++d_kb;
      return true;
    };

    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      int expert, row0, nt;
      locate(tile, expert, row0, nvalid, nt);
      const int n = nt * MM_BN + row;
      has_row = n < p.nrows;
      wrow = (const u8*)(uintptr_t)p.ptrs[expert] + p.add + (long long)(has_row ? n : 0) * p.row_bytes;
      const long long place = (long long)row0 + m;
      tok = place < p.total_rows ? (p.map ? (long long)p.map[place] : place) : -1;
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = 0.0f;
      RawBlk r0, r1;
      if (has_row) load_raw<FMT>(r0, wrow, j);
      for (int kb = 0; kb < nkb && ok; kb += 2) {
        ok = produce(kb, r0, r1);
        if (ok && kb >= 1) ok = drain(kb - 1);
        if (ok && kb + 1 < nkb) {
          ok = produce(kb + 1, r1, r0);
          if (ok) ok = drain(kb);
        }
      }
      if (ok) ok = drain(nkb - 1);
      if (ok && m < nvalid) {
        float* yrow = p.y + place * p.y_stride + (long long)nt * MM_BN + 32 * cq;
        const float fin = FMT == ILL_IQ2_XXS ? 0.125f : 1.0f;
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
          const int n0 = nt * MM_BN + 32 * cq + jj;
          if (n0 + 3 < p.nrows) {
            *(float4*)(yrow + jj) = make_float4(out[jj] * fin, out[jj + 1] * fin, out[jj + 2] * fin, out[jj + 3] * fin);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (n0 + e < p.nrows) yrow[jj + e] = out[jj + e] * fin;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// The Q8_K activations as the tensor cores take them, in expert order: XH[place, k] = fp16(q[t, k])
// (exact), t = MAP[place] (or place when MAP is null); and, when XE is given, the sums of 16 as
// XE[place, kb, 0..15] = fp16(bsums[t, 16 kb ..]) (exact: at most 2032), the other 48 of each 64 zero.
__global__ void __launch_bounds__(256) act_f16_kernel(long long rows, int cols, const i8* __restrict__ xq,
                                                      const int16_t* __restrict__ bsums,
                                                      const unsigned* __restrict__ map, __half* __restrict__ xh,
                                                      __half* __restrict__ xe) {
  pdl_launch_dependents();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread: 16 values
  const int per_row = cols / 16;
  if (gid >= rows * per_row) return;
  const long long place = gid / per_row;
  const int j = (int)(gid - place * per_row);
  const long long t = map ? (long long)map[place] : place;
  const uint4 q = *(const uint4*)(xq + t * cols + 16 * j);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int b0 = (int)(signed char)((w[i >> 1] >> (16 * (i & 1))) & 0xff);
    const int b1 = (int)(signed char)((w[i >> 1] >> (16 * (i & 1) + 8)) & 0xff);
    const __half2 hh = __floats2half2_rn((float)b0, (float)b1);
    h[i] = *(const uint32_t*)&hh;
  }
  uint4* dst = (uint4*)(xh + place * cols + 16 * j);
  dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
  dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
  if (xe) {
    // this thread's 16 quants are one sum of 16: element j%16 of block j/16; it also clears 3 of the 48 zeros
    const int kb = j >> 4, g = j & 15;
    __half* e = xe + (place * (cols / 256) + kb) * 64;
    e[g] = __float2half_rn((float)bsums[t * (cols / 16) + j]);
    e[16 + 3 * g] = __float2half_rn(0.0f);
    e[16 + 3 * g + 1] = __float2half_rn(0.0f);
    e[16 + 3 * g + 2] = __float2half_rn(0.0f);
  }
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

extern "C" int ill_act_f16(int64_t rows, int cols, ill_dptr xq, ill_dptr bsums, ill_dptr map, ill_dptr xh, ill_dptr xe,
                           ill_stream stream) {
  if (rows < 0 || cols <= 0 || cols % 256 || !xq || !xh || (xe && !bsums)) return ILL_ERR_ARG;
  if ((xq & 15) || (bsums & 1) || (map & 3) || (xh & 15) || (xe & 15)) return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  long long nrows = rows;
  const i8* qp = (const i8*)(uintptr_t)xq;
  const int16_t* bp = (const int16_t*)(uintptr_t)bsums;
  const unsigned* mp = (const unsigned*)(uintptr_t)map;
  __half* hp = (__half*)(uintptr_t)xh;
  __half* ep = (__half*)(uintptr_t)xe;
  void* args[] = {&nrows, &cols, &qp, &bp, &mp, &hp, &ep};
  const long long threads = rows * (cols / 16);
  return launch_kernel((const void*)act_f16_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

static int encode_map(CUtensorMap* map, ill_dptr base, int64_t inner, int64_t rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cuda_fail(cudaErrorNotSupported);
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)inner * 2};
  const cuuint32_t box[2] = {MM_BK, MM_BM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)(uintptr_t)base, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ILL_OK : cuda_fail(cudaErrorInvalidValue);
}

extern "C" int ill_moe_mm_id(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases,
                             int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr y,
                             int64_t y_stride, ill_stream stream) {
  if (fmt != ILL_IQ2_XXS && fmt != ILL_Q2_K) return ILL_ERR_UNSUPPORTED;
  if (ncols <= 0 || ncols % 256 || nrows <= 0 || ne <= 0 || ne > 65535 || total_rows < 0 || y_stride < nrows)
    return ILL_ERR_ARG;
  if (!ptrs || !counts || !bases || !xh || !xd || !y || (fmt == ILL_Q2_K && !xe)) return ILL_ERR_ARG;
  if ((ptrs & 7) || (counts & 3) || (bases & 3) || (xh & 15) || (xe & 15) || (xd & 3) || (map & 3) || (y & 15) ||
      (y_stride & 3) || (add & 3))
    return ILL_ERR_ALIGN;
  if (total_rows == 0) return ILL_OK;
  CUtensorMap xmap, emap;
  int rc = encode_map(&xmap, xh, ncols, total_rows);
  if (rc) return rc;
  rc = fmt == ILL_Q2_K ? encode_map(&emap, xe, (int64_t)(ncols / 256) * 64, total_rows) : encode_map(&emap, xh, ncols, total_rows);
  if (rc) return rc;
  MmParams p;
  p.ncols = ncols;
  p.nrows = nrows;
  p.row_bytes = ncols / 256 * fmt_block_bytes(fmt);
  p.add = add;
  p.ptrs = (const unsigned long long*)(uintptr_t)ptrs;
  p.counts = (const unsigned*)(uintptr_t)counts;
  p.bases = (const unsigned*)(uintptr_t)bases;
  p.xd = (const float*)(uintptr_t)xd;
  p.map = (const unsigned*)(uintptr_t)map;
  p.total_rows = total_rows;
  p.y = (float*)(uintptr_t)y;
  p.y_stride = y_stride;
  p.ne = ne;
  p.status = device_status_word();
  const long long max_tiles = ((total_rows + MM_BM - 1) / MM_BM + ne) * ((nrows + MM_BN - 1) / MM_BN);  // an upper bound
  // tiles, barriers, scales, the experts' first tiles, tables x 8, alignment
  const size_t smem = 2 * MM_STAGES * MM_TILE_BYTES + 256 + 2048 + 2304 + 8 * 2048 + 8 * 1024 + 1024;
  if (ne > 512) return ILL_ERR_TOO_LARGE;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const void* k = fmt == ILL_IQ2_XXS ? (const void*)mm_id_kernel<ILL_IQ2_XXS> : (const void*)mm_id_kernel<ILL_Q2_K>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  void* args[] = {&xmap, &emap, &p};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(max_tiles < sms ? max_tiles : sms), 1, 1);  // persistent: a CTA an SM, each walks tiles
  cfg.blockDim = dim3(MM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  e = cudaLaunchKernelExC(&cfg, k, args);
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}
