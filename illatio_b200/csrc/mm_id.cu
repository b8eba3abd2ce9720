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

constexpr int MM_BM = 128, MM_BN = 128, MM_BK = 64, MM_STAGES = 6;
constexpr int MM_THREADS = 320;                        // TMA warp, MMA warp, 8 dequantize / drain warps
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

// A thread's raw share of one block, prefetched a block ahead: half H of the block's quants (32
// bytes: IQ2_XXS sub-blocks 4h..4h+3; Q2_K quant bytes 32h..32h+31), Q2_K's 8 scale bytes of that
// half, and the block's fp16 scale(s).
struct RawBlk { uint32_t w[8]; uint32_t s[2]; uint32_t dd; };

template <int FMT>
__device__ __forceinline__ void load_raw(RawBlk& r, const u8* blk, int h) {
  if constexpr (FMT == ILL_IQ2_XXS) {
    ldg_words<8>(blk + 2 + 32 * h, r.w);
    r.dd = __ldg((const u16*)blk);
    r.s[0] = r.s[1] = 0;
  } else {
    const uint4* q = (const uint4*)(blk + 16 + 32 * h);  // a block is 4-byte aligned; 16-byte loads need more
    const uint32_t* q32 = (const uint32_t*)q;
#pragma unroll
    for (int i = 0; i < 8; ++i) r.w[i] = __ldg(q32 + i);
    r.s[0] = __ldg((const uint32_t*)(blk + 8 * h));
    r.s[1] = __ldg((const uint32_t*)(blk + 8 * h + 4));
    r.dd = __ldg((const uint32_t*)(blk + 80));
  }
}

// IQ2_XXS: one sub-block (IDX, AUX) as the 32 integers grid * sign * (2 LS + 1) (at most 43 * 31:
// exact in fp16), chunks CB .. CB+3 of the row.  The block's float part is d / 8
// (src/avx2.lisp:77-110 takes the products this way).
// GRID and SMASK point at this lane's copy of the tables (eight interleaved copies: entry e of
// copy c at [8 e + c], so lanes that use different copies never meet in a bank).
__device__ __forceinline__ void b_iq2xxs(uint32_t idx, uint32_t aux, int cb, u8* tile, int row, const uint2* grid,
                                         const uint2* smask) {
  const float ls = (float)(2 * (aux >> 28) + 1);
  const uint32_t s2 = h2_of(ls), bias = h2_of(-1152.0f * ls);  // (1024 + (b + 128)) * s - 1152 s = b * s
#pragma unroll
  for (int l = 0; l < 4; ++l) {
    const uint2 g = grid[8 * ((idx >> (8 * l)) & 0xff)];
    const uint2 m = smask[8 * ((aux >> (7 * l)) & 127)];
    // signed bytes: (g ^ m) - m per byte; then + 128 to make them unsigned for the conversion
    const uint32_t lo = ((g.x ^ m.x) + (m.x & 0x01010101u)) ^ 0x80808080u;
    const uint32_t hi = ((g.y ^ m.y) + (m.y & 0x01010101u)) ^ 0x80808080u;
    store_chunk(tile, row, cb + l,
                make_uint4(hfma2(bytes_to_h2_1024(lo, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(lo, 0x4342), s2, bias),
                           hfma2(bytes_to_h2_1024(hi, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(hi, 0x4342), s2, bias)));
  }
}

// Q2_K: K step JJ (0, 1) of the thread's half block: shifts k = 2 jj, 2 jj + 1; the 64 integers
// (scale & 15) * q (at most 45) as the row's 8 chunks.
__device__ __forceinline__ void b_q2k(const RawBlk& r, int jj, int flip, u8* tile, int row) {
#pragma unroll
  for (int kk0 = 0; kk0 < 2; ++kk0) {
    const int kk = kk0 ^ flip;  // the two lanes of a row write different halves of their tiles at any moment
    const int k = 2 * jj + kk;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int sb = 2 * k + half;  // scale byte of the half block
      const float sc = (float)((r.s[sb >> 2] >> (8 * (sb & 3))) & 15u);
      const uint32_t s2 = h2_of(sc), bias = h2_of(-1024.0f * sc);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t w0 = (r.w[4 * half + 2 * c] >> (2 * k)) & 0x03030303u;
        const uint32_t w1 = (r.w[4 * half + 2 * c + 1] >> (2 * k)) & 0x03030303u;
        store_chunk(tile, row, 4 * kk + 2 * half + c,
                    make_uint4(hfma2(bytes_to_h2_1024(w0, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(w0, 0x4342), s2, bias),
                               hfma2(bytes_to_h2_1024(w1, 0x4140), s2, bias), hfma2(bytes_to_h2_1024(w1, 0x4342), s2, bias)));
      }
    }
  }
}
// Q2_K: the half block's eight mins (scale >> 4) as chunk H of the "mins" tile
__device__ __forceinline__ void b_q2k_mins(const RawBlk& r, int h, u8* tile, int row) {
  const uint32_t lo = (r.s[0] >> 4) & 0x0f0f0f0fu, hi = (r.s[1] >> 4) & 0x0f0f0f0fu;
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
  int* tile_info = (int*)(tmem_slot + 1);        // expert, row0, rows valid
  float* wsc = (float*)(tail + 256);             // [2 buffers][2: d, dmin][128 rows] of the block
  uint2* iq_grid = (uint2*)(tail + 256 + 2048);  // eight interleaved copies
  uint2* iq_smask = iq_grid + 8 * 256;

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
    for (int s = 0; s < MM_STAGES; ++s) { mbar_init(&full_a[s], 1); mbar_init(&full_b[s], 8); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_free[b], 8); }
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
  __syncthreads();
  const int expert = tile_info[0], row0 = tile_info[1], nvalid = tile_info[2];
  if (expert < 0) return;  // past the last row tile: nothing allocated, nothing in flight
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nkb = p.ncols / 256;
  const int nsteps = nkb * SPB;
  const u8* wexp = (const u8*)(uintptr_t)p.ptrs[expert] + p.add;
  bool ok = true;

  if (warp == 0) {
    // ---- TMA producer of the X tiles
    if (lane == 0) {
      for (int st = 0; st < nsteps; ++st) {
        const int s = st % MM_STAGES, use = st / MM_STAGES;
        if (use > 0 && !mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY)) { ok = false; break; }
        const int kb = st / SPB, j = st - kb * SPB;
        mbar_expect_tx(&full_a[s], MM_TILE_BYTES);
        if (j < 4) tma_load_2d(a_tiles + s * MM_TILE_BYTES, &xmap, kb * 256 + j * MM_BK, row0, &full_a[s]);
        else tma_load_2d(a_tiles + s * MM_TILE_BYTES, &emap, kb * MM_BK, row0, &full_a[s]);  // the sums of 16
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      // fp32 accumulate, fp16 A and B, both K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(MM_BN >> 3) << 17) | ((uint32_t)(MM_BM >> 4) << 24);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int b = kb & 1;
        if (kb >= 2 && !mbar_wait(&acc_free[b], (uint32_t)(kb / 2 - 1) & 1u, p.status, ST_MM_WAIT_EPI)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d1 = tmem_base + (uint32_t)(b * ACCS * MM_BN);
        for (int j = 0; j < SPB; ++j) {
          const int st = kb * SPB + j, s = st % MM_STAGES;
          const uint32_t par = (uint32_t)(st / MM_STAGES) & 1u;
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
  } else {
    // ---- warps 2..9: the weights' integer parts into the B tiles; the accumulators drained block by
    // block with the block's float scales; the final store
    const int t = tid - 64;                        // 0..255
    const int row = t >> 1, half = t & 1;          // weight row in the tile, half of each K step
    const int n = nt * MM_BN + row;
    const bool has_row = n < p.nrows;
    const u8* wrow = wexp + (long long)(has_row ? n : 0) * p.row_bytes;
    constexpr int BB = FMT == ILL_IQ2_XXS ? 66 : 84;
    const int q = warp & 3;                        // TMEM lanes 32q .. 32q+31 are this warp's
    const int m = q * 32 + lane;                   // accumulator row
    const int chalf = (warp - 2) >> 2;             // columns 64*chalf .. +63
    const long long place = (long long)row0 + m;
    const long long tok = place < p.total_rows ? (p.map ? (long long)p.map[place] : place) : -1;
    float out[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) out[i] = 0.0f;

    // Block KB's B tiles from CUR (its raw words, loaded a block ago); NXT gets block KB+1's.
    // The thread's half H of the block is K steps 2h and 2h+1 (all 64 columns of its row).
    auto produce = [&](int kb, const RawBlk& cur, RawBlk& nxt) -> bool {
      const int b = kb & 1;
      if (kb + 1 < nkb && has_row) load_raw<FMT>(nxt, wrow + (long long)(kb + 1) * BB, half);
      if (kb >= 2) {  // the scales of block kb - 2 have been read by every drain warp
        bool w_ok = mbar_wait(&acc_free[b], (uint32_t)(kb / 2 - 1) & 1u, p.status, ST_MM_WAIT_EPI + 1);
        if (!__all_sync(0xffffffffu, w_ok)) return false;
      }
      if (half == 0) {
        float d = 0.0f, dmin = 0.0f;
        if (has_row) { d = h2f(cur.dd & 0xffff); dmin = h2f(cur.dd >> 16); }
        wsc[b * 256 + row] = d;
        wsc[b * 256 + 128 + row] = dmin;
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int st = kb * SPB + 2 * half + jj, s = st % MM_STAGES, use = st / MM_STAGES;
        bool w_ok = true;
        if (use > 0) w_ok = mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 1);
        if (!__all_sync(0xffffffffu, w_ok)) return false;
        u8* tile = b_tiles + s * MM_TILE_BYTES;
        if (has_row) {
          if constexpr (FMT == ILL_IQ2_XXS) {
            // the two lanes of a row write different halves of their (different) tiles at any moment: no bank meets
            const uint32_t i0 = half ? cur.w[4 * jj + 2] : cur.w[4 * jj], a0 = half ? cur.w[4 * jj + 3] : cur.w[4 * jj + 1];
            const uint32_t i1 = half ? cur.w[4 * jj] : cur.w[4 * jj + 2], a1 = half ? cur.w[4 * jj + 1] : cur.w[4 * jj + 3];
            b_iq2xxs(i0, a0, 4 * half, tile, row, iq_grid + (lane & 7), iq_smask + (lane & 7));
            b_iq2xxs(i1, a1, 4 - 4 * half, tile, row, iq_grid + (lane & 7), iq_smask + (lane & 7));
          } else {
            b_q2k(cur, jj, half, tile, row);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) store_chunk(tile, row, c, make_uint4(0, 0, 0, 0));
        }
        fence_async_smem();  // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane < 2) mbar_arrive(&full_b[s]);  // lane 0 for the h = 0 lanes' stage, lane 1 for the h = 1 lanes'
      }
      if constexpr (SPB == 5) {
        const int st = kb * SPB + 4, s = st % MM_STAGES, use = st / MM_STAGES;
        bool w_ok = true;
        if (use > 0) w_ok = mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 1);
        if (!__all_sync(0xffffffffu, w_ok)) return false;
        u8* tile = b_tiles + s * MM_TILE_BYTES;
        if (has_row) b_q2k_mins(cur, half, tile, row);
        else store_chunk(tile, row, half, make_uint4(0, 0, 0, 0));
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_b[s]);
      }
      return true;
    };
    auto drain = [&](int kb) -> bool {
      const int b = kb & 1;
      bool e_ok = mbar_wait(&acc_full[b], (uint32_t)(kb / 2) & 1u, p.status, ST_MM_WAIT_ACC);
      if (!__all_sync(0xffffffffu, e_ok)) return false;
      tc_fence_after();
      if (32 * q < nvalid) {  // a quarter of the tile with no valid row is not read
        const float dx = tok >= 0 ? p.xd[tok * nkb + kb] : 0.0f;
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * ACCS * MM_BN + 64 * chalf);
        const float4* wd = (const float4*)(wsc + b * 256 + 64 * chalf);
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(t0 + c0, v);
          if constexpr (FMT == ILL_IQ2_XXS) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 dw = wd[(c0 + i) >> 2];
              // IQ2XXS-DOT-AVX2 (src/avx2.lisp:107-110): total += d * y.d * sum; the 1/8 at the end
              out[c0 + i] = fmaf(__fmul_rn(dw.x, dx), __uint_as_float(v[i]), out[c0 + i]);
              out[c0 + i + 1] = fmaf(__fmul_rn(dw.y, dx), __uint_as_float(v[i + 1]), out[c0 + i + 1]);
              out[c0 + i + 2] = fmaf(__fmul_rn(dw.z, dx), __uint_as_float(v[i + 2]), out[c0 + i + 2]);
              out[c0 + i + 3] = fmaf(__fmul_rn(dw.w, dx), __uint_as_float(v[i + 3]), out[c0 + i + 3]);
            }
          } else {
            uint32_t v2[32];
            tmem_ld32(t0 + MM_BN + c0, v2);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 dw = wd[(c0 + i) >> 2], dm = wd[32 + ((c0 + i) >> 2)];
              const float dws[4] = {dw.x, dw.y, dw.z, dw.w}, dms[4] = {dm.x, dm.y, dm.z, dm.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                // Q2K-DOT-AVX2 (src/avx2.lisp:147-150): y.d * d * sum - y.d * dmin * mins
                const float t1 = fmaf(__fmul_rn(dx, dws[e]), __uint_as_float(v[i + e]), out[c0 + i + e]);
                out[c0 + i + e] = fmaf(-__fmul_rn(dx, dms[e]), __uint_as_float(v2[i + e]), t1);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[b]);
      return true;
    };

    RawBlk r0, r1;
    if (has_row) load_raw<FMT>(r0, wrow, half);
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
      float* yrow = p.y + place * p.y_stride + (long long)nt * MM_BN + 64 * chalf;
      const float fin = FMT == ILL_IQ2_XXS ? 0.125f : 1.0f;
#pragma unroll
      for (int j = 0; j < 64; j += 4) {
        const int n0 = nt * MM_BN + 64 * chalf + j;
        if (n0 + 3 < p.nrows) {
          *(float4*)(yrow + j) = make_float4(out[j] * fin, out[j + 1] * fin, out[j + 2] * fin, out[j + 3] * fin);
        } else {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            if (n0 + jj < p.nrows) yrow[j + jj] = out[j + jj] * fin;
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
  const int max_mtiles = (int)((total_rows + MM_BM - 1) / MM_BM) + ne;  // every expert may end with a partial tile
  const size_t smem = 2 * MM_STAGES * MM_TILE_BYTES + 256 + 2048 + 8 * 2048 + 8 * 1024 + 1024;  // tiles, barriers, scales, tables x 8, alignment
  const void* k = fmt == ILL_IQ2_XXS ? (const void*)mm_id_kernel<ILL_IQ2_XXS> : (const void*)mm_id_kernel<ILL_Q2_K>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  void* args[] = {&xmap, &emap, &p};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((nrows + MM_BN - 1) / MM_BN, max_mtiles, 1);
  cfg.blockDim = dim3(MM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  e = cudaLaunchKernelExC(&cfg, k, args);
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}
