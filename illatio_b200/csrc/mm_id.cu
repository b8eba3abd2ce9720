// mm_id.cu -- the routed experts' product for a chunk of tokens, on the 5th-generation
// tensor cores (tcgen05, operands and accumulators in tensor memory).
//
//   Y[place, n] = sum_k X[place, k] * W_e[n, k]      for every expert e and every row
//                                                    `place` in [bases[e], bases[e] + counts[e])
//
// X is the chunk's activations already grouped by expert (ill_moe_group), as fp16
// (ill_act_f16: the Q8_K quants, exact in fp16).  W_e is expert e's matrix of raw IQ2_XXS
// or Q2_K blocks at ptrs[e] + add -- or of Q4_K / Q6_K blocks: the dense prefill products run through the same
// kernel with the matrix as its one expert (ill_mm_chunk; mm_q4k_mma / mm_q6k_mma, src/cuda/kquant.cu:316-466).
//
// A persistent grid (a CTA per SM) walks tiles of 128 weight rows x up to 128 rows of X.  The
// weights are the tensor core's A operand and live in tensor memory: the dequantizing warps write
// their integer parts (exact in fp16) there with tcgen05.st, so they never pass through shared
// memory; X is the B operand, brought by TMA (128-byte swizzle).  The accumulator
// D[weight row, row of X] is drained once per 256-wide block of K and scaled by the block's two
// float scales, which is the order the reference's CPU kernels multiply in.
//   warp 0      one lane issues the TMA loads of the X tiles
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128 x N x 16, fp16 in,
//               fp32 accumulate) and commits each step back to the producers
//   warps 2-3   bring W_e's raw blocks and the X rows' block scales into rings in shared memory
//               (cp.async)
//   warps 4-7   drain the accumulators block by block (tcgen05.ld), scaling each block's integer
//               sums by the block's float scales; then store the tile (a lane = a weight row, so
//               the 32 lanes of a warp write 128 contiguous bytes of a row of Y)
//   warps 8-23  turn the raw blocks into the A operand (four threads a weight row, a K step each)
// The roles' register needs differ widely, so the warp groups trade registers (setmaxnreg).
// Every mbarrier wait is bounded; on a time-out the kernel records a code in the status
// word, skips what depends on the wait, frees its tensor memory and returns.
//
// Replaces d4_mm_id_iq2_xxs / d4_mm_id_q2_k (src/cuda/ds4f_mm.cu:229-257: mma.sync
// m16n8k16, 64x64 tiles) behind DK-FFN-ROUTED-CHUNK (src/cuda-ds4f-prefill.lisp:315-356).
#include <cuda.h>

#include "formats.cuh"
#include "iq2xxs_tables.cuh"
#include "quantdev.cuh"
#include "host.h"

namespace ill {

constexpr int MM_BM = 128;                             // rows of X a tile (the MMA's N)
constexpr int MM_BN = 128;                             // weight rows a tile (the MMA's M)
constexpr int MM_BK = 64;                              // K step: one 128-byte row of the swizzled X tile
constexpr int MM_RS = 3;                               // stages of the ring of raw weight blocks
constexpr int MM_XSC = 16;                             // blocks of X scales kept (the loader runs < 16 blocks ahead of the drain)
constexpr int MM_DR_WARPS = 4, MM_DQ_WARPS = 16, MM_LD_WARPS = 2;  // drain, dequantize, raw-load warps
// Registers a thread after the roles part: the four warps of TMA / MMA / raw loads give theirs up, the
// drain warps (a whole tile's row of 128 sums each) take them
constexpr int MM_REGS_AUX = 40, MM_REGS_DRAIN = 184, MM_REGS_DQ = 64;
constexpr int MM_THREADS = 32 * (2 + MM_LD_WARPS + MM_DR_WARPS + MM_DQ_WARPS);  // + the TMA warp and the MMA warp
constexpr uint32_t MM_TILE_BYTES = MM_BM * MM_BK * 2;  // 16 KB

struct MmParams {
  int ncols, nrows;            // K and N of every expert matrix
  int row_bytes;
  long long add, add2;         // a second matrix of every expert (gate and up in one launch) when Y2 is given
  const unsigned long long* ptrs;
  const unsigned* counts;
  const unsigned* bases;
  const float* xd;             // the activations' block scales, [token][K/256]
  const unsigned* map;         // token of each row of X (null: the row itself)
  const unsigned* ymap;        // row of Y each row of X is written to (null: the same row)
  const unsigned long long* ypeers;  // with YMAP: Y of every rank (peer memory); YMAP[place] = rank << 24 | row there
  long long total_rows;
  float* y;
  float* y2;
  long long y_stride;          // floats between rows of Y
  int ne;
  unsigned int* status;
  // a dense product (ill_mm_chunk): no tables on the device -- PTRS is null, the one "expert" is the matrix at
  // ONE_PTR with all ONE_COUNT rows of X; ACC: add into Y
  unsigned long long one_ptr;
  unsigned one_count;
  int acc;
};
// (DENSE is a template argument of the kernel, so that the experts' launches compile to what they were without it)
template <bool DENSE> __device__ __forceinline__ unsigned long long mm_ptr(const MmParams& p, int e) {
  if constexpr (DENSE) return p.one_ptr; else return p.ptrs[e];
}
template <bool DENSE> __device__ __forceinline__ int mm_count(const MmParams& p, int e) {
  if constexpr (DENSE) return (int)p.one_count; else return (int)p.counts[e];
}
template <bool DENSE> __device__ __forceinline__ int mm_base(const MmParams& p, int e) {
  if constexpr (DENSE) return 0; else return (int)p.bases[e];
}

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

// D[tmem] (+)= A[tmem] * B[smem]^T, 128 x N x 16, fp16 operands, fp32 accumulate.  A: 128 lanes x 8
// columns (two halves a column, K ascending); B: N rows of X, K-major.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// the same with A in shared memory (K-major, 128-byte swizzle)
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// 16-byte chunk C of row ROW of a K-major tile with the 128-byte swizzle
__device__ __forceinline__ void store_chunk(u8* tile, int row, int c, uint4 v) {
  *(uint4*)(tile + (row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4)) = v;
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
// this lane's 16 (4) words into 16 (4) consecutive columns of its tensor-memory lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3])
               : "memory");
}
// true in one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// two unsigned bytes (byte positions B0, B1 of V) as the halves 1024 + byte
__device__ __forceinline__ uint32_t bytes_to_h2_1024(uint32_t v, uint32_t sel) {
  return __byte_perm(v, 0x64646464u, sel);
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// the small integer N (twice, as two halves) without a conversion: 1024 + N has the bits 0x6400 | N
__device__ __forceinline__ uint32_t small_h2(uint32_t n) {
  uint32_t v = 0x64006400u | (n * 0x10001u);
  asm("add.rn.f16x2 %0, %0, %1;" : "+r"(v) : "r"(0xe400e400u));  // - 1024
  return v;
}

// pairs of fp32 in a 64-bit register, and the packed multiply / fused multiply-add of sm_100
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) { return pack2u(__float_as_uint(lo), __float_as_uint(hi)); }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// 4 bytes global -> shared, asynchronously (both addresses 4-byte aligned)
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {  // both 16-byte aligned
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// BAR gets one arrival (counted in its initial count) once this thread's earlier cp.async have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- the weights' integer parts, 32 at a time, as 16 words of two halves -----------------
// IQ2_XXS: one sub-block (IDX: four grid indices; AUX: four groups of seven signs, and the scale):
// the 32 integers grid * sign * (2 LS + 1) (at most 43 * 31: exact in fp16).  The block's float
// part is d / 8 (src/avx2.lisp:77-110 takes the products this way).  GRID points at this lane's copy
// of the grid as halves (16 bytes an entry, eight interleaved copies: entry e of copy c at [8 e + c],
// so the eight lanes of a 128-bit request's quarter never share a bank); SGN likewise at the table
// that gives, for the seven stored sign bits, the sign bits of the eight halves (the eighth sign is
// the parity of the seven: ksigns_iq2xs[i] = i | parity(i) << 7).
__device__ __forceinline__ void w_iq2xxs(uint32_t idx, uint32_t aux, const uint4* grid, const uint4* sgn, uint32_t* out) {
  const uint32_t s2 = small_h2(2 * (aux >> 28) + 1);
  uint4 g[4], m[4];
#pragma unroll
  for (int l = 0; l < 4; ++l) {
    g[l] = grid[8 * ((idx >> (8 * l)) & 0xff)];
    m[l] = sgn[8 * ((aux >> (7 * l)) & 127u)];
  }
#pragma unroll
  for (int l = 0; l < 4; ++l) {
    out[4 * l] = hmul2(g[l].x, s2) ^ m[l].x;
    out[4 * l + 1] = hmul2(g[l].y, s2) ^ m[l].y;
    out[4 * l + 2] = hmul2(g[l].z, s2) ^ m[l].z;
    out[4 * l + 3] = hmul2(g[l].w, s2) ^ m[l].w;
  }
}

// Q2_K: the 32 weights at shift K of a half's 32 quant bytes Q: (scale & 15) * q (at most 45), the
// scales SC_LO for the first sixteen and SC_HI for the rest (src/kquant.lisp:DEQUANTIZE-ROW-Q2-K order).
__device__ __forceinline__ void w_q2k(const uint32_t* q, int k, uint32_t sc_lo, uint32_t sc_hi, uint32_t* out) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t s2 = small_h2((half ? sc_hi : sc_lo) & 15u), bias = hmul2(s2, 0xe400e400u /* -1024 */);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t v = (q[4 * half + i] >> (2 * k)) & 0x03030303u;
      out[8 * half + 2 * i] = hfma2(bytes_to_h2_1024(v, 0x4140), s2, bias);
      out[8 * half + 2 * i + 1] = hfma2(bytes_to_h2_1024(v, 0x4342), s2, bias);
    }
  }
}
// Q2_K: eight mins (scale bytes M0, M1 >> 4) as four words
__device__ __forceinline__ void w_q2k_mins(uint32_t m0, uint32_t m1, uint32_t* v) {
  const uint32_t lo = (m0 >> 4) & 0x0f0f0f0fu, hi = (m1 >> 4) & 0x0f0f0f0fu;
  const uint32_t k1024 = 0xe400e400u;  // -1024 twice
  v[0] = bytes_to_h2_1024(lo, 0x4140); v[1] = bytes_to_h2_1024(lo, 0x4342);
  v[2] = bytes_to_h2_1024(hi, 0x4140); v[3] = bytes_to_h2_1024(hi, 0x4342);
#pragma unroll
  for (int i = 0; i < 4; ++i) asm("add.rn.f16x2 %0, %0, %1;" : "+r"(v[i]) : "r"(k1024));
}

// Per format.  A 256-wide block is four K steps; for Q2_K it also has a tile of the activations' sums
// of 16, multiplied with the mins (one K = 16 MMA into a second accumulator).
// Tensor memory, 512 columns: accumulators D[2] at 0 and 128 (a column = a row of X); then
//   IQ2_XXS  the A ring, 8 K steps x 32 columns, at 256
//   Q2_K     the mins' accumulator at 256; the A ring, 4 K steps, at 384 (the mins themselves, a
//   Q4_K     128 x 16 operand, go through two tiles in shared memory)
// Q4_K: byte I (0..11) of the block's packed scales and mins, held as the three words S
__device__ __forceinline__ uint32_t q4k_sb(const uint32_t* s, int i) { return (s[i >> 2] >> (8 * (i & 3))) & 0xffu; }
// get_scale_min_k4 (src/kquant.lisp:64-72): group J's 6-bit scale and min
__device__ __forceinline__ void q4k_scale_min(const uint32_t* s, int j, uint32_t& sc, uint32_t& mn) {
  if (j < 4) { sc = q4k_sb(s, j) & 63u; mn = q4k_sb(s, j + 4) & 63u; }
  else { sc = (q4k_sb(s, j + 4) & 0xFu) | ((q4k_sb(s, j - 4) >> 6) << 4); mn = (q4k_sb(s, j + 4) >> 4) | ((q4k_sb(s, j) >> 6) << 4); }
}
// Q4_K: 4 NW weights of a group -- the low (HI = 0) or high nibbles of the NW words of quant bytes Q -- times the
// group's scale: at most 15 * 63 = 945, exact in fp16 (the fused multiply-add rounds once)
template <int NW>
__device__ __forceinline__ void w_q4k(const uint32_t* q, int hi, uint32_t sc, uint32_t* out) {
  const uint32_t s2 = small_h2(sc), bias = hmul2(s2, 0xe400e400u /* -1024 */);
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    const uint32_t v = (q[i] >> (4 * hi)) & 0x0f0f0f0fu;
    out[2 * i] = hfma2(bytes_to_h2_1024(v, 0x4140), s2, bias);
    out[2 * i + 1] = hfma2(bytes_to_h2_1024(v, 0x4342), s2, bias);
  }
}
// Q4_K: four groups' mins, each twice (a group of 32 faces two of the activations' sums of 16), as four words
__device__ __forceinline__ void w_q4k_mins(const uint32_t* s, int g0, uint32_t* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t sc, mn;
    q4k_scale_min(s, g0 + i, sc, mn);
    v[i] = small_h2(mn);
  }
}

// N words starting BYTE_OFF bytes into the row's window RW (any 2-byte alignment of the offset is taken up by funnel shifts)
template <int N>
__device__ __forceinline__ void raw_words(const uint32_t* rw, uint32_t byte_off, uint32_t* out) {
  const uint32_t w0 = byte_off >> 2, sh = (byte_off & 3u) * 8u;
  uint32_t prev = rw[w0];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const uint32_t next = rw[w0 + i + 1];
    out[i] = __funnelshift_r(prev, next, sh);
    prev = next;
  }
}
// Q6_K: 16 weights of a K step -- the nibbles at shift 4 ODD of the four words QL, the 2-bit fields at shift QSH of the
// four words QH -- times their group's signed scale SC.  |SC * (q - 32)| reaches 4064 and fp16 holds only even
// integers above 2048, so the product goes to the tensor core in two exact parts: EVEN = (SC - SC % 2) * (q - 32), an
// even integer of at most 4096, and ODD = (SC % 2) * (q - 32); both are multiplied with the same activations into
// the same accumulator.
__device__ __forceinline__ void w_q6k(const uint32_t* ql, const uint32_t* qh, int odd, int qsh, int sc, uint32_t* even, uint32_t* oddp) {
  const int s0 = sc & 1;
  uint32_t s2 = small_h2((uint32_t)(sc - s0 + 128));
  asm("add.rn.f16x2 %0, %0, %1;" : "+r"(s2) : "r"(0xd800d800u));  // - 128
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t v = ((ql[i] >> (4 * odd)) & 0x0f0f0f0fu) | (((qh[i] >> qsh) & 0x03030303u) << 4);
    uint32_t a = bytes_to_h2_1024(v, 0x4140), b = bytes_to_h2_1024(v, 0x4342);
    asm("add.rn.f16x2 %0, %0, %1;" : "+r"(a) : "r"(0xe420e420u));  // - 1056: q - 32
    asm("add.rn.f16x2 %0, %0, %1;" : "+r"(b) : "r"(0xe420e420u));
    even[2 * i] = hmul2(a, s2);
    even[2 * i + 1] = hmul2(b, s2);
    oddp[2 * i] = s0 ? a : 0u;
    oddp[2 * i + 1] = s0 ? b : 0u;
  }
}

template <int FMT> struct MmGeom {
  static constexpr bool KM = FMT == ILL_Q2_K || FMT == ILL_Q4_K;  // formats with mins: a second, small product a block
  static constexpr int BB = FMT == ILL_Q2_K ? 84 : FMT == ILL_Q4_K ? 144 : FMT == ILL_Q6_K ? 210 : 66;
  static constexpr int NSLOT = KM || FMT == ILL_Q6_K ? 4 : 8;  // a multiple of four: a slot is always written by the same warps
  static constexpr int NX = FMT == ILL_Q4_K ? 5 : KM ? 6 : FMT == ILL_Q6_K ? 6 : 8;  // stages of the ring of X tiles = K steps in flight
  // A dequantizing warp waits for K step st - NSLOT on barrier (st - NSLOT) % NX; the barrier's next phase (K step
  // st - NSLOT + NX) must not be able to complete before that warp has passed, or the parity it waits for comes round again
  static_assert(NX >= NSLOT, "the ring of K-step barriers must be at least as long as the ring of A slots");
  static constexpr int NE = KM ? 4 : 0;     // Q2_K, Q4_K: two tiles of X's sums of 16, two of the mins
  static constexpr uint32_t A_COL = KM ? 384 : 256, DM_COL = 256;
  static constexpr uint32_t SLOTW = FMT == ILL_Q6_K ? 64 : 32;  // columns of an A slot (Q6_K: the even and the odd part)
  // A row's raw block reaches shared memory as the WIN bytes from the 16-byte boundary at or before it,
  // PITCH bytes apart (Q4_K: blocks of 144 bytes in rows that the launcher wants 16-byte aligned)
  static constexpr uint32_t WIN = FMT == ILL_Q2_K ? 96 : FMT == ILL_Q4_K ? 144 : FMT == ILL_Q6_K ? 224 : 80;
  static constexpr uint32_t PITCH = FMT == ILL_Q2_K ? 112 : FMT == ILL_Q4_K ? 160 : FMT == ILL_Q6_K ? 240 : 80;
  static constexpr uint32_t RAW_BYTES = 128 * PITCH;
  static constexpr size_t SMEM = (size_t)(NX + NE) * MM_TILE_BYTES + MM_RS * RAW_BYTES + 16 /* a word past the last row is read */ +
                                 512 /* barriers */ + 4 * 256 * 4 /* weight scales */ + MM_XSC * 128 * 4 /* X scales */ +
                                 2304 /* experts' first tiles */ + (FMT == ILL_IQ2_XXS ? 8 * 4096 + 8 * 2048 : 0) /* tables */ +
                                 1024 /* alignment */;
};

template <int FMT, bool DENSE>
__global__ void __launch_bounds__(MM_THREADS) mm_id_kernel(const __grid_constant__ CUtensorMap xmap,
                                                           const __grid_constant__ CUtensorMap emap, const MmParams p) {
  typedef MmGeom<FMT> G;
  constexpr int BB = G::BB, NSLOT = G::NSLOT, NX = G::NX;
  constexpr bool KM = G::KM;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ __align__(1024) u8 smem_raw[];
  // [X ring][Q2_K: sums of 16 x 2, mins x 2] (each tile 1024-byte aligned, as the 128-byte swizzle needs), the
  // ring of raw blocks, then barriers, scales, tables
  u8* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  u8* x_tiles = smem;
  u8* e_tiles = smem + NX * MM_TILE_BYTES;       // Q2_K: the sums of 16 of the tile's rows of X
  u8* m_tiles = e_tiles + 2 * MM_TILE_BYTES;     // Q2_K: the mins
  uint32_t* raw = (uint32_t*)(smem + (NX + G::NE) * MM_TILE_BYTES);
  u8* tail = (u8*)raw + MM_RS * G::RAW_BYTES + 16;
  // K step st of this CTA (four a block, counted over all its tiles) uses X stage st % NX, A slot st % NSLOT
  // and the pair of barriers st % NX
  uint64_t* kfull = (uint64_t*)tail;             // [NX] the X tile landed (TMA) and the K step of A is in tensor memory (4 warps)
  uint64_t* kempty = kfull + NX;                 // [NX] the MMAs of the K step completed
  uint64_t* mfull = kempty + NX;                 // [2] Q2_K: the block's sums of 16 landed and its mins are in their tile (8 warps)
  uint64_t* mempty = mfull + 2;                  // [2] the MMA that read them completed
  uint64_t* raw_full = mempty + 2;               // [RS] the raw-load lanes' copies landed
  uint64_t* raw_empty = raw_full + MM_RS;        // [RS] the dequantizing warps have read the stage
  uint64_t* acc_full = raw_empty + MM_RS;        // [2] a block's MMAs completed
  uint64_t* acc_free = acc_full + 2;             // [2] the drain warps read the buffer
  uint64_t* accm_free = acc_free + 2;            // [1] Q2_K: the drain warps read the mins' accumulator
  uint32_t* tmem_slot = (uint32_t*)(accm_free + 1);
  float* wsc = (float*)(tail + 512);             // [4 blocks in flight][2: d, dmin][128 weight rows]
  float* xsc = wsc + 4 * 256;                    // [XSC blocks][128 rows of X] the activations' block scales
  int* tile_first = (int*)(xsc + MM_XSC * 128);  // [ne + 1] first row tile of each expert; the total
  uint4* iq_grid = (uint4*)((u8*)tile_first + 2304);  // [256 entries][8 copies] the grid as halves
  uint4* iq_sgn = iq_grid + 8 * 256;             // [128 entries][8 copies] sign bits of the eight halves

  // the warp number through a shuffle: the compiler then knows that the role branches are warp-uniform
  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;

  // ---- once per CTA: the experts' row tiles counted (first tile of each expert, in shared memory),
  // barriers, tables, tensor memory.  The CTA then walks tiles blockIdx.x, + gridDim.x, ...
  if (warp == 0) {
    int before = 0;
    for (int e0 = 0; e0 < p.ne; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < p.ne ? mm_count<DENSE>(p, e) : 0;
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
    for (int s = 0; s < NX; ++s) { mbar_init(&kfull[s], 1 + MM_DQ_WARPS / 4); mbar_init(&kempty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&mfull[s], 1 + MM_DQ_WARPS / 2); mbar_init(&mempty[s], 1); }
    for (int s = 0; s < MM_RS; ++s) { mbar_init(&raw_full[s], 32 * MM_LD_WARPS); mbar_init(&raw_empty[s], MM_DQ_WARPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_free[b], MM_DR_WARPS); }
    mbar_init(accm_free, MM_DR_WARPS);
    mbar_fence_init();
  }
  if (FMT == ILL_IQ2_XXS) {
    for (int i = tid; i < 8 * 256; i += MM_THREADS) {
      const uint64_t g = ill_iq2xxs_grid[i >> 3];
      uint32_t h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __half2 hh = __floats2half2_rn((float)((g >> (16 * k)) & 0xff), (float)((g >> (16 * k + 8)) & 0xff));
        h[k] = *(const uint32_t*)&hh;
      }
      iq_grid[i] = make_uint4(h[0], h[1], h[2], h[3]);
    }
    for (int i = tid; i < 8 * 128; i += MM_THREADS) {
      const uint32_t s7 = (uint32_t)i >> 3, sg = s7 | ((__popc(s7) & 1u) << 7);
      uint32_t h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) h[k] = (((sg >> (2 * k)) & 1u) << 15) | (((sg >> (2 * k + 1)) & 1u) << 31);
      iq_sgn[i] = make_uint4(h[0], h[1], h[2], h[3]);
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);

  const int nkb = p.ncols / 256;
  const int ntn1 = (p.nrows + MM_BN - 1) / MM_BN;
  const int ntn = p.y2 ? 2 * ntn1 : ntn1;     // the second matrix's weight-row tiles follow the first's
  const int ntiles = tile_first[p.ne] * ntn;  // weight-row tiles vary fastest: CTAs running together share X
  bool ok = true;

  // tile index -> expert, first row of X, valid rows, weight-row tile
  // (NT >= ntn1: tile NT - ntn1 of the second matrix)
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
    row0 = mm_base<DENSE>(p, lo) + m_in * MM_BM;
    nvalid = min(MM_BM, mm_count<DENSE>(p, lo) - m_in * MM_BM);
    // counts / bases come from the caller: a tile never reaches past the TOTAL_ROWS rows X and Y have
    if ((long long)row0 >= p.total_rows) { row0 = 0; nvalid = 0; }
    else nvalid = min(nvalid, (int)(p.total_rows - row0));
  };

  if (warp < 2 + MM_LD_WARPS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(MM_REGS_AUX));
  if (warp == 0) {
    // ---- TMA producer of the X tiles
    if (lane == 0) {
      int g_st = 0, g_kb = 0;  // K steps and blocks issued so far by this CTA
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int expert, row0, nvalid, nt;
        locate(tile, expert, row0, nvalid, nt);
        for (int kb = 0; kb < nkb && ok; ++kb, ++g_kb) {
          for (int j = 0; j < 4; ++j, ++g_st) {
            const int s = g_st % NX;
            if (g_st >= NX && !mbar_wait(&kempty[s], (uint32_t)(g_st / NX - 1) & 1u, p.status, ST_MM_WAIT_EMPTY, 0)) { ok = false; break; }
            mbar_expect_tx(&kfull[s], MM_TILE_BYTES);
            tma_load_2d(x_tiles + s * MM_TILE_BYTES, &xmap, kb * 256 + j * MM_BK, row0, &kfull[s]);
          }
          if (KM && ok) {
            const int sm = g_kb & 1;
            if (g_kb >= 2 && !mbar_wait(&mempty[sm], (uint32_t)((g_kb >> 1) - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 3, 0)) { ok = false; break; }
            mbar_expect_tx(&mfull[sm], MM_TILE_BYTES);
            tma_load_2d(e_tiles + sm * MM_TILE_BYTES, &emap, kb * MM_BK, row0, &mfull[sm]);  // the sums of 16
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp walks the loop (so that addresses and descriptors stay in uniform
    // registers) and one elected lane issues
    {
      int g_st = 0, g_kb = 0;  // K steps and blocks consumed so far by this CTA
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int expert, row0, nvalid, nt;
        locate(tile, expert, row0, nvalid, nt);
        nvalid = __shfl_sync(0xffffffffu, nvalid, 0);
        // fp32 accumulate, fp16 A and B, both K-major, M = 128 weight rows, N = the tile's rows of X up to 16
        const int nmma = max(16, (nvalid + 15) & ~15);
        const uint32_t idesc = (1u << 4) | ((uint32_t)(nmma >> 3) << 17) | ((uint32_t)(MM_BN >> 4) << 24);
        for (int kb = 0; kb < nkb && ok; ++kb, ++g_kb) {
          const int b = g_kb & 1;
          if (g_kb >= 2) ok = __all_sync(0xffffffffu, mbar_wait(&acc_free[b], (uint32_t)(g_kb / 2 - 1) & 1u, p.status, ST_MM_WAIT_EPI));
          if (!ok) break;
          const uint32_t d1 = tmem_base + (uint32_t)(b * MM_BM);
          for (int j = 0; j < 4; ++j, ++g_st) {
            const int s = g_st % NX, slot = g_st % NSLOT;
            ok = __all_sync(0xffffffffu, mbar_wait(&kfull[s], (uint32_t)(g_st / NX) & 1u, p.status, ST_MM_WAIT_FULL));
            if (!ok) break;
            tc_fence_after();
            const uint64_t xdsc = umma_desc(x_tiles + s * MM_TILE_BYTES);
            const uint32_t a0 = tmem_base + G::A_COL + G::SLOTW * slot;
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < MM_BK / 16; ++k)  // 16 of K: 8 columns of A, 32 bytes inside X's swizzle atom
                umma_f16_ts(d1, a0 + 8 * k, xdsc + 2 * k, idesc, (j | k) ? 1u : 0u);
              if constexpr (FMT == ILL_Q6_K) {  // the weights' odd parts against the same activations
#pragma unroll
                for (int k = 0; k < MM_BK / 16; ++k) umma_f16_ts(d1, a0 + 32 + 8 * k, xdsc + 2 * k, idesc, 1u);
              }
              umma_commit(&kempty[s]);  // the X stage and the A slot are free when these MMAs are done
            }
            __syncwarp();
          }
          if (!ok) break;
          if constexpr (KM) {
            const int sm = g_kb & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&mfull[sm], (uint32_t)(g_kb >> 1) & 1u, p.status, ST_MM_WAIT_FULL + 3) &&
                                             (g_kb < 1 || mbar_wait(accm_free, (uint32_t)(g_kb - 1) & 1u, p.status, ST_MM_WAIT_EPI + 2)));
            if (!ok) break;
            tc_fence_after();
            // mins x sums of 16: one K = 16 product into the mins' accumulator
            if (elect_one()) {
              umma_f16_ss(tmem_base + G::DM_COL, umma_desc(m_tiles + sm * MM_TILE_BYTES), umma_desc(e_tiles + sm * MM_TILE_BYTES), idesc, 0u);
              umma_commit(&mempty[sm]);
            }
            __syncwarp();
          }
          if (elect_one()) umma_commit(&acc_full[b]);
          __syncwarp();
        }
      }
    }
  } else if (warp < 2 + MM_LD_WARPS) {
    // ---- warps 2, 3 bring each block's raw bytes (for every weight row the 16-byte-aligned window
    // around the row's block, 16 bytes a lane at a time: a warp's requests touch six or seven rows) and
    // the block's scale of each of the tile's rows of X into shared memory
    const int L = (warp - 2) * 32 + lane;
    constexpr int NL = 32 * MM_LD_WARPS, CPR = G::WIN / 16;  // chunks of a row's window
    int g_kb = 0;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      int expert, row0, nvalid, nt;
      locate(tile, expert, row0, nvalid, nt);
      const bool second = nt >= ntn1;
      if (second) nt -= ntn1;
      const u8* wbase = (const u8*)(uintptr_t)mm_ptr<DENSE>(p, expert) + (second ? p.add2 : p.add) + (long long)nt * MM_BN * p.row_bytes;
      const int rows_here = min(MM_BN, p.nrows - nt * MM_BN);
      // the tokens of the tile's rows L, L + NL of X (a row past the tile's last takes the first row's)
      const float* xdp[128 / NL];
#pragma unroll
      for (int i = 0; i < 128 / NL; ++i) {
        const long long place = (long long)row0 + (L + i * NL < nvalid ? L + i * NL : 0);
        const long long tok = p.map ? (long long)p.map[place] : place;
        xdp[i] = p.xd + tok * nkb;
      }
      for (int kb = 0; kb < nkb; ++kb, ++g_kb) {
        const int s = g_kb % MM_RS, use = g_kb / MM_RS;
        bool w_ok = true;
        if (use > 0) w_ok = mbar_wait(&raw_empty[s], (uint32_t)(use - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 2, 200);
        if (!__all_sync(0xffffffffu, w_ok)) { ok = false; break; }
#pragma unroll
        for (int i = 0; i < 128 / NL; ++i) {
          cp_async4(xsc + (g_kb % MM_XSC) * 128 + L + i * NL, xdp[i] + kb);

        }
        u8* dst = (u8*)raw + s * G::RAW_BYTES;
#pragma unroll 4
        for (int c = L; c < 128 * CPR; c += NL) {
          const int row = c / CPR, ch = c - row * CPR;
          if (row < rows_here) {
            const uintptr_t blk = (uintptr_t)(wbase + (long long)row * p.row_bytes + kb * BB);
            cp_async16(dst + row * G::PITCH + 16 * ch, (const void*)((blk & ~(uintptr_t)15) + 16 * ch));
          }
        }
        cp_async_arrive(&raw_full[s]);
      }
    }
    cp_async_wait_all();
  } else if (warp < 2 + MM_LD_WARPS + MM_DR_WARPS) {
    // ---- warps 4..7 drain the accumulators block by block, scaling each block's integer sums by the
    // block's float scales, and store the finished tile.  A warp reads the 32 tensor-memory lanes
    // its number gives it (warp % 4: 32 weight rows) and all the columns (rows of X).
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(MM_REGS_DRAIN));
    const int q = warp & 3;
    const int m = q * 32 + lane;                   // accumulator lane = weight row in the tile
    int d_kb = 0;                                  // blocks drained so far by this CTA
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      int expert, row0, nvalid, nt;
      locate(tile, expert, row0, nvalid, nt);
      uint64_t out[64];  // pairs of fp32: this weight row against the tile's 128 rows of X
#pragma unroll
      for (int i = 0; i < 64; ++i) out[i] = 0ull;
      for (int kb = 0; kb < nkb; ++kb, ++d_kb) {
        const int b = d_kb & 1;
        const bool e_ok = mbar_wait(&acc_full[b], (uint32_t)(d_kb / 2) & 1u, p.status, ST_MM_WAIT_ACC, 0);
        if (!__all_sync(0xffffffffu, e_ok)) { ok = false; break; }
        tc_fence_after();
        // Two fp32 at a time (fma.rn.f32x2: each half rounds as the scalar instruction does).
        // IQ2XXS-DOT-AVX2 (src/avx2.lisp:107-110): total += d * y.d * sum, the 1/8 at the end;
        // Q2K-DOT-AVX2 (src/avx2.lisp:147-150): y.d * d * sum - y.d * dmin * mins
        const float dw = wsc[(d_kb & 3) * 256 + m];
        const uint64_t dw2 = pack2(dw, dw);
        const float* xs = xsc + (d_kb % MM_XSC) * 128;
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16);
        if constexpr (KM) {
          const float dm = -wsc[(d_kb & 3) * 256 + 128 + m];
          const uint64_t dm2 = pack2(dm, dm);
#pragma unroll
          for (int part = 0; part < 4; ++part) {
            if (32 * part < nvalid) {  // columns past the tile's last row of X were not computed
              uint32_t v[32];
              tmem_ld32(t0 + G::DM_COL + 32 * part, v);
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const ulonglong2 dx = *(const ulonglong2*)(xs + 32 * part + i);
                uint64_t* o = out + (32 * part + i) / 2;
                o[0] = fma2(mul2(dx.x, dm2), pack2u(v[i], v[i + 1]), o[0]);
                o[1] = fma2(mul2(dx.y, dm2), pack2u(v[i + 2], v[i + 3]), o[1]);
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(accm_free);
        }
#pragma unroll
        for (int part = 0; part < 4; ++part) {
          if (32 * part < nvalid) {
            uint32_t v[32];
            tmem_ld32(t0 + b * MM_BM + 32 * part, v);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const ulonglong2 dx = *(const ulonglong2*)(xs + 32 * part + i);
              uint64_t* o = out + (32 * part + i) / 2;
              o[0] = fma2(mul2(dw2, dx.x), pack2u(v[i], v[i + 1]), o[0]);
              o[1] = fma2(mul2(dw2, dx.y), pack2u(v[i + 2], v[i + 3]), o[1]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_free[b]);
      }
      const bool second = nt >= ntn1;
      if (second) nt -= ntn1;
      const int n = nt * MM_BN + m;
      if (ok && n < p.nrows) {
        const float fin = FMT == ILL_IQ2_XXS ? 0.125f : 1.0f;
        float* ycol = (second ? p.y2 : p.y) + n;
        const unsigned ys = (unsigned)p.y_stride;
        if (p.ymap) {
          const unsigned* ym = p.ymap + row0;
#pragma unroll
          for (int i0 = 0; i0 < 128; i0 += 8) {
            if (i0 < nvalid) {
              unsigned yr[8];  // the rows first, then the stores: a load does not wait for the store before it
#pragma unroll
              for (int i = 0; i < 8; ++i) yr[i] = i0 + i < nvalid ? __ldg(ym + i0 + i) : 0u;
              if (p.ypeers) {
                // the combine of an expert-parallel chunk, fused: the row goes straight into the memory of the
                // rank that owns its token (a plain store over NVLink), tile by tile as the products finish
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (i0 + i < nvalid) {
                    float* dst = (float*)(uintptr_t)__ldg(p.ypeers + (yr[i] >> 24)) + (size_t)(yr[i] & 0xffffffu) * ys + n;
                    *dst = __uint_as_float((uint32_t)(out[(i0 + i) >> 1] >> (32 * (i & 1)))) * fin;
                  }
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (i0 + i < nvalid)
                    ycol[(size_t)yr[i] * ys] = __uint_as_float((uint32_t)(out[(i0 + i) >> 1] >> (32 * (i & 1)))) * fin;
              }
            }
          }
        } else {
          ycol += (size_t)row0 * ys;
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            if (i < nvalid) {
              const float v = __uint_as_float((uint32_t)(out[i >> 1] >> (32 * (i & 1)))) * fin;
              if constexpr (DENSE) *ycol = p.acc ? *ycol + v : v;
              else *ycol = v;
            }
            ycol += ys;
          }
        }
      }
    }
  } else {
    // ---- warps 8..23 turn the raw blocks into the A operand in tensor memory: thread (row, j) makes K
    // step j of its weight row in every block, so the tensor core can start on a block's first K
    // step while the others are still being made.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(MM_REGS_DQ));
    const int t = tid - 32 * (2 + MM_LD_WARPS + MM_DR_WARPS);  // 0..511
    const int row = t & 127, j = t >> 7;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's lanes: rows (warp % 4) * 32 ..
    const uint4* grid = iq_grid + (lane & 7);
    const uint4* sgn = iq_sgn + (lane & 7);
    int g_kb = 0;                                  // blocks produced so far by this CTA

    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      int expert, row0, nvalid, nt;
      locate(tile, expert, row0, nvalid, nt);
      const bool second = nt >= ntn1;
      if (second) nt -= ntn1;
      const int n = nt * MM_BN + row;
      const bool has_row = n < p.nrows;
      // the low bits of the row's address: where its blocks start inside their first word
      const uint32_t rowlow = (uint32_t)(mm_ptr<DENSE>(p, expert) + (unsigned long long)(second ? p.add2 : p.add) + (unsigned long long)n * p.row_bytes);
      for (int kb = 0; kb < nkb && ok; ++kb, ++g_kb) {
        const int rs = g_kb % MM_RS;
        const bool r_ok = mbar_wait(&raw_full[rs], (uint32_t)(g_kb / MM_RS) & 1u, p.status, ST_MM_WAIT_FULL + 2, 50);
        if (!__all_sync(0xffffffffu, r_ok)) { ok = false; break; }
        // this thread's words of the block (it starts O16 bytes into the row's window), then the raw
        // stage is free again
        const uint32_t o16 = (rowlow + (uint32_t)kb * BB) & 15u;
        const uint32_t* rw = raw + rs * (G::RAW_BYTES / 4) + row * (G::PITCH / 4);
        uint32_t w[KM ? 8 : 4], sc4 = 0, m0 = 0, m1 = 0, dd = 0, s12[3] = {0, 0, 0};
#pragma unroll
        for (int i = 0; i < (KM ? 8 : 4); ++i) w[i] = 0;
        if (has_row) {
          if constexpr (FMT == ILL_IQ2_XXS) {
            dd = (rw[o16 >> 2] >> (8 * (o16 & 2u))) & 0xffffu;
            const uint32_t o = o16 + 2 + 16 * j, w0 = o >> 2, sh = (o & 3u) * 8u;
            uint32_t prev = rw[w0];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t next = rw[w0 + i + 1];
              w[i] = __funnelshift_r(prev, next, sh);
              prev = next;
            }
          } else if constexpr (FMT == ILL_Q6_K) {
            // the block's scale and K step j's four group scales; the quants are read as they are unpacked (below)
            dd = (rw[(o16 + 208) >> 2] >> (8 * ((o16 + 208) & 2u))) & 0xffffu;
            raw_words<1>(rw, o16 + 192 + 4 * j, &sc4);
          } else if constexpr (FMT == ILL_Q4_K) {
            // K step j: the block's chunk j of 32 quant bytes (groups 2j and 2j + 1); the twelve bytes of scales and mins
            const uint32_t* bw = rw + (o16 >> 2);  // a Q4_K block is 16-byte aligned
            dd = bw[0];
            s12[0] = bw[1]; s12[1] = bw[2]; s12[2] = bw[3];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = bw[4 + 8 * j + i];
          } else {
            // K step j: half j / 2 of the block's quants at shifts 2 (j % 2) and 2 (j % 2) + 1; its four scale bytes
            const uint32_t* bw = rw + (o16 >> 2);  // a Q2_K block is 4-byte aligned
            sc4 = bw[j];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = bw[4 + 8 * (j >> 1) + i];
            if (j < 2) { m0 = bw[2 * j]; m1 = bw[2 * j + 1]; }
            dd = bw[20];
          }
        }
        __syncwarp();
        if (FMT != ILL_Q6_K && lane == 0) mbar_arrive(&raw_empty[rs]);  // (Q6_K reads its quants from the stage while unpacking)
        {
          // the slot's last K step was st - NSLOT: its MMAs must be done
          const int st = 4 * g_kb + j, slot = st % NSLOT, sp = st - NSLOT;
          bool w_ok = true;
          if (sp >= 0) w_ok = mbar_wait(&kempty[sp % NX], (uint32_t)(sp / NX) & 1u, p.status, ST_MM_WAIT_EMPTY + 1, 50);
          if (!__all_sync(0xffffffffu, w_ok)) { ok = false; break; }
          tc_fence_after();
          if (j == 0) {
            // The drain of four blocks back is over: the MMAs that freed this slot were issued after it.
            wsc[(g_kb & 3) * 256 + row] = h2f(dd & 0xffff);
            if (KM) wsc[(g_kb & 3) * 256 + 128 + row] = h2f(dd >> 16);
          }
          const uint32_t a0 = lane_base + G::A_COL + G::SLOTW * slot;
#pragma unroll
          for (int sb = 0; sb < 2; ++sb) {  // 32 weights = 16 columns at a time
            uint32_t v[16];
            if constexpr (FMT == ILL_IQ2_XXS) {
              w_iq2xxs(w[2 * sb], w[2 * sb + 1], grid, sgn, v);
              if (!has_row) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0;
              }
            } else if constexpr (FMT == ILL_Q6_K) {
              // K step j: half j / 2 of the block; columns 32 sb .. of the step are the nibbles at shift 4 (j % 2) of
              // ql[32 sb ..] with the 2-bit fields at shift 2 (2 (j % 2) + sb) of qh; sixteen weights (a group) at a time
#pragma unroll
              for (int hf = 0; hf < 2; ++hf) {
                uint32_t ev[8], od[8];
                if (has_row) {
                  uint32_t ql[4], qh[4];
                  raw_words<4>(rw, o16 + 64 * (j >> 1) + 32 * sb + 16 * hf, ql);
                  raw_words<4>(rw, o16 + 128 + 32 * (j >> 1) + 16 * hf, qh);
                  w_q6k(ql, qh, j & 1, 2 * (2 * (j & 1) + sb), (int)(signed char)((sc4 >> (16 * sb + 8 * hf)) & 0xffu), ev, od);
                } else {
#pragma unroll
                  for (int i = 0; i < 8; ++i) ev[i] = od[i] = 0;
                }
                tmem_st8(a0 + 16 * sb + 8 * hf, ev);
                tmem_st8(a0 + 32 + 16 * sb + 8 * hf, od);
              }
            } else if constexpr (FMT == ILL_Q4_K) {
              uint32_t sc, mn;
              q4k_scale_min(s12, 2 * j + sb, sc, mn);
#pragma unroll
              for (int hf = 0; hf < 2; ++hf) {  // sixteen weights at a time: fewer live registers than all 32
                uint32_t v8[8];
                w_q4k<4>(w + 4 * hf, sb, sc, v8);
                tmem_st8(a0 + 16 * sb + 8 * hf, v8);
              }
            } else {
              w_q2k(w, 2 * (j & 1) + sb, sc4 >> (16 * sb), sc4 >> (16 * sb + 8), v);
            }
            if constexpr (FMT != ILL_Q6_K && FMT != ILL_Q4_K) tmem_st16(a0 + 16 * sb, v);
          }
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&kfull[st % NX]);
          if (FMT == ILL_Q6_K && lane == 0) mbar_arrive(&raw_empty[rs]);
        }
        if constexpr (KM) {
          if (j < 2) {  // warp-uniform: the eight warps of K steps 0 and 1 also make the mins
            const int sm = g_kb & 1;
            bool w_ok = true;
            if (g_kb >= 2) w_ok = mbar_wait(&mempty[sm], (uint32_t)((g_kb >> 1) - 1) & 1u, p.status, ST_MM_WAIT_EMPTY + 3, 50);
            if (!__all_sync(0xffffffffu, w_ok)) { ok = false; break; }
            uint32_t v[4];
            // half j's eight mins: K = 8j .. 8j + 7 of the 16, chunk j of the row (Q4_K: groups 4j .. 4j + 3, each twice)
            if constexpr (FMT == ILL_Q4_K) w_q4k_mins(s12, 4 * j, v);
            else w_q2k_mins(m0, m1, v);
            store_chunk(m_tiles + sm * MM_TILE_BYTES, row, j, make_uint4(v[0], v[1], v[2], v[3]));
            fence_async_smem();  // the tensor core reads the tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&mfull[sm]);
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
// Row t's quants are at XQ + t * XQ_STRIDE bytes and its sums at BSUMS + t * BS_STRIDE bytes.  With XD_OUT,
// the row also carries its block scales (SC + t * XQ_STRIDE) and a weight (WT + t * XQ_STRIDE), copied
// to XD_OUT[place, kb] and W_OUT[place]: the rows of an expert-parallel exchange, unpacked.
__global__ void __launch_bounds__(256) act_f16_kernel(long long rows, int cols, const u8* __restrict__ xq, long long xq_stride,
                                                      const u8* __restrict__ bsums, long long bs_stride,
                                                      const unsigned* __restrict__ map, __half* __restrict__ xh,
                                                      __half* __restrict__ xe, const u8* __restrict__ sc,
                                                      const u8* __restrict__ wt, float* __restrict__ xd_out,
                                                      float* __restrict__ w_out, const unsigned* __restrict__ rows_dev) {
  pdl_launch_dependents();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread: 16 values
  const int per_row = cols / 16;
  if (gid >= rows * per_row) return;
  const long long place = gid / per_row;
  if (rows_dev && place >= (long long)*rows_dev) return;  // the rows in use, known on the device only
  const int j = (int)(gid - place * per_row);
  const long long t = map ? (long long)map[place] : place;
  const uint4 q = *(const uint4*)(xq + t * xq_stride + 16 * j);
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
    e[g] = __float2half_rn((float)((const int16_t*)(bsums + t * bs_stride))[j]);
    e[16 + 3 * g] = __float2half_rn(0.0f);
    e[16 + 3 * g + 1] = __float2half_rn(0.0f);
    e[16 + 3 * g + 2] = __float2half_rn(0.0f);
  }
  if (xd_out) {
    if (j < cols / 256) xd_out[place * (cols / 256) + j] = ((const float*)(sc + t * xq_stride))[j];
    if (j == per_row - 1) w_out[place] = *(const float*)(wt + t * xq_stride);
  }
}

// A row of an expert-parallel exchange: the token's Q8_K form and its routing weight in one piece,
//   [cols int8 quants][cols/256 float scales][cols/16 int16 sums][float weight][pad to 16 bytes]
// PACKED[place] from token MAP[place]'s quantized activations and W[place].  One block a row.
__global__ void __launch_bounds__(128) ep_pack_kernel(int cols, long long row_bytes, const uint32_t* __restrict__ xq,
                                                      const uint32_t* __restrict__ xs, const uint32_t* __restrict__ xsum,
                                                      const uint32_t* __restrict__ w, const unsigned* __restrict__ map,
                                                      uint32_t* __restrict__ packed) {
  pdl_launch_dependents();
  pdl_wait();
  const long long place = blockIdx.x;
  const long long t = map[place];
  const int nq = cols / 4, ns = cols / 256, nb = cols / 32;  // words of quants, scales, sums
  uint32_t* dst = packed + place * (row_bytes / 4);
  for (int i = threadIdx.x; i < nq + ns + nb + 1; i += blockDim.x) {
    uint32_t v;
    if (i < nq) v = xq[t * nq + i];
    else if (i < nq + ns) v = xs[t * ns + (i - nq)];
    else if (i < nq + ns + nb) v = xsum[t * nb + (i - nq - ns)];
    else v = w[place];
    dst[i] = v;
  }
}

// ep_pack_kernel for exchanges of a fixed size: rank g's rows go to slab g of PACKED, CAP rows a slab, in the
// order of their places; PSLOT[place] = the row's slot (g * cap + index in the slab).  BASES[e] = first place
// of expert e on this rank (ill_moe_group), so destination g's rows are places [bases[g * per], bases[(g + 1) *
// per]).  A slab that would overflow sets *OVERFLOW and drops the rows past CAP.
__global__ void __launch_bounds__(128) ep_pack_cap_kernel(int cols, long long row_bytes, const uint32_t* __restrict__ xq,
                                                          const uint32_t* __restrict__ xs, const uint32_t* __restrict__ xsum,
                                                          const uint32_t* __restrict__ w, const unsigned* __restrict__ map,
                                                          const unsigned* __restrict__ bases, int per, int world, int cap,
                                                          long long rows, uint32_t* __restrict__ packed,
                                                          unsigned* __restrict__ pslot, unsigned* __restrict__ overflow,
                                                          const unsigned long long* __restrict__ peers, int rank) {
  pdl_launch_dependents();
  pdl_wait();
  const long long place = blockIdx.x;
  __shared__ long long slot_s;
  __shared__ int dest_s;
  if (threadIdx.x == 0) {
    int g = 0;
    while (g + 1 < world && (long long)bases[(g + 1) * per] <= place) ++g;
    const long long idx = place - (long long)bases[g * per];
    dest_s = g;
    if (idx >= cap) { atomicOr(overflow, 1u); slot_s = -1; pslot[place] = 0; }
    else { slot_s = (long long)g * cap + idx; pslot[place] = (unsigned)slot_s; }
  }
  __syncthreads();
  long long slot = slot_s;
  if (slot < 0) return;
  if (peers) {
    // the dispatch without a collective: the row is stored into slab RANK of the receiving rank's buffer
    packed = (uint32_t*)(uintptr_t)peers[dest_s];
    slot = (long long)rank * cap + (slot - (long long)dest_s * cap);
  }
  const long long t = map[place];
  const int nq = cols / 4, ns = cols / 256, nb = cols / 32;  // words of quants, scales, sums
  uint32_t* dst = packed + slot * (row_bytes / 4);
  // the quants 16 bytes at a time (a token's quants and a packed row both start on 16-byte boundaries), the rest by words
  for (int i = threadIdx.x; i < nq / 4; i += blockDim.x) ((uint4*)dst)[i] = ((const uint4*)(xq + t * nq))[i];
  for (int i = nq + threadIdx.x; i < nq + ns + nb + 1; i += blockDim.x) {
    uint32_t v;
    if (i < nq + ns) v = xs[t * ns + (i - nq)];
    else if (i < nq + ns + nb) v = xsum[t * nb + (i - nq - ns)];
    else v = w[place];
    dst[i] = v;
  }
}

// The whole dispatch of an expert-parallel chunk in one launch: block T quantizes token T's activations once (Q8_K,
// the arithmetic of quant_q8_k_kernel: the same bits) into a packed row in shared memory and stores it, for each of
// the token's NU slots, into slab RANK of that expert's rank (peer memory) with the slot's weight appended -- the
// quantized token never passes through this rank's memory, and what ep_pack_cap_kernel, quant_q8_k_kernel and
// ep_put_counts_kernel do in three launches is done in one; the first blocks also store this rank's rows-per-expert
// into row RANK of every rank's table.  A slab that would overflow raises *OVERFLOW to EPOCH (never cleared: the
// chunk with that number overflowed) and drops the rows past CAP.
constexpr int EP_MAX_NU = 32;
__global__ void __launch_bounds__(128) ep_dispatch_kernel(int cols, int nu, long long row_bytes, const float* __restrict__ x,
                                                          const uint32_t* __restrict__ w, const unsigned* __restrict__ smap,
                                                          const unsigned* __restrict__ bases, const unsigned* __restrict__ counts,
                                                          int per, int world, int cap, unsigned* __restrict__ pslot,
                                                          unsigned* __restrict__ overflow, unsigned epoch,
                                                          const unsigned long long* __restrict__ peers_rows,
                                                          const unsigned long long* __restrict__ peers_rc, int rank) {
  extern __shared__ __align__(16) u8 srow[];  // the token's packed row (without the weight)
  __shared__ unsigned long long dst_s[EP_MAX_NU];  // where slot s's row goes (0: dropped)
  __shared__ uint32_t w_s[EP_MAX_NU];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  {
    const int i = blockIdx.x * 128 + tid;
    if (i < world * per) ((unsigned*)(uintptr_t)peers_rc[i / per])[rank * per + (i % per)] = counts[i];
  }
  const long long t = blockIdx.x;
  if (tid < nu) {
    const long long place = smap[t * nu + tid];
    int g = 0;
    while (g + 1 < world && (long long)bases[(g + 1) * per] <= place) ++g;
    const long long idx = place - (long long)bases[g * per];
    if (idx >= cap) { atomicMax(overflow, epoch); dst_s[tid] = 0; pslot[place] = 0; }
    else {
      pslot[place] = (unsigned)((long long)g * cap + idx);
      dst_s[tid] = peers_rows[g] + (unsigned long long)(((long long)rank * cap + idx) * row_bytes);
    }
    w_s[tid] = w[place];
  }
  const float* xr = x + t * cols;
  const int nb = cols / 256;
  float* dscale = (float*)(srow + cols);
  int16_t* dsum = (int16_t*)(srow + cols + nb * 4);
  for (int b = warp; b < nb; b += 4) {
    const float4 v0 = ((const float4*)(xr + b * 256))[2 * lane], v1 = ((const float4*)(xr + b * 256))[2 * lane + 1];
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    int q[8];
    float d;
    q8k_values(v, lane, q, d);
    uint32_t w0, w1;
    int sum = q8k_pack(q, w0, w1);
    ((uint2*)(srow + b * 256))[lane] = make_uint2(w0, w1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (!(lane & 1)) dsum[b * 16 + (lane >> 1)] = (int16_t)sum;
    if (lane == 0) dscale[b] = d;
  }
  __syncthreads();
  // the packed row to each of its destinations, 16 bytes a thread at a time (rows and slabs are 16-byte aligned);
  // the last word, after the sums, is the slot's weight
  const int body = cols + nb * 4 + cols / 8, nv = body / 16;
  for (int s = 0; s < nu; ++s) {
    u8* dst = (u8*)(uintptr_t)dst_s[s];
    if (!dst) continue;
    for (int i = tid; i < nv; i += 128) ((uint4*)dst)[i] = ((const uint4*)srow)[i];
    for (int i = nv * 4 + tid; i < body / 4; i += 128) ((uint32_t*)dst)[i] = ((const uint32_t*)srow)[i];
    if (tid == 0) *(uint32_t*)(dst + body) = w_s[s];
  }
}

// The receiving rank's plan, on the device, for exchanges of a fixed size: RC[s * per + e] = rows source s counted
// for local expert e.  The sender keeps, per destination, only the first CAP rows of its expert order, so of
// those RC rows the ones that arrived are GOT = min(RC, max(0, cap - rows of s's earlier experts)), at slots
// s * cap + (rows of s's earlier experts) ...  Everything below is built from GOT, never from RC, so that the rows
// planned are at most WORLD * CAP whatever the counts say: COUNTS / BASES of the local experts (what ill_moe_mm_id
// reads), P2R[place] = slot of the row placed there (expert by expert, source after source), R2P its inverse on the
// slots in use, P2R of the places past the last row = 0 (a row that exists, so that element-wise steps over all
// CAP * WORLD places read valid memory), TOTAL[0] = rows in all, and *OVERFLOW |= 1 when some source's rows were
// cut (its own flag is up too: that chunk's result is void).  One CTA.
__global__ void __launch_bounds__(256) ep_plan_dev_kernel(int world, int per, int cap, int rank, const unsigned* __restrict__ rc,
                                                          unsigned* __restrict__ counts, unsigned* __restrict__ bases,
                                                          unsigned* __restrict__ p2r, unsigned* __restrict__ r2p,
                                                          unsigned* __restrict__ pdst, unsigned* __restrict__ total,
                                                          unsigned* __restrict__ overflow, const unsigned long long* flag_peers,
                                                          unsigned* flags, unsigned epoch, unsigned long long wait_ns,
                                                          unsigned* status) {
  extern __shared__ unsigned plan_s[];
  unsigned* in_src = plan_s;                 // [world][per] rows of the source's earlier experts (as counted)
  unsigned* before = plan_s + world * per;   // [world][per] rows of the expert that arrived from earlier sources
  unsigned* got = before + world * per;      // [world][per] rows of the segment that arrived
  unsigned* lb = got + world * per;          // [per + 1] first place of each local expert; the total
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  if (flag_peers) {
    // the ranks meet first (slot 0): this rank's rows and counts are in its peers' buffers (the kernels before this
    // one in the stream stored them), and what RC and the slabs hold is complete once every peer has said the same.
    // A meeting that times out leaves a plan of no rows at all.
    const bool ok = ep_meet(flag_peers, flags, world, rank, 0, epoch, true, wait_ns, status);
    if (!__syncthreads_and(ok)) {
      for (int e = tid; e < per; e += blockDim.x) { counts[e] = 0; bases[e] = 0; }
      for (unsigned p = tid; p < (unsigned)(world * cap); p += blockDim.x) {
        p2r[p] = 0;
        if (pdst) pdst[p] = (unsigned)rank << 24 | ((unsigned)rank * cap);
      }
      if (tid == 0) total[0] = 0;
      return;
    }
  }
  for (int s = tid; s < world; s += blockDim.x) {
    unsigned a = 0;
    bool cut = false;
    for (int e = 0; e < per; ++e) {
      const unsigned n = rc[s * per + e];
      const unsigned room = a < (unsigned)cap ? (unsigned)cap - a : 0u;
      in_src[s * per + e] = a;
      got[s * per + e] = n < room ? n : room;
      cut |= n > room;
      a = a + n < a ? 0xffffffffu : a + n;   // saturate: counts are the caller's, not trusted
    }
    if (cut && overflow) { if (flag_peers) atomicMax(overflow, epoch); else atomicOr(overflow, 1u); }
  }
  __syncthreads();
  for (int e = tid; e < per; e += blockDim.x) {
    unsigned a = 0;
    for (int s = 0; s < world; ++s) { before[s * per + e] = a; a += got[s * per + e]; }
    counts[e] = a;
  }
  __syncthreads();
  if (tid == 0) {
    unsigned a = 0;
    for (int e = 0; e < per; ++e) { lb[e] = a; bases[e] = a; a += counts[e]; }
    lb[per] = a;                             // <= world * cap: every source contributes at most cap rows
    total[0] = a;
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  for (int seg = warp; seg < world * per; seg += nw) {
    const int s = seg / per, e = seg - s * per;
    const unsigned n = got[seg], a0 = (unsigned)s * cap + in_src[seg], p0 = lb[e] + before[seg];
    for (unsigned i = lane; i < n; i += 32) {  // in_src + i < cap for every i < got
      p2r[p0 + i] = a0 + i;
      r2p[a0 + i] = p0 + i;
      // where the row's result goes: rank s, row (this rank's slab there) * cap + its index in the slab
      if (pdst) pdst[p0 + i] = ((unsigned)s << 24) | ((unsigned)rank * cap + in_src[seg] + i);
    }
  }
  for (unsigned p = lb[per] + tid; p < (unsigned)(world * cap); p += blockDim.x) {
    p2r[p] = 0;
    if (pdst) pdst[p] = (unsigned)rank << 24 | ((unsigned)rank * cap);
  }
}

// This rank's rows per expert to the experts' ranks, without a collective: COUNTS[g * per + e] into row RANK of
// rank g's [world, per] table (peer memory).
__global__ void __launch_bounds__(256) ep_put_counts_kernel(int world, int per, int rank, const unsigned* __restrict__ counts,
                                                            const unsigned long long* __restrict__ peers,
                                                            unsigned* __restrict__ overflow) {
  pdl_launch_dependents();
  pdl_wait();
  if (overflow && blockIdx.x == 0 && threadIdx.x == 0) *overflow = 0;  // for the pack that follows in the stream
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < world * per; i += gridDim.x * blockDim.x) {
    const int g = i / per, e = i - g * per;
    ((unsigned*)(uintptr_t)peers[g])[rank * per + e] = counts[i];
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

static int act_f16_launch(int64_t rows, int cols, const u8* qp, long long qs, const u8* bp, long long bs, ill_dptr map,
                          ill_dptr xh, ill_dptr xe, const u8* sc, const u8* wt, ill_dptr xd_out, ill_dptr w_out,
                          ill_stream stream, ill_dptr rows_dev = 0) {
  long long nrows = rows;
  const unsigned* mp = (const unsigned*)(uintptr_t)map;
  __half* hp = (__half*)(uintptr_t)xh;
  __half* ep = (__half*)(uintptr_t)xe;
  float* xo = (float*)(uintptr_t)xd_out;
  float* wo = (float*)(uintptr_t)w_out;
  const unsigned* rd = (const unsigned*)(uintptr_t)rows_dev;
  void* args[] = {&nrows, &cols, &qp, &qs, &bp, &bs, &mp, &hp, &ep, &sc, &wt, &xo, &wo, &rd};
  const long long threads = rows * (cols / 16);
  return launch_kernel((const void*)act_f16_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

extern "C" int ill_act_f16(int64_t rows, int cols, ill_dptr xq, ill_dptr bsums, ill_dptr map, ill_dptr xh, ill_dptr xe,
                           ill_stream stream) {
  if (rows < 0 || cols <= 0 || cols % 256 || !xq || !xh || (xe && !bsums)) return ILL_ERR_ARG;
  if ((xq & 15) || (bsums & 1) || (map & 3) || (xh & 15) || (xe & 15)) return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  return act_f16_launch(rows, cols, (const u8*)(uintptr_t)xq, cols, (const u8*)(uintptr_t)bsums, cols / 8, map, xh, xe, nullptr,
                        nullptr, 0, 0, stream);
}

extern "C" int64_t ill_ep_row_bytes(int cols) {
  if (cols <= 0 || cols % 256) return 0;
  return ((int64_t)cols + cols / 256 * 4 + cols / 16 * 2 + 4 + 15) / 16 * 16;
}

extern "C" int ill_ep_pack(int64_t rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr w, ill_dptr map,
                           ill_dptr packed, ill_stream stream) {
  if (rows < 0 || cols <= 0 || cols % 256 || !xq || !xs || !xsum || !w || !map || !packed) return ILL_ERR_ARG;
  if ((xq & 3) || (xs & 3) || (xsum & 3) || (w & 3) || (map & 3) || (packed & 15)) return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  long long rb = ill_ep_row_bytes(cols);
  const uint32_t* qp = (const uint32_t*)(uintptr_t)xq;
  const uint32_t* sp = (const uint32_t*)(uintptr_t)xs;
  const uint32_t* bp = (const uint32_t*)(uintptr_t)xsum;
  const uint32_t* wp = (const uint32_t*)(uintptr_t)w;
  const unsigned* mp = (const unsigned*)(uintptr_t)map;
  uint32_t* pp = (uint32_t*)(uintptr_t)packed;
  void* args[] = {&cols, &rb, &qp, &sp, &bp, &wp, &mp, &pp};
  return launch_kernel((const void*)ep_pack_kernel, dim3((unsigned)rows), dim3(128), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_ep_pack_cap(int64_t rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr w, ill_dptr map,
                               ill_dptr bases, int per, int world, int cap, ill_dptr packed, ill_dptr pslot, ill_dptr overflow,
                               ill_dptr peers, int rank, ill_stream stream) {
  if (rows < 0 || cols <= 0 || cols % 256 || per < 1 || world < 1 || cap < 1 || !xq || !xs || !xsum || !w || !map || !bases ||
      (!packed && !peers) || !pslot || !overflow || rank < 0 || rank >= world)
    return ILL_ERR_ARG;
  if ((xq & 15) || (xs & 3) || (xsum & 3) || (w & 3) || (map & 3) || (bases & 3) || (packed & 15) || (pslot & 3) || (overflow & 3) ||
      (peers & 7))
    return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  long long rb = ill_ep_row_bytes(cols), nrows = rows;
  const uint32_t* qp = (const uint32_t*)(uintptr_t)xq;
  const uint32_t* sp = (const uint32_t*)(uintptr_t)xs;
  const uint32_t* bp = (const uint32_t*)(uintptr_t)xsum;
  const uint32_t* wp = (const uint32_t*)(uintptr_t)w;
  const unsigned* mp = (const unsigned*)(uintptr_t)map;
  const unsigned* bs = (const unsigned*)(uintptr_t)bases;
  uint32_t* pp = (uint32_t*)(uintptr_t)packed;
  unsigned* ps = (unsigned*)(uintptr_t)pslot;
  unsigned* ov = (unsigned*)(uintptr_t)overflow;
  const unsigned long long* pr = (const unsigned long long*)(uintptr_t)peers;
  void* args[] = {&cols, &rb, &qp, &sp, &bp, &wp, &mp, &bs, &per, &world, &cap, &nrows, &pp, &ps, &ov, &pr, &rank};
  return launch_kernel((const void*)ep_pack_cap_kernel, dim3((unsigned)rows), dim3(128), 0, args, (cudaStream_t)stream);
}

extern "C" int ill_ep_dispatch(int64_t ntok, int nu, int cols, ill_dptr x, ill_dptr w, ill_dptr smap, ill_dptr bases, ill_dptr counts,
                               int per, int world, int cap, int rank, ill_dptr peers_rows, ill_dptr peers_rc, ill_dptr pslot,
                               ill_dptr overflow, uint32_t epoch, ill_stream stream) {
  if (ntok < 0 || nu < 1 || nu > EP_MAX_NU || cols <= 0 || cols % 256 || per < 1 || world < 1 || cap < 1 || !x || !w || !smap || !bases ||
      !counts || !peers_rows || !peers_rc || !pslot || !overflow || rank < 0 || rank >= world || epoch == 0)
    return ILL_ERR_ARG;
  if ((x & 15) || (w & 3) || (smap & 3) || (bases & 3) || (counts & 3) || (pslot & 3) || (overflow & 3) || (peers_rows & 7) || (peers_rc & 7))
    return ILL_ERR_ALIGN;
  long long rb = ill_ep_row_bytes(cols);
  if (rb % 16 || rb > 64 * 1024) return ILL_ERR_UNSUPPORTED;
  const float* xp = (const float*)(uintptr_t)x;
  const uint32_t* wp = (const uint32_t*)(uintptr_t)w;
  const unsigned* mp = (const unsigned*)(uintptr_t)smap;
  const unsigned* bs = (const unsigned*)(uintptr_t)bases;
  const unsigned* cp = (const unsigned*)(uintptr_t)counts;
  unsigned* ps = (unsigned*)(uintptr_t)pslot;
  unsigned* ov = (unsigned*)(uintptr_t)overflow;
  const unsigned long long* pr = (const unsigned long long*)(uintptr_t)peers_rows;
  const unsigned long long* pc = (const unsigned long long*)(uintptr_t)peers_rc;
  void* args[] = {&cols, &nu, &rb, &xp, &wp, &mp, &bs, &cp, &per, &world, &cap, &ps, &ov, &epoch, &pr, &pc, &rank};
  const long long need = ((long long)world * per + 127) / 128;  // blocks that carry the counts
  if (ntok < need) return ILL_ERR_UNSUPPORTED;  // fewer tokens than that: use ill_ep_put_counts and ill_ep_pack_cap
  if (rb > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute((const void*)ep_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rb);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  return launch_kernel((const void*)ep_dispatch_kernel, dim3((unsigned)ntok), dim3(128), (size_t)rb, args, (cudaStream_t)stream);
}

extern "C" int ill_ep_put_counts(int world, int per, int rank, ill_dptr counts, ill_dptr peers, ill_dptr overflow,
                                 ill_stream stream) {
  if (world < 1 || per < 1 || rank < 0 || rank >= world || !counts || !peers) return ILL_ERR_ARG;
  if ((counts & 3) || (peers & 7) || (overflow & 3)) return ILL_ERR_ALIGN;
  const unsigned* cp = (const unsigned*)(uintptr_t)counts;
  const unsigned long long* pr = (const unsigned long long*)(uintptr_t)peers;
  unsigned* ov = (unsigned*)(uintptr_t)overflow;
  void* args[] = {&world, &per, &rank, &cp, &pr, &ov};
  return launch_kernel((const void*)ep_put_counts_kernel, dim3((unsigned)((world * per + 255) / 256)), dim3(256), 0, args,
                       (cudaStream_t)stream);
}

static int ep_plan_dev_launch(int world, int per, int cap, int rank, ill_dptr rc, ill_dptr counts, ill_dptr bases, ill_dptr p2r,
                              ill_dptr r2p, ill_dptr pdst, ill_dptr total, ill_dptr overflow, ill_dptr flag_peers, ill_dptr flags,
                              uint32_t epoch, int64_t wait_ns, ill_stream stream);

extern "C" int ill_ep_plan_dev(int world, int per, int cap, int rank, ill_dptr rc, ill_dptr counts, ill_dptr bases, ill_dptr p2r,
                               ill_dptr r2p, ill_dptr pdst, ill_dptr total, ill_dptr overflow, ill_stream stream) {
  return ep_plan_dev_launch(world, per, cap, rank, rc, counts, bases, p2r, r2p, pdst, total, overflow, 0, 0, 0, 0, stream);
}

extern "C" int ill_ep_plan_dev_sync(int world, int per, int cap, int rank, ill_dptr rc, ill_dptr counts, ill_dptr bases, ill_dptr p2r,
                                    ill_dptr r2p, ill_dptr pdst, ill_dptr total, ill_dptr overflow, ill_dptr flag_peers,
                                    ill_dptr flags, uint32_t epoch, int64_t wait_ns, ill_stream stream) {
  if (!flag_peers || !flags || (flag_peers & 7) || (flags & 3) || world > EP_MAX_RANKS || wait_ns < 0) return ILL_ERR_ARG;
  return ep_plan_dev_launch(world, per, cap, rank, rc, counts, bases, p2r, r2p, pdst, total, overflow, flag_peers, flags, epoch,
                            wait_ns, stream);
}

static int ep_plan_dev_launch(int world, int per, int cap, int rank, ill_dptr rc, ill_dptr counts, ill_dptr bases, ill_dptr p2r,
                              ill_dptr r2p, ill_dptr pdst, ill_dptr total, ill_dptr overflow, ill_dptr flag_peers, ill_dptr flags,
                              uint32_t epoch, int64_t wait_ns, ill_stream stream) {
  if (world < 1 || world > 255 || per < 1 || cap < 1 || (long long)world * cap > 0xffffff || rank < 0 || rank >= world ||
      (long long)world * per > 8192 || !rc || !counts || !bases || !p2r || !r2p || !total)
    return ILL_ERR_ARG;
  if ((rc & 3) || (counts & 3) || (bases & 3) || (p2r & 3) || (r2p & 3) || (pdst & 3) || (total & 3) || (overflow & 3)) return ILL_ERR_ALIGN;
  const unsigned* rp = (const unsigned*)(uintptr_t)rc;
  unsigned* cp = (unsigned*)(uintptr_t)counts;
  unsigned* bp = (unsigned*)(uintptr_t)bases;
  unsigned* pp = (unsigned*)(uintptr_t)p2r;
  unsigned* ip = (unsigned*)(uintptr_t)r2p;
  unsigned* tp = (unsigned*)(uintptr_t)total;
  unsigned* dp = (unsigned*)(uintptr_t)pdst;
  unsigned* ov = (unsigned*)(uintptr_t)overflow;
  const unsigned long long* fp = (const unsigned long long*)(uintptr_t)flag_peers;
  unsigned* fl = (unsigned*)(uintptr_t)flags;
  unsigned long long wn = (unsigned long long)wait_ns;
  unsigned* stw = device_status_word();
  void* args[] = {&world, &per, &cap, &rank, &rp, &cp, &bp, &pp, &ip, &dp, &tp, &ov, &fp, &fl, &epoch, &wn, &stw};
  const size_t smem = ((size_t)3 * world * per + per + 1) * 4;
  const void* k = (const void*)ep_plan_dev_kernel;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  return launch_kernel(k, dim3(1), dim3(256), smem, args, (cudaStream_t)stream);
}

extern "C" int ill_ep_unpack(int64_t rows, int cols, ill_dptr packed, ill_dptr map, ill_dptr xh, ill_dptr xe, ill_dptr xd,
                             ill_dptr w, ill_dptr rows_dev, ill_stream stream) {
  if (rows < 0 || cols <= 0 || cols % 256 || !packed || !xh || !xd || !w) return ILL_ERR_ARG;
  if ((packed & 15) || (map & 3) || (xh & 15) || (xe & 15) || (xd & 3) || (w & 3) || (rows_dev & 3)) return ILL_ERR_ALIGN;
  if (rows == 0) return ILL_OK;
  const long long rb = ill_ep_row_bytes(cols);
  const u8* base = (const u8*)(uintptr_t)packed;
  return act_f16_launch(rows, cols, base, rb, base + cols + cols / 256 * 4, rb, map, xh, xe, base + cols,
                        base + cols + cols / 256 * 4 + cols / 16 * 2, xd, w, stream, rows_dev);
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

static int mm_id_launch(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases, int ne,
                        int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr ymap, ill_dptr ypeers,
                        ill_dptr y, int64_t y_stride, ill_stream stream, int64_t add2 = 0, ill_dptr y2 = 0, ill_dptr one_ptr = 0,
                        int acc = 0);

extern "C" int ill_moe_mm_id2(int fmt, int ncols, int nrows, int64_t add, int64_t add2, ill_dptr ptrs, ill_dptr counts,
                              ill_dptr bases, int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map,
                              ill_dptr y, ill_dptr y2, int64_t y_stride, ill_stream stream) {
  if (!y || !y2 || (y2 & 15) || (add2 & 3)) return ILL_ERR_ARG;
  return mm_id_launch(fmt, ncols, nrows, add, ptrs, counts, bases, ne, total_rows, xh, xe, xd, map, 0, 0, y, y_stride, stream, add2,
                      y2);
}

extern "C" int ill_moe_mm_id(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases,
                             int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr ymap,
                             ill_dptr y, int64_t y_stride, ill_stream stream) {
  if (!y) return ILL_ERR_ARG;
  return mm_id_launch(fmt, ncols, nrows, add, ptrs, counts, bases, ne, total_rows, xh, xe, xd, map, ymap, 0, y, y_stride, stream);
}

extern "C" int ill_moe_mm_id_peers(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases,
                                   int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr ydst,
                                   ill_dptr ypeers, int64_t y_stride, ill_stream stream) {
  if (!ydst || !ypeers || (ypeers & 7)) return ILL_ERR_ARG;
  // Y is only named through YPEERS; any aligned non-null value keeps the common checks happy
  return mm_id_launch(fmt, ncols, nrows, add, ptrs, counts, bases, ne, total_rows, xh, xe, xd, map, ydst, ypeers, 16, y_stride,
                      stream);
}

extern "C" int ill_mm_chunk(int fmt, ill_dptr w, int rows, int cols, ill_dptr xh, ill_dptr xe, ill_dptr xd, int64_t n, ill_dptr y,
                            int acc, ill_stream stream) {
  if (!w || !y || n < 0 || n > 0x7fffffffll) return ILL_ERR_ARG;
  if (fmt != ILL_Q4_K && fmt != ILL_Q6_K) return ILL_ERR_UNSUPPORTED;
  return mm_id_launch(fmt, cols, rows, 0, 0, 0, 0, 1, n, xh, xe, xd, 0, 0, 0, y, rows, stream, 0, 0, w, acc ? 1 : 0);
}

// two matrices of one shape against the same chunk in one launch (a gated FFN's gate and up): twice the tiles for
// the persistent CTAs to share, so the last round of tiles is fuller than in two launches
extern "C" int ill_mm_chunk2(int fmt, ill_dptr w, ill_dptr w2, int rows, int cols, ill_dptr xh, ill_dptr xe, ill_dptr xd, int64_t n,
                             ill_dptr y, ill_dptr y2, ill_stream stream) {
  if (!w || !w2 || !y || !y2 || (y2 & 15) || n < 0 || n > 0x7fffffffll) return ILL_ERR_ARG;
  if (fmt != ILL_Q4_K && fmt != ILL_Q6_K) return ILL_ERR_UNSUPPORTED;
  const int64_t add2 = (int64_t)(w2 - w);  // the second matrix, relative to the first (unsigned wrap-around is intended)
  if (add2 & (fmt == ILL_Q4_K ? 15 : 3)) return ILL_ERR_ALIGN;
  return mm_id_launch(fmt, cols, rows, 0, 0, 0, 0, 1, n, xh, xe, xd, 0, 0, 0, y, rows, stream, add2, y2, w, 0);
}

static int mm_id_launch(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases, int ne,
                        int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr ymap, ill_dptr ypeers,
                        ill_dptr y, int64_t y_stride, ill_stream stream, int64_t add2, ill_dptr y2, ill_dptr one_ptr, int acc) {
  if (fmt != ILL_IQ2_XXS && fmt != ILL_Q2_K && fmt != ILL_Q4_K && fmt != ILL_Q6_K) return ILL_ERR_UNSUPPORTED;
  const bool km = fmt == ILL_Q2_K || fmt == ILL_Q4_K;  // formats with mins: the sums of 16 of X come along
  if (ncols <= 0 || ncols % 256 || nrows <= 0 || ne <= 0 || ne > 65535 || total_rows < 0 || y_stride < nrows ||
      y_stride > 0xffffffffll)
    return ILL_ERR_ARG;
  if (!one_ptr && (!ptrs || !counts || !bases)) return ILL_ERR_ARG;
  if (!xh || !xd || !y || (km && !xe)) return ILL_ERR_ARG;
  if (fmt == ILL_Q4_K && (one_ptr & 15)) return ILL_ERR_ALIGN;
  if ((ptrs & 7) || (counts & 3) || (bases & 3) || (xh & 15) || (xe & 15) || (xd & 3) || (map & 3) || (ymap & 3) || (y & 15) ||
      (y_stride & 3) || (add & 3))
    return ILL_ERR_ALIGN;
  if (fmt == ILL_Q4_K && ((add | add2) & 15)) return ILL_ERR_ALIGN;  // (and every PTRS[e]: the kernel copies 16-byte pieces of the rows as they lie)
  if (total_rows == 0) return ILL_OK;
  CUtensorMap xmap, emap;
  int rc = encode_map(&xmap, xh, ncols, total_rows);
  if (rc) return rc;
  rc = km ? encode_map(&emap, xe, (int64_t)(ncols / 256) * 64, total_rows) : encode_map(&emap, xh, ncols, total_rows);
  if (rc) return rc;
  MmParams p;
  p.ncols = ncols;
  p.nrows = nrows;
  p.row_bytes = ncols / 256 * fmt_block_bytes(fmt);
  p.add = add;
  p.add2 = add2;
  p.ptrs = (const unsigned long long*)(uintptr_t)ptrs;
  p.counts = (const unsigned*)(uintptr_t)counts;
  p.bases = (const unsigned*)(uintptr_t)bases;
  p.xd = (const float*)(uintptr_t)xd;
  p.map = (const unsigned*)(uintptr_t)map;
  p.ymap = (const unsigned*)(uintptr_t)ymap;
  p.ypeers = (const unsigned long long*)(uintptr_t)ypeers;
  p.total_rows = total_rows;
  p.y = (float*)(uintptr_t)y;
  p.y2 = (float*)(uintptr_t)y2;
  p.y_stride = y_stride;
  p.ne = ne;
  p.one_ptr = one_ptr;
  p.one_count = (unsigned)total_rows;
  p.acc = acc;
  p.status = device_status_word();
  const long long max_tiles = ((total_rows + MM_BM - 1) / MM_BM + ne) * ((nrows + MM_BN - 1) / MM_BN) * (y2 ? 2 : 1);  // an upper bound
  const size_t smem = fmt == ILL_IQ2_XXS ? MmGeom<ILL_IQ2_XXS>::SMEM : fmt == ILL_Q2_K ? MmGeom<ILL_Q2_K>::SMEM
                      : fmt == ILL_Q4_K ? MmGeom<ILL_Q4_K>::SMEM : MmGeom<ILL_Q6_K>::SMEM;
  if (ne > 512) return ILL_ERR_TOO_LARGE;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const void* k = fmt == ILL_IQ2_XXS ? (const void*)mm_id_kernel<ILL_IQ2_XXS, false>
                  : fmt == ILL_Q2_K ? (const void*)mm_id_kernel<ILL_Q2_K, false>
                  : fmt == ILL_Q4_K ? (one_ptr ? (const void*)mm_id_kernel<ILL_Q4_K, true> : (const void*)mm_id_kernel<ILL_Q4_K, false>)
                                    : (one_ptr ? (const void*)mm_id_kernel<ILL_Q6_K, true> : (const void*)mm_id_kernel<ILL_Q6_K, false>);
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  // The warp groups trade registers after launch; what they ask for together must fit in what the
  // CTA was given, or the drain warps would wait for registers for ever.
  cudaFuncAttributes fa;
  e = cudaFuncGetAttributes(&fa, k);
  if (e != cudaSuccess) return cuda_fail(e);
  if (fa.numRegs * MM_THREADS < 128 * (MM_REGS_AUX + MM_REGS_DRAIN) + 32 * MM_DQ_WARPS * MM_REGS_DQ) return ILL_ERR_UNSUPPORTED;
  void* args[] = {&xmap, &emap, &p};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(max_tiles < sms ? max_tiles : sms), 1, 1);  // persistent: a CTA an SM, each walks tiles
  cfg.blockDim = dim3(MM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  e = cudaLaunchKernelExC(&cfg, k, args);
  return e == cudaSuccess ? ILL_OK : cuda_fail(e);
}
