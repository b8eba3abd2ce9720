// Dense products for a chunk of tokens (prefill): Y[token][row] = W[row] . X[token] for more than 16 tokens,
// W in Q8_0 / Q4_K / Q6_K blocks, X quantized to Q8_0 (for Q8_0) or Q8_K (for the K formats) -- the same integer
// arithmetic a row of the one-token product does, 16 rows x 8 tokens at a time on the tensor cores' int8 path
// (mma.sync m16n8k32 / m16n8k16), each group's integer sum scaled as the CPU path scales it.
//
// Design.  A CTA of eight warps takes 128 rows x TN tokens (TN = 32, 64 or 128); warp w owns rows 16 w .. 16 w + 15
// against all TN tokens, so a block of weights is unpacked into tensor-core fragments once and used TN / 8 times
// from registers.  The columns go by in steps of 256:
//   * weights: every warp runs its own ring of stages, lanes 0..15 each copying one row's 256 columns of blocks
//     (144 / 210 / 272 bytes, widened to 16-byte boundaries) with cp.async.bulk onto the stage's mbarrier; a stage
//     is free again as soon as its block sits in registers, so the next copy is issued before the arithmetic;
//   * activations: the step's TN x 256 quants and their scales are brought by all threads with cp.async into one
//     of two buffers while the other is being used -- one __syncthreads a step; a token tile's quants reach the
//     registers as B fragments through ldmatrix.
// Token tiles are the fastest-varying CTA index: the CTAs that share a tile of rows run together and the weights
// come from HBM once.  Waits are bounded (status word, ST_MV_WAIT + 0x40 + format); a warp that gave up keeps
// meeting the CTA's barriers and lets its copies land before the CTA leaves.
//
// Replaces mm_q8_mma2 / mm_q4k_mma / mm_q6k_mma behind CMAT-MUL-N for prefill chunks
// (src/cuda-dense.lisp:220-255; src/cuda/dense.cu:885-1100, src/cuda/kquant.cu:316-466).
#include "formats.cuh"
#include "host.h"
#include "mma_i8.cuh"

namespace ill {

constexpr int MD_WARPS = 8, MD_THREADS = 32 * MD_WARPS, MD_ROWS = 16 * MD_WARPS, MD_MAX_STAGES = 3;
constexpr int MD_XPITCH = 272;  // bytes between the tokens' 256 quants of a step: 68 words, so eight tokens x four words hit 32 banks

struct MdParams {
  const u8* w;
  int rows, cols, row_bytes, nsteps;
  const i8* xq;
  const float* xs;
  const int16_t* xsum;
  float* y;
  const float* bias;
  int acc, n;
  int warps;             // warps a CTA (16 rows each)
  int stages;            // stages of a warp's ring of weights (2 or 3)
  int pitch;             // bytes between the rows of a staged piece
  uint32_t stage_bytes;
  uint32_t xbuf_bytes, xs_off, xsum_off;  // one activation buffer: its size, where its scales and (Q4_K) sums start
  uint32_t ring_off, part_off;
  unsigned* status;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// four 8 x 16-byte matrices of shared memory -> each lane its four bytes of row lane / 4 of each: lane l gives the
// address of row l % 8 of matrix l / 8.  For a token tile's 64 bytes of quants this is the B fragment of two k32
// (or four k16) steps: r[0], r[1] = b0, b1 of the first k32 step, r[2], r[3] of the second.
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

// ---- a step's block(s) of 16 rows as tensor-core fragments, and their use against eight tokens ---------------
// load(): ROW0 / ROW8 = the staged bytes of rows g and g + 8 (g = lane / 4), NB = valid blocks in the step.
// apply(): B = the tile's eight tokens' 256 quants as B fragments (ldsm4 of 64 bytes each); YA / YB the Q8_K scales
// of tokens 8 nt + 2 (lane % 4) and + 1 (Q8_0: SA / SB their eight scales); ACC the lane's four outputs:
// i -> row g + 8 (i / 2), token 8 nt + 2 (lane % 4) + i % 2.
//
// The integer sums are the CPU path's, exactly.  Q6_K's 0..63 quants go in as signed q - 32 (no sums of activations
// needed), each group of 16 a k16 product scaled by its signed scale; Q4_K's mins meet the activations' sums of 16.
// (Carrying Q4_K's scales on the tensor core -- (s & 7) q and (s >> 3) q both fit a byte, so a block is c1 + 8 c2 of
// two accumulating chains, the mins a third -- was measured slower: an int8 mma.sync costs about seven issue slots
// here, so fewer of them with an integer multiply-add a group wins.)
template <int FMT> struct MdFrag;

template <> struct MdFrag<ILL_Q8_0> {
  static constexpr int SB = 272;  // eight blocks of 34 bytes
  static constexpr int SPITCH = 32;  // bytes between the tokens' eight scales of a step
  uint32_t a[8][4];
  float d0[8], d8[8];
  __device__ __forceinline__ void load(const u8* row0, const u8* row8, int lane, int nb) {
    const int t4 = 4 * (lane & 3);
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const u8 *r0 = row0 + 34 * b, *r8 = row8 + 34 * b;
      const bool in = b < nb;  // past the row's last block: zeros
      a[b][0] = in ? lds32u(r0 + 2 + t4) : 0u;
      a[b][1] = in ? lds32u(r8 + 2 + t4) : 0u;
      a[b][2] = in ? lds32u(r0 + 18 + t4) : 0u;
      a[b][3] = in ? lds32u(r8 + 18 + t4) : 0u;
      d0[b] = in ? ldh(r0) : 0.0f;
      d8[b] = in ? ldh(r8) : 0.0f;
    }
  }
  __device__ __forceinline__ void apply(const uint32_t (&x)[4][4], const u8* sa, const u8* sb, float, float, float (&acc)[4]) const {
    const float4 xa0 = *(const float4*)sa, xa1 = *(const float4*)(sa + 16), xb0 = *(const float4*)sb, xb1 = *(const float4*)(sb + 16);
    const float da[8] = {xa0.x, xa0.y, xa0.z, xa0.w, xa1.x, xa1.y, xa1.z, xa1.w};
    const float db[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t bb[2] = {x[b >> 1][2 * (b & 1)], x[b >> 1][2 * (b & 1) + 1]};
      int c[4] = {0, 0, 0, 0};
      mma_k32(c, a[b], bb, false);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        // Q8-ROW-DOT-AT: sum += float(isum) * (d_w * d_x)
        acc[i] = __fadd_rn(acc[i], __fmul_rn((float)c[i], __fmul_rn(i < 2 ? d0[b] : d8[b], (i & 1) ? db[b] : da[b])));
    }
  }
};

template <> struct MdFrag<ILL_Q4_K> {
  static constexpr int SB = 144;
  static constexpr int SPITCH = 48;  // bytes between the tokens' sixteen sums of a step: four tokens' 16-byte reads on different banks
  uint32_t lo[4][4], hi[4][4];
  int sc0[8], sc8[8];
  int mn0[4], mn8[4];  // the mins of groups 2 j and 2 j + 1, each in two bytes: dp2a against the group's two sums of 16
  float d0, m0, d8, m8;
  __device__ __forceinline__ void load(const u8* row0, const u8* row8, int lane, int) {
    const int t4 = 4 * (lane & 3);
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // 64 weights: groups 2k (low nibbles) and 2k + 1 (high)
      const uint32_t w0 = lds32u(row0 + 16 + 32 * k + t4), w1 = lds32u(row8 + 16 + 32 * k + t4);
      const uint32_t w2 = lds32u(row0 + 32 + 32 * k + t4), w3 = lds32u(row8 + 32 + 32 * k + t4);
      lo[k][0] = w0 & 0x0F0F0F0Fu; lo[k][1] = w1 & 0x0F0F0F0Fu; lo[k][2] = w2 & 0x0F0F0F0Fu; lo[k][3] = w3 & 0x0F0F0F0Fu;
      hi[k][0] = (w0 >> 4) & 0x0F0F0F0Fu; hi[k][1] = (w1 >> 4) & 0x0F0F0F0Fu;
      hi[k][2] = (w2 >> 4) & 0x0F0F0F0Fu; hi[k][3] = (w3 >> 4) & 0x0F0F0F0Fu;
      int a, b, ma, mb;
      scale_min_k4(row0 + 4, 2 * k, a, ma); scale_min_k4(row0 + 4, 2 * k + 1, b, mb);
      sc0[2 * k] = a; sc0[2 * k + 1] = b;
      mn0[k] = ma * 0x0101 | (mb * 0x0101) << 16;
      scale_min_k4(row8 + 4, 2 * k, a, ma); scale_min_k4(row8 + 4, 2 * k + 1, b, mb);
      sc8[2 * k] = a; sc8[2 * k + 1] = b;
      mn8[k] = ma * 0x0101 | (mb * 0x0101) << 16;
    }
    d0 = ldh(row0); m0 = ldh(row0 + 2); d8 = ldh(row8); m8 = ldh(row8 + 2);
  }
  // SA / SB: the sixteen sums of 16 (int16) of the two tokens' step
  __device__ __forceinline__ void apply(const uint32_t (&x)[4][4], const u8* sa, const u8* sb, float ya, float yb, float (&acc)[4]) const {
    int isum[4] = {0, 0, 0, 0}, imin[4] = {0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t b0[2] = {x[k][0], x[k][1]}, b1[2] = {x[k][2], x[k][3]};
      int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
      mma_k32(c0, lo[k], b0, true);
      mma_k32(c1, hi[k], b1, true);
#pragma unroll
      for (int i = 0; i < 4; ++i) isum[i] += c0[i] * (i < 2 ? sc0[2 * k] : sc8[2 * k]) + c1[i] * (i < 2 ? sc0[2 * k + 1] : sc8[2 * k + 1]);
    }
    // the mins' side: sum over the groups of min * (the group's two sums of 16)
    const int4 a0 = *(const int4*)sa, a1 = *(const int4*)(sa + 16), c0 = *(const int4*)sb, c1 = *(const int4*)(sb + 16);
    const int pa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const int pb[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int m = i < 2 ? mn0[k] : mn8[k];
        imin[i] = dp2a_hi((i & 1) ? pb[2 * k + 1] : pa[2 * k + 1], m, dp2a_lo((i & 1) ? pb[2 * k] : pa[2 * k], m, imin[i]));
      }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float yd = (i & 1) ? yb : ya;
      // Q4K-ROW-DOT: sum -= (yd * dmin) * imin; sum += (yd * d) * isum
      const float s = __fsub_rn(acc[i], __fmul_rn(__fmul_rn(yd, i < 2 ? m0 : m8), (float)imin[i]));
      acc[i] = __fadd_rn(s, __fmul_rn(__fmul_rn(yd, i < 2 ? d0 : d8), (float)isum[i]));
    }
  }
};

// four 6-bit values 0..63, a byte each -> the signed bytes value - 32
__device__ __forceinline__ uint32_t q6_signed(uint32_t v) {
  const uint32_t t = v ^ 0x20202020u, s = t & 0x20202020u;  // t = value - 32 modulo 64; s: its sign (bit 5)
  return t | (s << 1) | (s << 2);
}

template <> struct MdFrag<ILL_Q6_K> {
  static constexpr int SB = 210;
  static constexpr int SPITCH = 0;
  uint32_t q[16][2];  // [group of 16][row g / g + 8]: the lane's four quants as signed bytes -32..31
  int sc0[16], sc8[16];
  float d0, d8;
  __device__ __forceinline__ void load(const u8* row0, const u8* row8, int lane, int) {
    const int t4 = 4 * (lane & 3);
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int is = 0; is < 2; ++is) {
        const int l = 16 * is + t4;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const u8* row = r ? row8 : row0;
          const uint32_t A = lds32u(row + 64 * c + l), B = lds32u(row + 64 * c + 32 + l), H = lds32u(row + 128 + 32 * c + l);
          // run RUN of the half covers weights 128 c + 32 run ..: its group of 16 is 8 c + 2 run + is
          q[8 * c + 0 + is][r] = q6_signed((A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u));
          q[8 * c + 2 + is][r] = q6_signed((B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u));
          q[8 * c + 4 + is][r] = q6_signed(((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u));
          q[8 * c + 6 + is][r] = q6_signed(((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u));
        }
      }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t w0 = lds32u(row0 + 192 + 4 * w), w8 = lds32u(row8 + 192 + 4 * w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sc0[4 * w + j] = (int)(signed char)(w0 >> (8 * j));
        sc8[4 * w + j] = (int)(signed char)(w8 >> (8 * j));
      }
    }
    d0 = ldh(row0 + 208); d8 = ldh(row8 + 208);
  }
  __device__ __forceinline__ void apply(const uint32_t (&x)[4][4], const u8*, const u8*, float ya, float yb, float (&acc)[4]) const {
    int isum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int grp = 0; grp < 16; ++grp) {  // group GRP's 16 weights face the token's 16 quants at 16 grp
      int cc[4] = {0, 0, 0, 0};
      mma_k16_s8(cc, q[grp][0], q[grp][1], x[grp >> 2][grp & 3], false);
#pragma unroll
      for (int i = 0; i < 4; ++i) isum[i] += cc[i] * (i < 2 ? sc0[grp] : sc8[grp]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      // Q6K-ROW-DOT: sum += (d * yd) * float(sum over the groups of scale * dot(q - 32, x))
      acc[i] = __fadd_rn(acc[i], __fmul_rn(__fmul_rn(i < 2 ? d0 : d8, (i & 1) ? yb : ya), (float)isum[i]));
  }
};

// MINB = 2 (token tiles of 64): a thread stays within 128 registers and two CTAs share an SM
template <int FMT, int NT8, int MINB>
__global__ void __launch_bounds__(MD_THREADS, MINB) mmd_kernel(const MdParams p) {
  extern __shared__ __align__(128) u8 smem[];
  constexpr int TN = 8 * NT8, SB = MdFrag<FMT>::SB, MD_SPITCH = MdFrag<FMT>::SPITCH;
  const int MD_STAGES = p.stages;
  constexpr bool KQ = FMT != ILL_Q8_0;  // Q8_K activations: one scale a step (Q8_0: eight)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int ntt = (p.n + TN - 1) / TN, nthreads = blockDim.x;  // eight warps, or fewer when the matrix has few rows
  const int tok0 = (int)(blockIdx.x % ntt) * TN, row_base = (int)(blockIdx.x / ntt) * (nthreads / 2) + warp * 16;
  const int nsteps = p.nsteps;
  const bool live = row_base < p.rows;  // a warp whose rows are all past the end only helps to bring the activations
  u8* ring = smem + p.ring_off + (size_t)warp * MD_STAGES * p.stage_bytes;
  __shared__ uint64_t full_s[MD_WARPS * MD_MAX_STAGES];
  uint64_t* full = full_s + warp * MD_MAX_STAGES;

  int issued = 0;
  auto issue_w = [&]() {  // all lanes of the warp; lanes 0..15 copy a row's step each
    if (!live || issued >= nsteps) return;
    const int s = issued % MD_STAGES;
    const int row = row_base + lane;
    uint32_t bytes = 0;
    const u8* src = nullptr;
    if (lane < 16 && row < p.rows) {
      src = p.w + (long long)row * p.row_bytes + (long long)issued * SB;
      const uint32_t len = (uint32_t)min(SB, p.row_bytes - issued * SB);
      bytes = (uint32_t)((((uintptr_t)src + len + 15) & ~(uintptr_t)15) - ((uintptr_t)src & ~(uintptr_t)15));
    }
    uint32_t total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) mbar_expect_tx(&full[s], total);
    __syncwarp();
    if (bytes) bulk_g2s(ring + (size_t)s * p.stage_bytes + (size_t)lane * p.pitch, (const void*)((uintptr_t)src & ~(uintptr_t)15), bytes, &full[s]);
    ++issued;
  };
  auto fill_x = [&](int step) {  // all threads: the step's activations -> buffer step % 2
    u8* xb = smem + (size_t)(step & 1) * p.xbuf_bytes;
    const int c0 = 256 * step;
    for (int i = tid; i < TN * 16; i += nthreads) {
      const int tk = i >> 4, ch = i & 15;
      if (tok0 + tk < p.n && c0 + 16 * ch < p.cols)
        cp_async16(xb + tk * MD_XPITCH + 16 * ch, p.xq + (long long)(tok0 + tk) * p.cols + c0 + 16 * ch);
    }
    if constexpr (KQ) {
      for (int i = tid; i < TN; i += nthreads)
        if (tok0 + i < p.n) cp_async4(xb + p.xs_off + 4 * i, p.xs + (long long)(tok0 + i) * nsteps + step);
      if constexpr (FMT == ILL_Q4_K) {
        for (int i = tid; i < TN * 2; i += nthreads) {
          const int tk = i >> 1, ch = i & 1;
          if (tok0 + tk < p.n)
            cp_async16(xb + p.xsum_off + tk * MD_SPITCH + 16 * ch, p.xsum + (long long)(tok0 + tk) * (p.cols / 16) + 16 * step + 8 * ch);
        }
      }
    } else {
      for (int i = tid; i < TN * 2; i += nthreads) {
        const int tk = i >> 1, ch = i & 1;
        if (tok0 + tk < p.n && c0 + 128 * ch < p.cols)
          cp_async16(xb + p.xs_off + tk * MD_SPITCH + 16 * ch, p.xs + (long long)(tok0 + tk) * (p.cols / 32) + 8 * step + 4 * ch);
      }
    }
    cp_async_commit();
  };

  // both activation buffers start as zeros: the tokens past the last, and the columns past a Q8_0 row's end, stay so
  for (uint32_t i = 16u * tid; i < 2u * p.xbuf_bytes; i += 16u * nthreads) *(uint4*)(smem + i) = make_uint4(0, 0, 0, 0);
  if (lane == 0) {
    for (int s = 0; s < MD_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  for (int s = 0; s < MD_STAGES; ++s) issue_w();  // the weights do not depend on the previous kernel
  pdl_launch_dependents();
  pdl_wait();
  fill_x(0);

  float acc[NT8][4];
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
  bool dead = false;
  int done = 0;
  for (int step = 0; step < nsteps; ++step) {
    cp_async_wait_all();
    __syncthreads();  // the step's activations are in; everyone is through with the other buffer
    if (step + 1 < nsteps) fill_x(step + 1);
    if (!live || dead) continue;
    const int s = step % MD_STAGES;
    bool ok = mbar_wait(&full[s], (uint32_t)(step / MD_STAGES) & 1u, p.status, ST_MV_WAIT + 0x40 + FMT);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) { dead = true; continue; }
    ++done;
    MdFrag<FMT> f;
    {
      const u8* piece = ring + (size_t)s * p.stage_bytes;
      // a row's bytes start where its block starts inside the 16-byte aligned span that was copied
      const long long o0 = (long long)(row_base + g) * p.row_bytes + (long long)step * SB;
      const long long o8 = o0 + 8ll * p.row_bytes;
      const u8* row0 = piece + (size_t)g * p.pitch + (((uintptr_t)p.w + o0) & 15);
      const u8* row8 = piece + (size_t)(g + 8) * p.pitch + (((uintptr_t)p.w + o8) & 15);
      f.load(row0, row8, lane, min(8, (p.cols - 256 * step) / 32));
    }
    __syncwarp();
    issue_w();  // the stage is free: its block sits in registers
    const u8* xb = smem + (size_t)(step & 1) * p.xbuf_bytes;
    const u8* xl = xb + (lane & 7) * MD_XPITCH + 16 * (lane >> 3);  // this lane's row of the four matrices ldsm4 reads
    // Q8_0: the eight scales of token 2 t (+ 8 nt); Q4_K: its sixteen sums of 16
    const u8* scl = xb + (FMT == ILL_Q4_K ? p.xsum_off : p.xs_off) + 2 * t * MD_SPITCH;
    const float* ys = (const float*)(xb + p.xs_off) + 2 * t;
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      uint32_t x[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) ldsm4(x[j], xl + 8 * nt * MD_XPITCH + 64 * j);
      float ya = 0.0f, yb = 0.0f;
      if constexpr (KQ) { ya = ys[8 * nt]; yb = ys[8 * nt + 1]; }
      f.apply(x, scl + 8 * nt * MD_SPITCH, scl + (8 * nt + 1) * MD_SPITCH, ya, yb, acc[nt]);
    }
  }
  if (dead) {
    // copies still in flight into this warp's stages get a bounded time to land before shared memory is released
    for (int k = done; k < issued; ++k) mbar_wait(&full[k % MD_STAGES], (uint32_t)(k / MD_STAGES) & 1u, nullptr, 0);
    return;
  }
  if (!live) return;
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long row = row_base + g + 8 * (i >> 1);
      const int tok = tok0 + 8 * nt + 2 * t + (i & 1);
      if (row < p.rows && tok < p.n) {
        float v = acc[nt][i];
        if (p.bias) v += p.bias[row];
        float* yp = p.y + (long long)tok * p.rows + row;
        *yp = p.acc ? *yp + v : v;
      }
    }
}

// ---- up to sixteen tokens of rows too long for mvt.cu to keep the activations resident ------------------------
// One 16-row tile a CTA, its column steps dealt to the eight warps (warp w takes steps w, w + 8, ...): each warp
// streams its own steps' weights (its ring) AND its own steps' activations (cp.async by its lanes into two buffers of
// its own), so the warps never wait for one another until the end, where their partial sums meet in shared memory
// in warp order.  A matrix of few rows and many columns (5120 x 17408) thus fills the machine with rows / 16 CTAs
// of eight busy warps, where the chunk kernel above would run two warps a CTA through all 68 steps.
template <int FMT, int NT8>
__global__ void __launch_bounds__(MD_THREADS, 1) mmk_kernel(const MdParams p) {
  extern __shared__ __align__(128) u8 smem[];
  constexpr int TN = 8 * NT8, SB = MdFrag<FMT>::SB, SP = MdFrag<FMT>::SPITCH;
  constexpr bool KQ = FMT != ILL_Q8_0;
  const int stages = p.stages;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int ntt = (p.n + TN - 1) / TN;
  const int tok0 = (int)(blockIdx.x % ntt) * TN, row_base = (int)(blockIdx.x / ntt) * 16;
  const int nsteps = p.nsteps;
  u8* xw = smem + (size_t)warp * 2 * p.xbuf_bytes;  // this warp's two activation buffers
  u8* ring = smem + p.ring_off + (size_t)warp * stages * p.stage_bytes;
  float* part = (float*)(smem + p.part_off);        // [warp][16 rows][TN]
  __shared__ uint64_t full_s[MD_WARPS * MD_MAX_STAGES];
  uint64_t* full = full_s + warp * MD_MAX_STAGES;

  int issued = 0;  // of this warp's steps
  auto issue_w = [&]() {
    const int step = warp + MD_WARPS * issued;
    if (step >= nsteps) return;
    const int s = issued % stages;
    const int row = row_base + lane;
    uint32_t bytes = 0;
    const u8* src = nullptr;
    if (lane < 16 && row < p.rows) {
      src = p.w + (long long)row * p.row_bytes + (long long)step * SB;
      const uint32_t len = (uint32_t)min(SB, p.row_bytes - step * SB);
      bytes = (uint32_t)((((uintptr_t)src + len + 15) & ~(uintptr_t)15) - ((uintptr_t)src & ~(uintptr_t)15));
    }
    uint32_t total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) mbar_expect_tx(&full[s], total);
    __syncwarp();
    if (bytes) bulk_g2s(ring + (size_t)s * p.stage_bytes + (size_t)lane * p.pitch, (const void*)((uintptr_t)src & ~(uintptr_t)15), bytes, &full[s]);
    ++issued;
  };
  auto fill_x = [&](int k) {  // this warp's K-th step -> its buffer k % 2 (a group of cp.async, possibly empty)
    const int step = warp + MD_WARPS * k;
    if (step < nsteps) {
      u8* xb = xw + (size_t)(k & 1) * p.xbuf_bytes;
      const int c0 = 256 * step;
      for (int i = lane; i < TN * 16; i += 32) {
        const int tk = i >> 4, ch = i & 15;
        if (tok0 + tk < p.n && c0 + 16 * ch < p.cols)
          cp_async16(xb + tk * MD_XPITCH + 16 * ch, p.xq + (long long)(tok0 + tk) * p.cols + c0 + 16 * ch);
      }
      if constexpr (KQ) {
        for (int i = lane; i < TN; i += 32)
          if (tok0 + i < p.n) cp_async4(xb + p.xs_off + 4 * i, p.xs + (long long)(tok0 + i) * nsteps + step);
        if constexpr (FMT == ILL_Q4_K) {
          for (int i = lane; i < TN * 2; i += 32) {
            const int tk = i >> 1, ch = i & 1;
            if (tok0 + tk < p.n)
              cp_async16(xb + p.xsum_off + tk * SP + 16 * ch, p.xsum + (long long)(tok0 + tk) * (p.cols / 16) + 16 * step + 8 * ch);
          }
        }
      } else {
        for (int i = lane; i < TN * 2; i += 32) {
          const int tk = i >> 1, ch = i & 1;
          if (tok0 + tk < p.n && c0 + 128 * ch < p.cols)
            cp_async16(xb + p.xs_off + tk * SP + 16 * ch, p.xs + (long long)(tok0 + tk) * (p.cols / 32) + 8 * step + 4 * ch);
        }
      }
    }
    cp_async_commit();
  };

  // the warp's activation buffers start as zeros (tokens past the last, columns past a Q8_0 row's end)
  for (uint32_t i = 16u * lane; i < 2u * p.xbuf_bytes; i += 16u * 32u) *(uint4*)(xw + i) = make_uint4(0, 0, 0, 0);
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  for (int s = 0; s < stages; ++s) issue_w();  // the weights do not depend on the previous kernel
  pdl_launch_dependents();
  pdl_wait();
  fill_x(0);

  float acc[NT8][4];
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
  bool dead = false;
  int done = 0;
  for (int k = 0; warp + MD_WARPS * k < nsteps && !dead; ++k) {
    const int step = warp + MD_WARPS * k;
    fill_x(k + 1);                                          // the other buffer: its readers are through (the __syncwarp below)
    asm volatile("cp.async.wait_group 1;" ::: "memory");   // all but that newest group: step k's activations are in
    __syncwarp();
    const int s = k % stages;
    bool ok = mbar_wait(&full[s], (uint32_t)(k / stages) & 1u, p.status, ST_MV_WAIT + 0x48 + FMT);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) { dead = true; break; }
    ++done;
    MdFrag<FMT> f;
    {
      const u8* piece = ring + (size_t)s * p.stage_bytes;
      const long long o0 = (long long)(row_base + g) * p.row_bytes + (long long)step * SB;
      const long long o8 = o0 + 8ll * p.row_bytes;
      const u8* row0 = piece + (size_t)g * p.pitch + (((uintptr_t)p.w + o0) & 15);
      const u8* row8 = piece + (size_t)(g + 8) * p.pitch + (((uintptr_t)p.w + o8) & 15);
      f.load(row0, row8, lane, min(8, (p.cols - 256 * step) / 32));
    }
    __syncwarp();
    issue_w();
    const u8* xb = xw + (size_t)(k & 1) * p.xbuf_bytes;
    const u8* xl = xb + (lane & 7) * MD_XPITCH + 16 * (lane >> 3);
    const u8* scl = xb + (FMT == ILL_Q4_K ? p.xsum_off : p.xs_off) + 2 * t * SP;
    const float* ys = (const float*)(xb + p.xs_off) + 2 * t;
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      uint32_t x[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) ldsm4(x[j], xl + 8 * nt * MD_XPITCH + 64 * j);
      float ya = 0.0f, yb = 0.0f;
      if constexpr (KQ) { ya = ys[8 * nt]; yb = ys[8 * nt + 1]; }
      f.apply(x, scl + 8 * nt * SP, scl + (8 * nt + 1) * SP, ya, yb, acc[nt]);
    }
    __syncwarp();  // every lane is through with buffer k % 2 before the next iteration's copies into it are issued
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (dead) {
    // copies still in flight into this warp's stages get a bounded time to land before shared memory is released
    for (int k = done; k < issued; ++k) mbar_wait(&full[k % stages], (uint32_t)(k / stages) & 1u, nullptr, 0);
  }
  // the warps' partial sums meet: thread (row, token) adds them in warp order
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      part[(warp * 16 + g + 8 * (i >> 1)) * TN + 8 * nt + 2 * t + (i & 1)] = dead ? 0.0f : acc[nt][i];
  if (__syncthreads_or(dead)) return;  // a warp gave up (status word set): the tile is not stored
  for (int o = tid; o < 16 * TN; o += MD_THREADS) {
    const int r = o / TN, tk = o - r * TN;
    const long long row = row_base + r;
    const int tok = tok0 + tk;
    if (row < p.rows && tok < p.n) {
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < MD_WARPS; ++w) v = __fadd_rn(v, part[(w * 16 + r) * TN + tk]);
      if (p.bias) v += p.bias[row];
      float* yp = p.y + (long long)tok * p.rows + row;
      *yp = p.acc ? *yp + v : v;
    }
  }
}

template <int FMT>
static int mmd_launch(const MdParams& p, int tn, size_t smem, int grid, cudaStream_t st) {
  const void* k = tn == 32 ? (const void*)mmd_kernel<FMT, 4, 1> : tn == 64 ? (const void*)mmd_kernel<FMT, 8, 2> : (const void*)mmd_kernel<FMT, 16, 1>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  MdParams pp = p;
  void* args[] = {&pp};
  return launch_kernel(k, dim3(grid), dim3(32 * p.warps), smem, args, st);
}

// The chunk product on the tensor cores, for the formats and layouts it is written for; ILL_ERR_UNSUPPORTED
// otherwise (the caller then takes the token loop of the CUDA-core kernel).
int mmd_try(int fmt, uint64_t w, int rows, int cols, uint64_t xq, uint64_t xs, uint64_t xsum, uint64_t y, uint64_t bias, int acc,
            int n, void* stream) {
  if (fmt != ILL_Q8_0 && fmt != ILL_Q4_K && fmt != ILL_Q6_K) return ILL_ERR_UNSUPPORTED;
  if (n < 2) return ILL_ERR_UNSUPPORTED;
  const bool kq = fmt != ILL_Q8_0;
  // 16-byte pieces of the activations are copied as they lie: the quants of a step, eight Q8_0 scales Q4_K's sixteen sums
  if (xq & 15) return ILL_ERR_UNSUPPORTED;
  if (kq ? cols % 256 != 0 : ((xs & 15) || cols % 128)) return ILL_ERR_UNSUPPORTED;
  if (fmt == ILL_Q4_K && (xsum & 15)) return ILL_ERR_UNSUPPORTED;
  const int bw = fmt_block_weights(fmt), bb = fmt_block_bytes(fmt);
  MdParams p = {};
  p.w = (const u8*)(uintptr_t)w;
  p.rows = rows;
  p.cols = cols;
  p.row_bytes = cols / bw * bb;
  p.nsteps = (cols + 255) / 256;
  p.xq = (const i8*)(uintptr_t)xq;
  p.xs = (const float*)(uintptr_t)xs;
  p.xsum = (const int16_t*)(uintptr_t)xsum;
  p.y = (float*)(uintptr_t)y;
  p.bias = (const float*)(uintptr_t)bias;
  p.acc = acc;
  p.n = n;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  // Tokens a CTA: 128 amortize a block's unpacking best (one CTA of eight warps an SM, up to 255 registers); tiles
  // of 64 keep a thread within 128 registers so that two CTAs share an SM -- measured equal to slower where both
  // fill the machine, so they are for chunks of up to 64 tokens and for matrices with so few rows that tiles of 128
  // would leave the SMs with fewer than eight warps each; 32 below that.
  int tn = n <= 32 ? 32 : n <= 64 ? 64 : 128;
  while (tn > 32 && (long long)((rows + 15) / 16) * ((n + tn - 1) / tn) < 8ll * sms) tn >>= 1;
  // Warps a CTA: eight (128 rows), fewer when that would leave SMs without a CTA (few rows of many columns)
  p.warps = MD_WARPS;
  while (p.warps > 1 && (long long)((rows + 16 * p.warps - 1) / (16 * p.warps)) * ((n + tn - 1) / tn) < sms) p.warps >>= 1;
  // a row's step: its 16-byte aligned span (a block is read from its stage once a step, so the rows' pitch need not
  // spread them over the banks); 16 bytes after the last row for the unaligned loads' second word
  const int sb = fmt == ILL_Q8_0 ? 272 : bb;
  p.pitch = (sb + 15 + 15) / 16 * 16;
  p.stage_bytes = (uint32_t)(16 * p.pitch + 16);
  uint32_t off = (uint32_t)tn * MD_XPITCH;
  p.xs_off = off;
  off += kq ? 4u * tn : (uint32_t)tn * MdFrag<ILL_Q8_0>::SPITCH;
  off = (off + 15) / 16 * 16;
  p.xsum_off = off;
  if (fmt == ILL_Q4_K) off += (uint32_t)tn * MdFrag<ILL_Q4_K>::SPITCH;
  p.xbuf_bytes = (off + 127) / 128 * 128;
  p.ring_off = 2 * p.xbuf_bytes;
  // three stages a ring where two CTAs still fit an SM with them (or where one CTA has the SM anyway), else two
  const size_t ring1 = (size_t)p.warps * p.stage_bytes, two_ctas = (233472 / 2 - 1024 - 256);
  p.stages = (tn == 128 || p.ring_off + 3 * ring1 <= two_ctas) ? 3 : 2;
  const size_t smem = p.ring_off + (size_t)p.stages * ring1;
  if (smem > 226 * 1024) return ILL_ERR_UNSUPPORTED;
  p.status = device_status_word();
  const long long grid = (long long)((rows + 16 * p.warps - 1) / (16 * p.warps)) * ((n + tn - 1) / tn);
  if (grid > 0x7fffffffll) return ILL_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (fmt) {
    case ILL_Q8_0: return mmd_launch<ILL_Q8_0>(p, tn, smem, (int)grid, st);
    case ILL_Q4_K: return mmd_launch<ILL_Q4_K>(p, tn, smem, (int)grid, st);
    default: return mmd_launch<ILL_Q6_K>(p, tn, smem, (int)grid, st);
  }
}

template <int FMT>
static int mmk_launch(const MdParams& p, int tn, size_t smem, int grid, cudaStream_t st) {
  const void* k = tn == 8 ? (const void*)mmk_kernel<FMT, 1> : (const void*)mmk_kernel<FMT, 2>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e);
  MdParams pp = p;
  void* args[] = {&pp};
  return launch_kernel(k, dim3(grid), dim3(MD_THREADS), smem, args, st);
}

// Up to sixteen tokens with the columns dealt to a CTA's warps (mmk_kernel): for rows of many columns.
int mmk_try(int fmt, uint64_t w, int rows, int cols, uint64_t xq, uint64_t xs, uint64_t xsum, uint64_t y, uint64_t bias, int acc,
            int n, void* stream) {
  if (fmt != ILL_Q8_0 && fmt != ILL_Q4_K && fmt != ILL_Q6_K) return ILL_ERR_UNSUPPORTED;
  if (n < 2 || n > 16) return ILL_ERR_UNSUPPORTED;
  const bool kq = fmt != ILL_Q8_0;
  if (xq & 15) return ILL_ERR_UNSUPPORTED;
  if (kq ? cols % 256 != 0 : ((xs & 15) || cols % 128)) return ILL_ERR_UNSUPPORTED;
  if (fmt == ILL_Q4_K && (xsum & 15)) return ILL_ERR_UNSUPPORTED;
  const int bw = fmt_block_weights(fmt), bb = fmt_block_bytes(fmt);
  MdParams p = {};
  p.w = (const u8*)(uintptr_t)w;
  p.rows = rows;
  p.cols = cols;
  p.row_bytes = cols / bw * bb;
  p.nsteps = (cols + 255) / 256;
  if (p.nsteps < 2 * MD_WARPS) return ILL_ERR_UNSUPPORTED;  // too few steps to deal out
  p.xq = (const i8*)(uintptr_t)xq;
  p.xs = (const float*)(uintptr_t)xs;
  p.xsum = (const int16_t*)(uintptr_t)xsum;
  p.y = (float*)(uintptr_t)y;
  p.bias = (const float*)(uintptr_t)bias;
  p.acc = acc;
  p.n = n;
  p.warps = MD_WARPS;
  const int tn = n <= 8 ? 8 : 16;
  const int sb = fmt == ILL_Q8_0 ? 272 : bb;
  p.pitch = (sb + 15 + 15) / 16 * 16;
  p.stage_bytes = (uint32_t)(16 * p.pitch + 16);
  uint32_t off = (uint32_t)tn * MD_XPITCH;
  p.xs_off = off;
  off += kq ? 4u * tn : (uint32_t)tn * MdFrag<ILL_Q8_0>::SPITCH;
  off = (off + 15) / 16 * 16;
  p.xsum_off = off;
  if (fmt == ILL_Q4_K) off += (uint32_t)tn * MdFrag<ILL_Q4_K>::SPITCH;
  p.xbuf_bytes = (off + 127) / 128 * 128;
  p.ring_off = 2 * MD_WARPS * p.xbuf_bytes;
  p.stages = MD_MAX_STAGES;
  p.part_off = (uint32_t)((p.ring_off + (size_t)MD_WARPS * p.stages * p.stage_bytes + 127) / 128 * 128);
  const size_t smem = p.part_off + (size_t)MD_WARPS * 16 * tn * 4;
  if (smem > 226 * 1024) return ILL_ERR_UNSUPPORTED;
  p.status = device_status_word();
  const long long grid = (long long)((rows + 15) / 16) * ((n + tn - 1) / tn);
  if (grid > 0x7fffffffll) return ILL_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (fmt) {
    case ILL_Q8_0: return mmk_launch<ILL_Q8_0>(p, tn, smem, (int)grid, st);
    case ILL_Q4_K: return mmk_launch<ILL_Q4_K>(p, tn, smem, (int)grid, st);
    default: return mmk_launch<ILL_Q6_K>(p, tn, smem, (int)grid, st);
  }
}

}  // namespace ill
