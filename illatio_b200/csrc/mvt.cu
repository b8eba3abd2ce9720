// mvt.cu -- a quantized matrix times a few tokens (2 .. 16) with the weights read once: the integer
// block dots on the tensor cores' int8 path instead of one dp4a pass per token.
//
// At 2-16 tokens the product is still bound by the weights' bytes, but on CUDA cores every token costs a full
// pass of dp4a over the unpacked weights (mvn_kernel: batch 16 took 22-30 times the time of batch 1).  Here a warp
// holds 16 weight rows x one block of columns as the A operand of mma.sync (m16n8k32 / m16n8k16, u8 or s8
// weights, s8 activations, s32 accumulate) and the tokens as B, eight a tile: the weights are unpacked once
// whatever the number of tokens.  The integers are the CPU kernels' (exact); each block's sum meets its float
// scales as in the reference's portable loops (src/tensor.lisp:321-336, src/kquant.lisp:171-236).
//
//   * A persistent CTA of eight warps stages the tokens' quantized activations in shared memory once (token
//     stride padded by 16 bytes, so that the eight tokens of a B fragment sit on different banks), then walks
//     tiles of 16 rows.  The eight warps share a tile's blocks (warp w takes blocks w, w + 8, ...): small matrices
//     still fill the SMs.  Each warp streams its (tile, block) pieces -- 16 row segments, a bulk copy each, issued
//     by 16 lanes -- through its own ring of stages, across tile boundaries.
//   * A tile's partial sums (a float per row, token and warp) meet in shared memory in a fixed order.
//
// mma.sync is the legacy tensor path: right here, where N is 8 or 16 and the bound is HBM; the chunk-sized
// products (hundreds of rows of X an expert) use tcgen05 (mm_id.cu).
//
// Replaces mv_q8_n / mm_q8_mma's small-batch use and mv_k's token loop behind CMAT-MUL-N
// (src/cuda-dense.lisp:220-255; src/cuda/dense.cu:643-885, src/cuda/kquant.cu:169-466) for Q8_0, Q4_K and Q6_K.
#include "formats.cuh"
#include "host.h"
#include "mma_i8.cuh"

namespace ill {

// A tile's columns are split over a group of eight warps; a CTA holds one or two groups (a tile each at a time)
// that share the staged activations, and each warp a ring of two to four stages.
constexpr int MT_WARPS = 8, MT_GROUP_THREADS = 32 * MT_WARPS, MT_ROWS = 16, MT_MAX_STAGES = 4, MT_MAX_GROUPS = 2;

struct MtParams {
  const u8* w;
  int rows, cols, row_bytes, nblocks;  // blocks a row
  int cb, npieces;      // blocks a staged piece (a warp's unit of copying); pieces a row
  const i8* xq;
  const float* xs;
  const int16_t* xsum;
  float* y;
  const float* bias;
  int acc, n;
  int pitch;            // bytes between the rows of a staged piece
  uint32_t stage_bytes;
  int stages, groups;   // stages a warp's ring; groups of eight warps a CTA
  int x_stride;         // bytes between the tokens' quants in shared memory
  uint32_t xs_off, bs_off, ring_off, part_off;
  unsigned* status;
};


// The tokens' activations in shared memory.
struct MtX {
  const i8* q;        // token t's quants at q + t * stride
  int stride;
  const float* s;     // [t][scales a token]
  const int16_t* bs;  // [t][sums a token]: Q4_K sums of 32, Q6_K sums of 16
  int nsc, nbs, n;
};
// the B fragment's word: token TOK's quants K .. K+3 (the tokens past the last are staged as zeros)
__device__ __forceinline__ uint32_t xword(const MtX& x, int tok, int k) {
  return *(const uint32_t*)(x.q + (size_t)tok * x.stride + k);
}

// ---- one block of 16 rows against the tokens: ACC[nt][i] += ... --------------------------------------
// ROW0 / ROW8: the block's bytes of rows g and g + 8 of the tile (g = lane / 4) in the staged piece; BLK the
// block's number in the row; NT8 tiles of eight tokens.  Output i of a tile: row g + 8 (i / 2), token 8 nt + 2 (lane % 4) + i % 2.
template <int FMT, int NT8> struct MtBlock;

template <int NT8> struct MtBlock<ILL_Q8_0, NT8> {
  static constexpr int BS_PER = 0;
  __device__ static void run(const u8* row0, const u8* row8, int blk, const MtX& x, int lane, float (&acc)[NT8][4]) {
    const int g = lane >> 2, t4 = 4 * (lane & 3);
    uint32_t a[4];
    a[0] = lds32u(row0 + 2 + t4); a[1] = lds32u(row8 + 2 + t4); a[2] = lds32u(row0 + 18 + t4); a[3] = lds32u(row8 + 18 + t4);
    const float d0 = ldh(row0), d8 = ldh(row8);
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      uint32_t b[2] = {xword(x, 8 * nt + g, 32 * blk + t4), xword(x, 8 * nt + g, 32 * blk + 16 + t4)};
      int c[4] = {0, 0, 0, 0};
      mma_k32(c, a, b, false);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = 8 * nt + 2 * (lane & 3) + (i & 1);
        const float xs = x.s[tok * x.nsc + blk];
        // Q8-ROW-DOT-AT: sum += float(isum) * (d_w * d_x)
        acc[nt][i] = __fadd_rn(acc[nt][i], __fmul_rn((float)c[i], __fmul_rn(i < 2 ? d0 : d8, xs)));
      }
    }
  }
};

template <int NT8> struct MtBlock<ILL_Q4_K, NT8> {
  static constexpr int BS_PER = 8;  // sums of 32 a block
  __device__ static void run(const u8* row0, const u8* row8, int blk, const MtX& x, int lane, float (&acc)[NT8][4]) {
    const int g = lane >> 2, t4 = 4 * (lane & 3);
    int isum[NT8][4], imin[NT8][4];
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) isum[nt][i] = imin[nt][i] = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // 64 weights: groups 2k (low nibbles) and 2k + 1 (high)
      const uint32_t w0 = lds32u(row0 + 16 + 32 * k + t4), w1 = lds32u(row8 + 16 + 32 * k + t4);
      const uint32_t w2 = lds32u(row0 + 32 + 32 * k + t4), w3 = lds32u(row8 + 32 + 32 * k + t4);
      const uint32_t lo[4] = {w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, w2 & 0x0F0F0F0Fu, w3 & 0x0F0F0F0Fu};
      const uint32_t hi[4] = {(w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu, (w2 >> 4) & 0x0F0F0F0Fu, (w3 >> 4) & 0x0F0F0F0Fu};
      int sc0[2], mn0[2], sc8[2], mn8[2];
      scale_min_k4(row0 + 4, 2 * k, sc0[0], mn0[0]); scale_min_k4(row0 + 4, 2 * k + 1, sc0[1], mn0[1]);
      scale_min_k4(row8 + 4, 2 * k, sc8[0], mn8[0]); scale_min_k4(row8 + 4, 2 * k + 1, sc8[1], mn8[1]);
#pragma unroll
      for (int nt = 0; nt < NT8; ++nt) {
        const int kb = 256 * blk + 64 * k + t4;
        uint32_t b0[2] = {xword(x, 8 * nt + g, kb), xword(x, 8 * nt + g, kb + 16)};
        uint32_t b1[2] = {xword(x, 8 * nt + g, kb + 32), xword(x, 8 * nt + g, kb + 48)};
        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
        mma_k32(c0, lo, b0, true);
        mma_k32(c1, hi, b1, true);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = 8 * nt + 2 * (lane & 3) + (i & 1);
          isum[nt][i] += c0[i] * (i < 2 ? sc0[0] : sc8[0]) + c1[i] * (i < 2 ? sc0[1] : sc8[1]);
          const int bsp = *(const int*)(x.bs + tok * x.nbs + 8 * blk + 2 * k);  // the two groups' sums of 32
          imin[nt][i] = dp2a_lo(bsp, (i < 2 ? mn0[0] : mn8[0]) | ((i < 2 ? mn0[1] : mn8[1]) << 8), imin[nt][i]);
        }
      }
    }
    const float d0 = ldh(row0), m0 = ldh(row0 + 2), d8 = ldh(row8), m8 = ldh(row8 + 2);
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = 8 * nt + 2 * (lane & 3) + (i & 1);
        const float yd = x.s[tok * x.nsc + blk];
        // Q4K-ROW-DOT: sum -= (yd * dmin) * imin; sum += (yd * d) * isum
        float s = __fsub_rn(acc[nt][i], __fmul_rn(__fmul_rn(yd, i < 2 ? m0 : m8), (float)imin[nt][i]));
        acc[nt][i] = __fadd_rn(s, __fmul_rn(__fmul_rn(yd, i < 2 ? d0 : d8), (float)isum[nt][i]));
      }
  }
};

template <int NT8> struct MtBlock<ILL_Q6_K, NT8> {
  static constexpr int BS_PER = 16;  // a block's sixteen sums of 16, staged as two bytes each: (sum >> 4, sum & 15)
  __device__ static void run(const u8* row0, const u8* row8, int blk, const MtX& x, int lane, float (&acc)[NT8][4]) {
    const int g = lane >> 2, t4 = 4 * (lane & 3);
    int isum[NT8][4];
    const signed char* sc0 = (const signed char*)(row0 + 192);
    const signed char* sc8 = (const signed char*)(row8 + 192);
    {
      // The quants are 0..63: their -32 comes off as 32 * sum over the groups of scale * (the activations' sum of
      // the group) -- itself a product of the block's 16 x 16 scales with the tokens' sums, taken on the tensor
      // cores with each sum split in two int8 halves: sum = 16 * (sum >> 4) + (sum & 15).
      const uint32_t s0 = lds32u(row0 + 192 + t4), s8 = lds32u(row8 + 192 + t4);
      const u8* hl = (const u8*)x.bs;
#pragma unroll
      for (int nt = 0; nt < NT8; ++nt) {
        const u8* b = hl + ((size_t)(8 * nt + g) * x.nbs + 16 * blk) * 2;
        int hi[4] = {0, 0, 0, 0}, lo[4] = {0, 0, 0, 0};
        mma_k16_s8(hi, s0, s8, *(const uint32_t*)(b + t4), false);
        mma_k16_s8(lo, s0, s8, *(const uint32_t*)(b + 16 + t4), true);
#pragma unroll
        for (int i = 0; i < 4; ++i) isum[nt][i] = -32 * (16 * hi[i] + lo[i]);
      }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c)      // half of the block: 128 weights
#pragma unroll
      for (int is = 0; is < 2; ++is) {  // weights l = 16 is .. 16 is + 15 of each of the half's four runs of 32
        const int l = 16 * is + t4;
        uint32_t q[2][4];  // [row g / g + 8][run]: the lane's four 6-bit quants of each run
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const u8* row = r ? row8 : row0;
          const uint32_t A = lds32u(row + 64 * c + l), B = lds32u(row + 64 * c + 32 + l), H = lds32u(row + 128 + 32 * c + l);
          q[r][0] = (A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u);
          q[r][1] = (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u);
          q[r][2] = ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u);
          q[r][3] = ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int run = 0; run < 4; ++run) {
          const int grp = 8 * c + 2 * run + is;  // the group of 16 and its scale
          const int s0 = sc0[grp], s8 = sc8[grp];
#pragma unroll
          for (int nt = 0; nt < NT8; ++nt) {
            int cc[4] = {0, 0, 0, 0};
            mma_k16_u8(cc, q[0][run], q[1][run], xword(x, 8 * nt + g, 256 * blk + 128 * c + 32 * run + l));
#pragma unroll
            for (int i = 0; i < 4; ++i) isum[nt][i] += cc[i] * (i < 2 ? s0 : s8);
          }
        }
      }
    const float d0 = ldh(row0 + 208), d8 = ldh(row8 + 208);
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = 8 * nt + 2 * (lane & 3) + (i & 1);
        const float yd = x.s[tok * x.nsc + blk];
        // Q6K-ROW-DOT: sum += (d * yd) * float(isum - 32 imins)
        acc[nt][i] = __fadd_rn(acc[nt][i], __fmul_rn(__fmul_rn(i < 2 ? d0 : d8, yd), (float)isum[nt][i]));
      }
  }
};

// the meeting of one group's eight warps (barrier 1 + group), with an OR over a flag
__device__ __forceinline__ bool group_sync_or(int grp, bool flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %2, 0;\n\t"
      "barrier.cta.red.or.pred.aligned p, %1, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(1 + grp), "r"((uint32_t)flag), "n"(MT_GROUP_THREADS)
      : "memory");
  return out != 0;
}

template <int FMT, int NT8>
__global__ void __launch_bounds__(MT_GROUP_THREADS * MT_MAX_GROUPS) mvt_kernel(const MtParams p) {
  extern __shared__ __align__(128) u8 smem[];
  constexpr int BB = Fmt<FMT>::BB, BW = Fmt<FMT>::BW;
  const int tid = threadIdx.x, lane = tid & 31, cwarp = tid >> 5;  // the warp's number in the CTA
  const int warp = cwarp & (MT_WARPS - 1), grp = cwarp / MT_WARPS, gtid = tid & (MT_GROUP_THREADS - 1);
  const int nthreads = blockDim.x, stages = p.stages;
  const int tile0 = blockIdx.x * p.groups + grp, tile_step = gridDim.x * p.groups;
  i8* xq_s = (i8*)smem;
  float* xs_s = (float*)(smem + p.xs_off);
  int16_t* bs_s = (int16_t*)(smem + p.bs_off);
  u8* ring = smem + p.ring_off + (size_t)cwarp * stages * p.stage_bytes;
  float* part = (float*)(smem + p.part_off) + (size_t)grp * 2 * MT_WARPS * 256;  // [group][2][warps][16 rows][16 tokens]
  __shared__ uint64_t full_s[MT_MAX_GROUPS * MT_WARPS * MT_MAX_STAGES];
  uint64_t* full = full_s + cwarp * MT_MAX_STAGES;

  const int ntiles = (p.rows + MT_ROWS - 1) / MT_ROWS;
  const int nb = p.nblocks, cb = p.cb, np = p.npieces;
  // this warp's pieces in order: its group's tiles tile0, + tile_step, ...; of each the pieces warp, warp + 8, ...
  int i_tile = tile0, i_blk = warp, issued = 0;  // i_blk counts pieces
  auto issue_next = [&]() {  // all lanes; lanes 0..15 copy a row segment each
    while (i_tile < ntiles && i_blk >= np) { i_tile += tile_step; i_blk = warp; }
    if (i_tile >= ntiles) return;
    const int s = issued % stages;
    const int row = i_tile * MT_ROWS + lane;
    uint32_t bytes = 0;
    const u8* src = nullptr;
    if (lane < MT_ROWS && row < p.rows) {
      src = p.w + (long long)row * p.row_bytes + (long long)i_blk * cb * BB;
      const uint32_t len = (uint32_t)min(cb, nb - i_blk * cb) * BB;
      bytes = (uint32_t)((((uintptr_t)src + len + 15) & ~(uintptr_t)15) - ((uintptr_t)src & ~(uintptr_t)15));
    }
    uint32_t total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) mbar_expect_tx(&full[s], total);
    __syncwarp();
    if (bytes) bulk_g2s(ring + (size_t)s * p.stage_bytes + (size_t)lane * p.pitch, (const void*)((uintptr_t)src & ~(uintptr_t)15), bytes, &full[s]);
    ++issued;
    i_blk += MT_WARPS;
  };
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  for (int s = 0; s < stages; ++s) issue_next();  // the weights do not depend on the previous kernel
  pdl_launch_dependents();
  pdl_wait();

  // the tokens' activations -> shared memory, the tokens past the last (up to a whole tile of eight) as zeros
  const int nsc = p.cols / BW, nbs = MtBlock<FMT, NT8>::BS_PER * (p.cols / 256);
  constexpr int NTOK = 8 * NT8;
  for (int i = tid; i < NTOK * (p.cols / 16); i += nthreads) {
    const int t = i / (p.cols / 16), j = i - t * (p.cols / 16);
    *(uint4*)(xq_s + (size_t)t * p.x_stride + 16 * j) = t < p.n ? ((const uint4*)(p.xq + (size_t)t * p.cols))[j] : make_uint4(0, 0, 0, 0);
  }
  for (int i = tid; i < NTOK * nsc; i += nthreads) xs_s[i] = i < p.n * nsc ? p.xs[i] : 0.0f;
  if constexpr (FMT == ILL_Q4_K) {
    for (int i = tid; i < NTOK * nbs; i += nthreads) {  // sums of 32: pairs of the sums of 16
      const int t = i / nbs, j = i - t * nbs;
      const int16_t* b = p.xsum + (size_t)t * (p.cols / 16) + 2 * j;
      bs_s[i] = t < p.n ? (int16_t)(b[0] + b[1]) : (int16_t)0;
    }
  } else if constexpr (FMT == ILL_Q6_K) {
    // per block 32 bytes: the sixteen sums' high parts (sum >> 4, signed), then their low parts (sum & 15)
    u8* hl = (u8*)bs_s;
    for (int i = tid; i < NTOK * nbs; i += nthreads) {
      const int t = i / nbs, j = i - t * nbs, b = j >> 4, gq = j & 15;
      const int v = t < p.n ? (int)p.xsum[(size_t)t * (p.cols / 16) + j] : 0;
      hl[((size_t)t * nbs + 16 * b) * 2 + gq] = (u8)(signed char)(v >> 4);
      hl[((size_t)t * nbs + 16 * b) * 2 + 16 + gq] = (u8)(v & 15);
    }
  }
  __syncthreads();
  MtX x;
  x.q = xq_s; x.stride = p.x_stride; x.s = xs_s; x.bs = bs_s; x.nsc = nsc; x.nbs = nbs; x.n = p.n;

  const int g = lane >> 2;
  int done = 0, it = 0;
  bool dead = false;
  for (int tile = tile0; tile < ntiles; tile += tile_step, ++it) {
    float acc[NT8][4];
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    for (int pc = warp; pc < np && !dead; pc += MT_WARPS) {
      const int s = done % stages;
      bool ok = mbar_wait(&full[s], (uint32_t)(done / stages) & 1u, p.status, ST_MV_WAIT + 0x20 + FMT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { dead = true; break; }
      const u8* piece = ring + (size_t)s * p.stage_bytes;
      // a row's segment starts where its block starts inside the 16-byte aligned span that was copied
      const long long o0 = (long long)(tile * MT_ROWS + g) * p.row_bytes + (long long)pc * cb * BB;
      const long long o8 = o0 + 8ll * p.row_bytes;
      const u8* row0 = piece + (size_t)g * p.pitch + (((uintptr_t)p.w + o0) & 15);
      const u8* row8 = piece + (size_t)(g + 8) * p.pitch + (((uintptr_t)p.w + o8) & 15);
      const int nhere = min(cb, nb - pc * cb);
      for (int j = 0; j < nhere; ++j) MtBlock<FMT, NT8>::run(row0 + j * BB, row8 + j * BB, pc * cb + j, x, lane, acc);
      __syncwarp();
      ++done;
      issue_next();
    }
    // the eight warps' partial sums meet: thread (row, token) adds them in warp order
    float* mine = part + (size_t)(it & 1) * MT_WARPS * 256 + warp * 256;
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) mine[(g + 8 * (i >> 1)) * 16 + 8 * nt + 2 * (lane & 3) + (i & 1)] = acc[nt][i];
    if (group_sync_or(grp, dead)) { dead = true; break; }
    {
      const int r = gtid >> 4, t = gtid & 15;
      const long long row = (long long)tile * MT_ROWS + r;
      if (t < p.n && row < p.rows) {
        const float* all = part + (size_t)(it & 1) * MT_WARPS * 256 + r * 16 + t;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < MT_WARPS; ++w) v = __fadd_rn(v, all[w * 256]);
        if (p.bias) v += p.bias[row];
        float* yp = p.y + (long long)t * p.rows + row;
        *yp = p.acc ? *yp + v : v;
      }
    }
  }
  if (dead) {
    // copies still in flight into this warp's stages get a bounded time to land before shared memory is released
    for (int k = done + 1; k < issued; ++k) mbar_wait(&full[k % stages], (uint32_t)(k / stages) & 1u, nullptr, 0);
  }
}

template <int FMT>
static int mvt_launch(const MtParams& p, size_t smem, int grid, cudaStream_t st) {
  const void* k = p.n <= 8 ? (const void*)mvt_kernel<FMT, 1> : (const void*)mvt_kernel<FMT, 2>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  MtParams pp = p;
  void* args[] = {&pp};
  return launch_kernel(k, dim3(grid), dim3(MT_GROUP_THREADS * p.groups), smem, args, st);
}

// The several-token product on the tensor cores, for the formats it is written for; ILL_ERR_UNSUPPORTED
// otherwise (the caller then takes the CUDA-core kernel).
int mvt_try(int fmt, uint64_t w, int rows, int cols, uint64_t xq, uint64_t xs, uint64_t xsum, uint64_t y, uint64_t bias, int acc,
            int n, void* stream) {
  if (fmt != ILL_Q8_0 && fmt != ILL_Q4_K && fmt != ILL_Q6_K) return ILL_ERR_UNSUPPORTED;
  if (n < 2 || n > 16) return ILL_ERR_UNSUPPORTED;
  const int bw = fmt_block_weights(fmt), bb = fmt_block_bytes(fmt);
  MtParams p = {};
  p.w = (const u8*)(uintptr_t)w;
  p.rows = rows;
  p.cols = cols;
  p.nblocks = cols / bw;
  p.row_bytes = p.nblocks * bb;
  p.xq = (const i8*)(uintptr_t)xq;
  p.xs = (const float*)(uintptr_t)xs;
  p.xsum = (const int16_t*)(uintptr_t)xsum;
  p.y = (float*)(uintptr_t)y;
  p.bias = (const float*)(uintptr_t)bias;
  p.acc = acc;
  p.n = n;
  // a row's segment: its block's 16-byte aligned span, rows a multiple of 16 bytes apart that is an odd multiple
  // of 16 mod 128 (eight rows x four words then sit on 32 different banks)
  // blocks a piece: about 200-300 bytes a row segment (a bulk copy each), but every warp should get a piece
  int cb = fmt == ILL_Q8_0 ? 8 : fmt == ILL_Q4_K ? 2 : 1;
  while (cb > 1 && (p.nblocks + cb - 1) / cb < MT_WARPS) cb >>= 1;
  p.cb = cb;
  p.npieces = (p.nblocks + cb - 1) / cb;
  int pitch = (cb * bb + 15 + 15) / 16 * 16;
  while ((pitch / 16) % 8 % 2 == 0) pitch += 16;
  p.pitch = pitch;
  p.stage_bytes = (uint32_t)(MT_ROWS * pitch + 16);
  p.stage_bytes = (p.stage_bytes + 127) / 128 * 128;
  p.x_stride = cols + 16;
  const int nsc = cols / bw, bs_per = fmt == ILL_Q4_K ? 8 : fmt == ILL_Q6_K ? 16 : 0;
  const uint32_t ntok = n <= 8 ? 8 : 16;  // staged tokens: whole tiles of eight
  uint32_t off = ntok * (uint32_t)p.x_stride;
  off = (off + 15) / 16 * 16;
  p.xs_off = off;
  off += 4u * ntok * nsc;
  off = (off + 15) / 16 * 16;
  p.bs_off = off;
  off += 2u * ntok * bs_per * (cols / 256);
  off = (off + 127) / 128 * 128;
  p.ring_off = off;
  // two groups with rings as deep as fit (four stages at most, two at least), else one group
  const uint32_t budget = 220u * 1024u, part_bytes = 2u * MT_WARPS * 256 * 4, ring1 = (uint32_t)MT_WARPS * p.stage_bytes;
  const int ntiles = (rows + MT_ROWS - 1) / MT_ROWS;
  p.groups = 0;
  for (int g = MT_MAX_GROUPS; g >= 1 && !p.groups; --g) {
    if (off + g * (part_bytes + 2 * ring1) > budget) continue;
    p.groups = g;
    p.stages = (int)((budget - off - g * part_bytes) / (g * ring1));
    if (p.stages > MT_MAX_STAGES) p.stages = MT_MAX_STAGES;
  }
  if (!p.groups) return ILL_ERR_UNSUPPORTED;  // too many tokens of too many columns: the caller splits them
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  if (p.groups == 2 && ntiles < 2 * sms && p.stages < 3) {  // few tiles: a group a CTA spreads them over more SMs
    p.groups = 1;
    p.stages = (int)((budget - off - part_bytes) / ring1);
    if (p.stages > MT_MAX_STAGES) p.stages = MT_MAX_STAGES;
  }
  off += (uint32_t)p.groups * p.stages * ring1;
  p.part_off = off;
  off += (uint32_t)p.groups * part_bytes;
  const size_t smem = off;
  p.status = device_status_word();
  const int per_sm = (int)((227u * 1024u) / (smem + 1024u)) >= 2 ? 2 : 1;
  int grid = sms * per_sm;
  if (grid * p.groups > ntiles) grid = (ntiles + p.groups - 1) / p.groups;
  cudaStream_t st = (cudaStream_t)stream;
  switch (fmt) {
    case ILL_Q8_0: return mvt_launch<ILL_Q8_0>(p, smem, grid, st);
    case ILL_Q4_K: return mvt_launch<ILL_Q4_K>(p, smem, grid, st);
    default: return mvt_launch<ILL_Q6_K>(p, smem, grid, st);
  }
}

}  // namespace ill
