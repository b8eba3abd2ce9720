// formats.cuh -- the five GGUF block formats as the kernels read them.
//
// A "unit" is the slice of a row one lane multiplies at a time: a Q8_0 block
// (32 weights), an IQ2_XXS sub-block (32 weights), or a quarter of a Q4_K /
// Q6_K / Q2_K super-block (64 weights) chosen so that every 16- or 32-weight
// scale group lies whole inside one unit.  For each format:
//
//   XReg  one token's activations for a unit, in registers
//   WReg  the unit's weights unpacked to int8x4 words, plus its scales
//   load_x / load_w / dot
//
// Integer dots are exact (dp4a); the float steps per unit follow the reference
// CPU kernels' formulas (src/tensor.lisp:321-336, src/kquant.lisp:171-236,
// src/iquant.lisp:126-215), so results differ from them only by the order in
// which fp32 partial sums are added.  Every float step is written with the
// rounding intrinsics (no multiply-add contraction), so that a unit's value is
// the same bits in every kernel that includes this file.
//
// Weights are read from a shared-memory copy of the raw row bytes at any byte
// alignment; activations from a shared-memory copy laid out by x_layout().
#pragma once
#include "common.cuh"

namespace ill {

template <int FMT> struct Fmt;
template <> struct Fmt<ILL_Q8_0>    { static constexpr int BB = 34,  BW = 32,  UW = 32, UPB = 1; };
template <> struct Fmt<ILL_Q4_K>    { static constexpr int BB = 144, BW = 256, UW = 64, UPB = 4; };
template <> struct Fmt<ILL_Q6_K>    { static constexpr int BB = 210, BW = 256, UW = 64, UPB = 4; };
template <> struct Fmt<ILL_Q2_K>    { static constexpr int BB = 84,  BW = 256, UW = 64, UPB = 4; };
template <> struct Fmt<ILL_IQ2_XXS> { static constexpr int BB = 66,  BW = 256, UW = 32, UPB = 8; };

__host__ __device__ inline int fmt_block_bytes(int fmt) {
  return fmt == ILL_Q8_0 ? 34 : fmt == ILL_Q4_K ? 144 : fmt == ILL_Q6_K ? 210 : fmt == ILL_Q2_K ? 84
         : fmt == ILL_IQ2_XXS ? 66 : 0;
}
__host__ __device__ inline int fmt_block_weights(int fmt) {
  return fmt == ILL_Q8_0 ? 32 : (fmt >= ILL_Q4_K && fmt <= ILL_IQ2_XXS) ? 256 : 0;
}

// One token's activations in shared memory.
struct ActS {
  const i8* q;        // quants, 16-byte aligned
  const float* s;     // one scale per 32 (Q8_0) or per 256 (Q8_K)
  const int16_t* bs;  // sums of 16 quants (Q8_K)
};

// words at an arbitrarily aligned shared-memory byte pointer (pointer arithmetic
// only, so the compiler keeps the shared address space)
template <int N>
__device__ __forceinline__ void ld_words(const u8* p, uint32_t (&out)[N]) {
  const uint32_t mis = (uint32_t)(uintptr_t)p & 3u;
  const uint32_t* b = (const uint32_t*)(p - mis);
  const uint32_t sh = mis * 8u;
  uint32_t prev = b[0];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    uint32_t next = b[i + 1];
    out[i] = __funnelshift_r(prev, next, sh);
    prev = next;
  }
}
// words at a pointer known to be 4-byte (AL 4) or 16-byte (AL 16) aligned
template <int N, int AL>
__device__ __forceinline__ void ld_words_al(const u8* p, uint32_t (&out)[N]) {
  if constexpr (AL >= 16 && N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const uint4 v = ((const uint4*)p)[i];
      out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
  } else if constexpr (AL >= 4) {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = ((const uint32_t*)p)[i];
  } else {
    ld_words<N>(p, out);
  }
}
__device__ __forceinline__ uint32_t ld_u16(const u8* p) { return *(const u16*)p; }  // p is 2-byte aligned

template <int N>
__device__ __forceinline__ void ld_x128(const i8* p, uint32_t* out) {  // N uint4 loads, 16-byte aligned
#pragma unroll
  for (int i = 0; i < N; ++i) {
    uint4 v = ((const uint4*)p)[i];
    out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
  }
}

// unsigned bytes of A times signed bytes of B, accumulated
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// two signed 16-bit halves of A times the two low signed bytes of B, accumulated
__device__ __forceinline__ int dp2a_lo(int a, int b, int c) {
  int d;
  asm("dp2a.lo.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// The IQ2_XXS codebook (256 x 8 magnitudes) and the sign patterns expanded to byte masks (0xFF where the weight
// is negative), in shared memory, IQ_COPIES interleaved copies each (entry e of copy c at [IQ_COPIES e + c]).  A
// lane reads copy lane % 16: a 64-bit request is served half a warp at a time, and the sixteen lanes of a half then
// sit on sixteen different pairs of banks whatever entries they ask for -- no bank conflicts, where eight copies
// still left 60% of the wavefronts to them.  GRID / SMASK point at the lane's copy.
constexpr int IQ_COPIES = 16;
constexpr int IQ_TABLE_BYTES = IQ_COPIES * (256 + 128) * 8;
struct IqTables { const uint2* grid; const uint2* smask; };

template <int FMT> struct XReg;  // one token's activations for a unit
template <int FMT> struct WReg;  // a unit's weights, unpacked
template <int FMT> struct UPos;  // where a unit lies in its row: byte offsets and shifts, fixed per lane

// ---- Q8_0: unit = block ------------------------------------------------------
template <> struct XReg<ILL_Q8_0> { uint32_t q[8]; float s; };
template <> struct WReg<ILL_Q8_0> { uint32_t q[8]; float d; };
template <> struct UPos<ILL_Q8_0> { int off; };

__device__ __forceinline__ void unit_pos(UPos<ILL_Q8_0>& o, int u) { o.off = 34 * u; }
__device__ __forceinline__ void load_x(XReg<ILL_Q8_0>& x, const ActS& a, int u) {
  ld_x128<2>(a.q + 32 * u, x.q);
  x.s = a.s[u];
}
template <int AL = 1>
__device__ __forceinline__ void load_w(WReg<ILL_Q8_0>& w, const u8* row, const UPos<ILL_Q8_0>& o, const IqTables&) {
  const u8* p = row + o.off;
  w.d = h2f(ld_u16(p));
  ld_words<8>(p + 2, w.q);
}
__device__ __forceinline__ float dot(const WReg<ILL_Q8_0>& w, const XReg<ILL_Q8_0>& x) {
  int a0 = 0, a1 = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a0 = __dp4a((int)w.q[i], (int)x.q[i], a0);
    a1 = __dp4a((int)w.q[4 + i], (int)x.q[4 + i], a1);
  }
  return __fmul_rn((float)(a0 + a1), __fmul_rn(w.d, x.s));
}

// ---- Q4_K: unit = 64 weights (groups 2k and 2k+1 of a super-block) ------------
// bsp packs the two groups' activation sums as int16 halves for dp2a.
template <> struct XReg<ILL_Q4_K> { uint32_t q[16]; float d; int bsp; };
template <> struct WReg<ILL_Q4_K> { uint32_t q[8]; float d, dmin; uint32_t sc, mn; };  // sc, mn: two bytes each
template <> struct UPos<ILL_Q4_K> { int off, qoff, sh; bool high; };

__device__ __forceinline__ void unit_pos(UPos<ILL_Q4_K>& o, int u) {
  const int k = u & 3;
  o.off = 144 * (u >> 2);
  o.qoff = o.off + 16 + 32 * k;
  o.sh = 16 * (k & 1);
  o.high = k >= 2;
}
__device__ __forceinline__ void load_x(XReg<ILL_Q4_K>& x, const ActS& a, int u) {
  const int i = u >> 2, k = u & 3;
  ld_x128<4>(a.q + 256 * i + 64 * k, x.q);
  x.d = a.s[i];
  const int2 b = *(const int2*)(a.bs + 16 * i + 4 * k);  // four int16 sums, 8-byte aligned
  const int bs0 = (int)(short)(b.x & 0xffff) + (b.x >> 16), bs1 = (int)(short)(b.y & 0xffff) + (b.y >> 16);
  x.bsp = (bs0 & 0xffff) | (bs1 << 16);
}
template <int AL = 1>
__device__ __forceinline__ void load_w(WReg<ILL_Q4_K>& w, const u8* row, const UPos<ILL_Q4_K>& o, const IqTables&) {
  uint32_t h[4];  // d|dmin, then the 12 scale bytes
  ld_words_al<4, AL>(row + o.off, h);
  ld_words_al<8, AL>(row + o.qoff, w.q);
  w.d = h2f(h[0] & 0xffff);
  w.dmin = h2f(h[0] >> 16);
  // get_scale_min_k4 for groups j = 2k, 2k+1 (src/kquant.lisp:64-72), both at once
  // as two bytes: j < 4 reads six bits of bytes j and j+4; j >= 4 joins the nibbles
  // of byte j+4 with the top two bits of bytes j-4 and j
  const uint32_t a = (h[1] >> o.sh) & 0xffffu, b = (h[2] >> o.sh) & 0xffffu, c = (h[3] >> o.sh) & 0xffffu;
  const uint32_t sc_lo = a & 0x3f3fu, mn_lo = b & 0x3f3fu;
  const uint32_t sc_hi = (c & 0x0f0fu) | ((a >> 2) & 0x3030u), mn_hi = ((c >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u);
  w.sc = o.high ? sc_hi : sc_lo;
  w.mn = o.high ? mn_hi : mn_lo;
}
__device__ __forceinline__ float dot(const WReg<ILL_Q4_K>& w, const XReg<ILL_Q4_K>& x) {
  // high nibbles stay in place (16 * q as an unsigned byte); the 16 comes out of the sum
  int lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    lo = __dp4a((int)(w.q[i] & 0x0F0F0F0Fu), (int)x.q[i], lo);
    hi = dp4a_us(w.q[i] & 0xF0F0F0F0u, (int)x.q[8 + i], hi);
  }
  const int isum = lo * (int)(w.sc & 0xff) + (hi >> 4) * (int)(w.sc >> 8);
  const int imin = dp2a_lo(x.bsp, (int)w.mn, 0);
  return __fsub_rn(__fmul_rn(__fmul_rn(x.d, w.d), (float)isum), __fmul_rn(__fmul_rn(x.d, w.dmin), (float)imin));
}

// ---- Q6_K: unit = half c, 16-weight column hq of each 32: four groups of 16 ------
template <> struct XReg<ILL_Q6_K> { uint32_t q[16]; float d; int bs[4]; };  // bs: 32 * the group's sum
template <> struct WReg<ILL_Q6_K> { uint32_t q[16]; float d; int sc[4]; };
template <> struct UPos<ILL_Q6_K> { int offa, offh, offs, offd, sh; };

__device__ __forceinline__ void unit_pos(UPos<ILL_Q6_K>& o, int u) {
  const int i = u >> 2, c = (u >> 1) & 1, hq = u & 1, b = 210 * i;
  o.offa = b + 64 * c + 16 * hq;
  o.offh = b + 128 + 32 * c + 16 * hq;
  o.offs = b + 192 + 8 * c;
  o.offd = b + 208;
  o.sh = 8 * hq;
}
__device__ __forceinline__ void load_x(XReg<ILL_Q6_K>& x, const ActS& a, int u) {
  const int i = u >> 2, c = (u >> 1) & 1, hq = u & 1;
  const i8* q = a.q + 256 * i + 128 * c + 16 * hq;
  const int16_t* bs = a.bs + 16 * i + 8 * c + hq;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    ld_x128<1>(q + 32 * g, x.q + 4 * g);
    x.bs[g] = 32 * (int)bs[2 * g];
  }
  x.d = a.s[i];
}
template <int AL = 1>
__device__ __forceinline__ void load_w(WReg<ILL_Q6_K>& w, const u8* row, const UPos<ILL_Q6_K>& o, const IqTables&) {
  uint32_t a[4], b[4], h[4], s[2];
  ld_words<4>(row + o.offa, a);
  ld_words<4>(row + o.offa + 32, b);
  ld_words<4>(row + o.offh, h);
  ld_words<2>(row + o.offs, s);  // the half's eight int8 scales
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w.q[j]      = (a[j] & 0x0F0F0F0Fu) | ((h[j] << 4) & 0x30303030u);
    w.q[4 + j]  = (b[j] & 0x0F0F0F0Fu) | ((h[j] << 2) & 0x30303030u);
    w.q[8 + j]  = ((a[j] >> 4) & 0x0F0F0F0Fu) | (h[j] & 0x30303030u);
    w.q[12 + j] = ((b[j] >> 4) & 0x0F0F0F0Fu) | ((h[j] >> 2) & 0x30303030u);
  }
  // scale of group g: byte hq + 2g of the eight
  const uint32_t lo = s[0] >> o.sh, hi = s[1] >> o.sh;
  w.sc[0] = (int)(signed char)(lo & 0xff);
  w.sc[1] = (int)(signed char)((lo >> 16) & 0xff);
  w.sc[2] = (int)(signed char)(hi & 0xff);
  w.sc[3] = (int)(signed char)((hi >> 16) & 0xff);
  w.d = h2f(ld_u16(row + o.offd));
}
__device__ __forceinline__ float dot(const WReg<ILL_Q6_K>& w, const XReg<ILL_Q6_K>& x) {
  int isum = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    int d = -x.bs[g];  // the quants are 0..63; their -32 comes off through the activations' sum
#pragma unroll
    for (int j = 0; j < 4; ++j) d = __dp4a((int)w.q[4 * g + j], (int)x.q[4 * g + j], d);
    isum += w.sc[g] * d;
  }
  return __fmul_rn(__fmul_rn(w.d, x.d), (float)isum);
}

// ---- Q2_K: unit = half h, 16-byte half: four groups of 16 ---------------------
template <> struct XReg<ILL_Q2_K> { uint32_t q[16]; float d; int bs01, bs23; };  // the four sums of 16 as int16 pairs
template <> struct WReg<ILL_Q2_K> { uint32_t q[4]; float d, dmin; uint32_t sc4; };  // the unit's four scale bytes
template <> struct UPos<ILL_Q2_K> { int offs, offq, offd, sh; };

__device__ __forceinline__ void unit_pos(UPos<ILL_Q2_K>& o, int u) {
  const int i = u >> 2, h = (u >> 1) & 1, half = u & 1, b = 84 * i;
  o.offs = b + 8 * h;
  o.offq = b + 16 + 32 * h + 16 * half;
  o.offd = b + 80;
  o.sh = 8 * half;
}
__device__ __forceinline__ void load_x(XReg<ILL_Q2_K>& x, const ActS& a, int u) {
  const int i = u >> 2, h = (u >> 1) & 1, half = u & 1;
  const i8* q = a.q + 256 * i + 128 * h + 16 * half;
  const int16_t* bs = a.bs + 16 * i + 8 * h + half;
#pragma unroll
  for (int k = 0; k < 4; ++k) ld_x128<1>(q + 32 * k, x.q + 4 * k);
  x.bs01 = ((int)bs[0] & 0xffff) | ((int)bs[2] << 16);
  x.bs23 = ((int)bs[4] & 0xffff) | ((int)bs[6] << 16);
  x.d = a.s[i];
}
// two signed 16-bit halves of A times the two high signed bytes of B, accumulated
__device__ __forceinline__ int dp2a_hi(int a, int b, int c) {
  int d;
  asm("dp2a.hi.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
template <int AL = 1>
__device__ __forceinline__ void load_w(WReg<ILL_Q2_K>& w, const u8* row, const UPos<ILL_Q2_K>& o, const IqTables&) {
  uint32_t s[2], dd[1];
  constexpr int A = AL >= 4 ? 4 : 1;  // an 84-byte block keeps 4-byte alignment at best
  ld_words_al<2, A>(row + o.offs, s);  // the half's eight scale bytes
  ld_words_al<4, A>(row + o.offq, w.q);
  ld_words_al<1, A>(row + o.offd, dd);
  // the unit's groups use scale bytes half, half + 2, half + 4, half + 6 of the eight: gathered into one word
  w.sc4 = __byte_perm(s[0], s[1], o.sh ? 0x7531 : 0x6420);
  w.d = h2f(dd[0] & 0xffff);
  w.dmin = h2f(dd[0] >> 16);
}
__device__ __forceinline__ float dot(const WReg<ILL_Q2_K>& w, const XReg<ILL_Q2_K>& x) {
  // The 2-bit fields are masked where they sit (unsigned bytes up to 192 against signed ones): group k's dot comes out
  // 4^k times too large, exactly, and one shift a group puts that right.  A group's dot is at most 16 * 3 * 128 in
  // magnitude, so the four fit 16 bits and meet their four scales (the low nibbles of the scale bytes) in two dp2a;
  // the mins (the high nibbles) meet the activations' sums of 16 the same way.
  int d[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    d[k] = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) d[k] = dp4a_us(w.q[j] & (0x03030303u << (2 * k)), (int)x.q[4 * k + j], d[k]);
  }
  const int p01 = (int)__byte_perm((uint32_t)d[0], (uint32_t)(d[1] >> 2), 0x5410);
  const int p23 = (int)__byte_perm((uint32_t)(d[2] >> 4), (uint32_t)(d[3] >> 6), 0x5410);
  const int sc = (int)(w.sc4 & 0x0f0f0f0fu), mn = (int)((w.sc4 >> 4) & 0x0f0f0f0fu);
  const int isum = dp2a_hi(p23, sc, dp2a_lo(p01, sc, 0));
  const int mins = dp2a_hi(x.bs23, mn, dp2a_lo(x.bs01, mn, 0));
  return __fsub_rn(__fmul_rn(__fmul_rn(x.d, w.d), (float)isum), __fmul_rn(__fmul_rn(x.d, w.dmin), (float)mins));
}

// ---- IQ2_XXS: unit = sub-block of 32 -------------------------------------------
template <> struct XReg<ILL_IQ2_XXS> { uint32_t q[8]; float d; };
template <> struct WReg<ILL_IQ2_XXS> { uint32_t q[8]; float d; float ls; };
template <> struct UPos<ILL_IQ2_XXS> { int off, qoff; };

__device__ __forceinline__ void unit_pos(UPos<ILL_IQ2_XXS>& o, int u) {
  o.off = 66 * (u >> 3);
  o.qoff = o.off + 2 + 8 * (u & 7);
}
__device__ __forceinline__ void load_x(XReg<ILL_IQ2_XXS>& x, const ActS& a, int u) {
  ld_x128<2>(a.q + 32 * u, x.q);
  x.d = a.s[u >> 3];
}
template <int AL = 1>
__device__ __forceinline__ void load_w(WReg<ILL_IQ2_XXS>& w, const u8* row, const UPos<ILL_IQ2_XXS>& o,
                                       const IqTables& t) {
  uint32_t v[2];
  ld_words<2>(row + o.qoff, v);
  const uint32_t idx = v[0], aux = v[1];
#pragma unroll
  for (int l = 0; l < 4; ++l) {
    const uint2 g = t.grid[IQ_COPIES * ((idx >> (8 * l)) & 0xff)];
    const uint2 m = t.smask[IQ_COPIES * ((aux >> (7 * l)) & 127)];
    // (g ^ m) - m per byte; g is 8, 25 or 43, never 0, so adding 1 to a flipped byte never carries
    w.q[2 * l] = (g.x ^ m.x) + (m.x & 0x01010101u);
    w.q[2 * l + 1] = (g.y ^ m.y) + (m.y & 0x01010101u);
  }
  w.ls = 0.5f + (float)(aux >> 28);
  w.d = h2f(ld_u16(row + o.off));
}
__device__ __forceinline__ float dot(const WReg<ILL_IQ2_XXS>& w, const XReg<ILL_IQ2_XXS>& x) {
  int acc = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc = __dp4a((int)w.q[i], (int)x.q[i], acc);
  return __fmul_rn(__fmul_rn(__fmul_rn(w.d, x.d), __fmul_rn((float)acc, w.ls)), 0.25f);
}

// ---- activations staged in shared memory as planes ---------------------------------
// For rows staged in column chunks the activations cannot stay in registers; they
// are read from shared memory per unit.  To keep those reads free of bank
// conflicts (consecutive lanes take consecutive units) the 16-byte pieces of a
// unit's activations are stored plane by plane: piece j of unit u at
// (j * U + u) * 16; the sums of 16 likewise, [g][u] as int16 (Q6_K, Q2_K), or
// already paired and packed per unit (Q4_K).
struct ActP {
  const u8* q;        // planes of 16-byte pieces
  const float* s;     // scales, as in ActS
  const int16_t* bs;  // planes of sums (Q6_K, Q2_K); Q4_K: packed pair sums, an int per unit
  int U;
};
template <int FMT> struct PlaneGeom;
template <> struct PlaneGeom<ILL_Q8_0>    { static constexpr int PPU = 2, BSP = 0; };
template <> struct PlaneGeom<ILL_IQ2_XXS> { static constexpr int PPU = 2, BSP = 0; };
template <> struct PlaneGeom<ILL_Q4_K>    { static constexpr int PPU = 4, BSP = 2; };  // 4 bytes a unit
template <> struct PlaneGeom<ILL_Q6_K>    { static constexpr int PPU = 4, BSP = 4; };  // 4 int16 a unit
template <> struct PlaneGeom<ILL_Q2_K>    { static constexpr int PPU = 4, BSP = 4; };

// source piece (16 bytes of the token's quants) of piece j of unit u
template <int FMT>
__device__ __forceinline__ int plane_src(int u, int j) {
  if constexpr (FMT == ILL_Q6_K || FMT == ILL_Q2_K) return 16 * (u >> 2) + 8 * ((u >> 1) & 1) + 2 * j + (u & 1);
  else return PlaneGeom<FMT>::PPU * u + j;
}
// bytes of shared memory the planes of a token with U units take (16-byte multiple)
template <int FMT>
__host__ __device__ inline uint32_t plane_bytes(int U, int nsc) {
  return (uint32_t)(PlaneGeom<FMT>::PPU * U * 16) + ((uint32_t)(4 * nsc + 15) & ~15u) +
         ((uint32_t)(PlaneGeom<FMT>::BSP * 2 * U + 15) & ~15u);
}
// Stage one token's activations (global, ActS layout) as planes at DST; all threads of the CTA.
template <int FMT>
__device__ __forceinline__ void planes_fill(u8* dst, const ActS& a, int U, int nsc, ActP& out) {
  constexpr int PPU = PlaneGeom<FMT>::PPU;
  uint4* dq = (uint4*)dst;
  for (int d = threadIdx.x; d < PPU * U; d += blockDim.x) {
    const int j = d / U, u = d - j * U;
    dq[d] = ((const uint4*)a.q)[plane_src<FMT>(u, j)];
  }
  float* ds = (float*)(dst + PPU * U * 16);
  for (int i = threadIdx.x; i < nsc; i += blockDim.x) ds[i] = a.s[i];
  int16_t* db = (int16_t*)((u8*)ds + ((4 * nsc + 15) & ~15));
  if constexpr (FMT == ILL_Q4_K) {
    int* dp = (int*)db;
    for (int u = threadIdx.x; u < U; u += blockDim.x) {
      const int16_t* b = a.bs + 4 * u;  // 16 i + 4 k with u = 4 i + k
      dp[u] = ((b[0] + b[1]) & 0xffff) | ((b[2] + b[3]) << 16);
    }
  } else if constexpr (FMT == ILL_Q6_K || FMT == ILL_Q2_K) {
    for (int d = threadIdx.x; d < 4 * U; d += blockDim.x) {
      const int g = d / U, u = d - g * U;
      db[d] = a.bs[16 * (u >> 2) + 8 * ((u >> 1) & 1) + 2 * g + (u & 1)];
    }
  }
  out.q = dst;
  out.s = ds;
  out.bs = db;
  out.U = U;
}
template <int FMT>
__device__ __forceinline__ void load_x_planes(XReg<FMT>& x, const ActP& a, int u) {
  constexpr int PPU = PlaneGeom<FMT>::PPU;
#pragma unroll
  for (int j = 0; j < PPU; ++j) {
    const uint4 v = ((const uint4*)a.q)[j * a.U + u];
    x.q[4 * j] = v.x; x.q[4 * j + 1] = v.y; x.q[4 * j + 2] = v.z; x.q[4 * j + 3] = v.w;
  }
  if constexpr (FMT == ILL_Q8_0) x.s = a.s[u];
  else if constexpr (FMT == ILL_IQ2_XXS) x.d = a.s[u >> 3];
  else {
    x.d = a.s[u >> 2];
    if constexpr (FMT == ILL_Q4_K) x.bsp = ((const int*)a.bs)[u];
    else if constexpr (FMT == ILL_Q6_K) {
#pragma unroll
      for (int g = 0; g < 4; ++g) x.bs[g] = 32 * (int)a.bs[g * a.U + u];
    } else {
      x.bs01 = ((int)a.bs[u] & 0xffff) | ((int)a.bs[a.U + u] << 16);
      x.bs23 = ((int)a.bs[2 * a.U + u] & 0xffff) | ((int)a.bs[3 * a.U + u] << 16);
    }
  }
}

// Fills the IQ2_XXS tables in shared memory (call from all threads, then sync).
__device__ __forceinline__ void iq_tables_fill(uint2* grid, uint2* smask, const uint64_t* ggrid, const u8* gsigns) {
  for (int i = threadIdx.x; i < IQ_COPIES * 256; i += blockDim.x) {
    const uint64_t g = ggrid[i / IQ_COPIES];
    grid[i] = make_uint2((uint32_t)g, (uint32_t)(g >> 32));
  }
  for (int i = threadIdx.x; i < IQ_COPIES * 128; i += blockDim.x) {
    const uint32_t s = gsigns[i / IQ_COPIES];
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if ((s >> j) & 1) lo |= 0xffu << (8 * j);
      if ((s >> (4 + j)) & 1) hi |= 0xffu << (8 * j);
    }
    smask[i] = make_uint2(lo, hi);
  }
}

// ---- one weight as a float, for rows-as-floats -----------------------------------
// The reference's dequantization, operation for operation (no fused
// multiply-add: the intrinsics round each step).
template <int FMT>
__device__ __forceinline__ float dequant_weight(const u8* __restrict__ row, int col, const uint64_t* ggrid,
                                                const u8* gsigns);

__device__ __forceinline__ float gh2f(const u8* p) { return h2f((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

template <>
__device__ __forceinline__ float dequant_weight<ILL_Q8_0>(const u8* __restrict__ row, int col, const uint64_t*,
                                                          const u8*) {
  const u8* p = row + 34 * (col >> 5);
  return __fmul_rn(gh2f(p), (float)(int)(signed char)p[2 + (col & 31)]);
}
template <>
__device__ __forceinline__ float dequant_weight<ILL_Q4_K>(const u8* __restrict__ row, int col, const uint64_t*,
                                                          const u8*) {
  const u8* p = row + 144 * (col >> 8);
  const int w = col & 255, k = w >> 6, hi = (w >> 5) & 1, l = w & 31, j = 2 * k + hi;
  const u8* q = p + 4;
  int sc, mn;
  if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
  else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
  const u8 byte = p[16 + 32 * k + l];
  const int qv = hi ? (byte >> 4) : (byte & 0xF);
  return __fsub_rn(__fmul_rn(__fmul_rn(gh2f(p), (float)sc), (float)qv), __fmul_rn(gh2f(p + 2), (float)mn));
}
template <>
__device__ __forceinline__ float dequant_weight<ILL_Q6_K>(const u8* __restrict__ row, int col, const uint64_t*,
                                                          const u8*) {
  const u8* p = row + 210 * (col >> 8);
  const int w = col & 255, c = w >> 7, g = (w >> 5) & 3, l = w & 31;
  const u8 lo = p[64 * c + 32 * (g & 1) + l], h = p[128 + 32 * c + l];
  const int q = ((g < 2) ? (lo & 0xF) : (lo >> 4)) | (((h >> (2 * g)) & 3) << 4);
  const int sc = (int)(signed char)p[192 + 8 * c + (l >> 4) + 2 * g];
  return __fmul_rn(__fmul_rn(gh2f(p + 208), (float)sc), (float)(q - 32));
}
template <>
__device__ __forceinline__ float dequant_weight<ILL_Q2_K>(const u8* __restrict__ row, int col, const uint64_t*,
                                                          const u8*) {
  const u8* p = row + 84 * (col >> 8);
  const int w = col & 255, h = w >> 7, k = (w >> 5) & 3, half = (w >> 4) & 1, l = w & 15;
  const u8 sb = p[8 * h + 2 * k + half];
  const int q = (p[16 + 32 * h + 16 * half + l] >> (2 * k)) & 3;
  return __fsub_rn(__fmul_rn(__fmul_rn(gh2f(p + 80), (float)(sb & 15)), (float)q),
                   __fmul_rn(gh2f(p + 82), (float)(sb >> 4)));
}
template <>
__device__ __forceinline__ float dequant_weight<ILL_IQ2_XXS>(const u8* __restrict__ row, int col,
                                                             const uint64_t* ggrid, const u8* gsigns) {
  const u8* p = row + 66 * (col >> 8);
  const int w = col & 255, ib = w >> 5, l = (w >> 3) & 3, j = w & 7;
  const u8* so = p + 2 + 8 * ib;
  const uint32_t aux = (uint32_t)so[4] | ((uint32_t)so[5] << 8) | ((uint32_t)so[6] << 16) | ((uint32_t)so[7] << 24);
  const float db = __fmul_rn(__fmul_rn(gh2f(p), __fadd_rn(0.5f, (float)(aux >> 28))), 0.25f);
  const float mag = (float)(uint32_t)((ggrid[so[l]] >> (8 * j)) & 0xff);
  const float sg = ((gsigns[(aux >> (7 * l)) & 127] >> j) & 1) ? -1.0f : 1.0f;
  return __fmul_rn(__fmul_rn(db, mag), sg);
}

}  // namespace ill
