/* illatio_b200.h -- C ABI of libillatio_b200.so.
 *
 * A B200 (sm_100a) implementation of illatio's quantized-product hot path: the
 * dequant-fused matrix x vector product over raw GGUF blocks (Q8_0, Q4_K, Q6_K,
 * Q2_K, IQ2_XXS) and the routed mixture-of-experts product.  The reference
 * drives its CUDA kernels from Common Lisp through `launch` (src/cuda.lisp:
 * 323-352); a host binds these functions instead, with SBCL's
 * `load-shared-object` / `alien-funcall` exactly as it binds libcuda
 * (src/cuda.lisp:17-49).
 *
 * Conventions (they mirror the reference's driver binding):
 *   - Device pointers are CUdeviceptr values passed as uint64_t; `ill_stream`
 *     is a CUstream / cudaStream_t.  0 is the default stream.
 *   - Every function returns 0 on success or an ILL_ERR_* code; nothing throws,
 *     aborts or traps.  `ill_error_string` gives the text.
 *   - Calls only enqueue work on the stream and return; none synchronises
 *     (except where stated).  The caller owns every buffer; the library
 *     allocates and frees nothing and keeps no pointer across calls.
 *   - The caller makes the right device current first (cuCtxSetCurrent /
 *     cudaSetDevice), as CUDA-CURRENT does (src/cuda.lisp:90-92).
 *   - Weights are raw GGUF blocks, row-major, exactly as they lie in the file:
 *     no repacking (the reference's repack_q8 / repack_q6k are not needed).
 *     The buffer must be readable up to the next 16-byte boundary past its end
 *     (true of any cuMemAlloc'd buffer).
 *   - Activations are quantized the way the reference's CPU path quantizes
 *     them, so results follow the CPU kernels: Q8_0 blocks (int8 + a float
 *     scale per 32) for Q8_0 weights, Q8_K super-blocks (int8 + a float scale
 *     per 256 + an int16 sum per 16) for Q4_K / Q6_K / Q2_K / IQ2_XXS weights.
 */
#ifndef ILLATIO_B200_H
#define ILLATIO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ILL_API __attribute__((visibility("default")))

typedef uint64_t ill_dptr;
typedef void* ill_stream;

/* weight formats (GGUF block types, src/gguf.lisp:31-40) */
#define ILL_Q8_0 0    /*  32 weights /  34 bytes */
#define ILL_Q4_K 1    /* 256 weights / 144 bytes */
#define ILL_Q6_K 2    /* 256 weights / 210 bytes */
#define ILL_Q2_K 3    /* 256 weights /  84 bytes */
#define ILL_IQ2_XXS 4 /* 256 weights /  66 bytes */

#define ILL_OK 0
#define ILL_ERR_ARG 1         /* a size or flag is out of range, or a required pointer is null */
#define ILL_ERR_ALIGN 2       /* a pointer or stride is not aligned as documented */
#define ILL_ERR_UNSUPPORTED 3 /* a shape this build has no kernel for */
#define ILL_ERR_CUDA 4        /* a CUDA runtime call failed; see ill_last_cuda_error */
#define ILL_ERR_DEVICE_WAIT 5 /* a kernel gave up a bounded wait (ill_device_status) */
#define ILL_ERR_TOO_LARGE 6   /* a size exceeds a documented fixed maximum */

/* ---- library --------------------------------------------------------------- */

/* Library version, major*100 + minor. */
ILL_API int ill_b200_version(void);

/* Text for a status code (static storage).  Plays the part cuGetErrorString
 * plays for the reference's CU macro (src/cuda.lisp:41-49). */
ILL_API const char* ill_error_string(int code);

/* The cudaError_t behind the calling thread's most recent ILL_ERR_CUDA. */
ILL_API int ill_last_cuda_error(void);

/* Bytes per block and weights per block of FMT (0 for an unknown format);
 * src/gguf.lisp:31-40. */
ILL_API int ill_block_bytes(int fmt);
ILL_API int ill_block_weights(int fmt);

/* Reads the current device's status word into *OUT after synchronising STREAM,
 * and clears it.  0 means no kernel gave up a wait.  (The reference has no
 * device-side waits; this is the counterpart of checking each driver call,
 * src/cuda.lisp:41-49.) */
ILL_API int ill_device_status(unsigned int* out, ill_stream stream);

/* Exercises the library's bounded wait: a one-warp kernel waits LIMIT_NS
 * nanoseconds (1000 .. 100000000) for an mbarrier phase that never completes, gives
 * up, records a code in the status word (ill_device_status then returns
 * ILL_ERR_DEVICE_WAIT) and writes 1 to *GAVE_UP (a uint32 on the device; may be 0).
 * The device and the context stay usable.  For tests of the failure path; no
 * counterpart in the reference, which has no device-side waits. */
ILL_API int ill_test_wait_timeout(int64_t limit_ns, ill_dptr gave_up, ill_stream stream);

/* Launches use programmatic dependent launch: a kernel may start streaming its
 * weights while the previous kernel of the stream drains; it still waits for that
 * kernel's results before it reads its activations or writes.  Setting ILL_PDL=0 in
 * the environment before the library is loaded makes every launch a plain one; there
 * is no run-time switch (the library keeps no mutable process-wide state).  (The
 * reference launches with cuLaunchKernel, src/cuda.lisp:345-350.) */

/* ---- activations ----------------------------------------------------------- */

/* X (nblocks*32 floats) -> Q8_0 blocks: d = amax/127, q = round-half-even(x *
 * (1/d)) with the unrounded d; XS[b] = d rounded through fp16 when F16_SCALE,
 * else d itself (ds4's activations).  XSUM (int32 per block, may be 0) gets
 * each block's sum of quants.  Replaces quant_q8 (src/cuda/dense.cu:84) and
 * d4_quant (src/cuda/ds4f.cu:35); bit-for-bit QUANTIZE-Q8! (src/tensor.lisp:
 * 245-262).  XQ must be 16-byte aligned. */
ILL_API int ill_quant_q8_0(ill_dptr x, ill_dptr xq, ill_dptr xs, ill_dptr xsum, int64_t nblocks, int f16_scale,
                           ill_stream stream);

/* X (nblocks*256 floats) -> Q8_K super-blocks: XQ int8, XD one float per 256,
 * BSUMS one int16 per 16 quants.  Bit-for-bit QUANTIZE-Q8K! (src/kquant.lisp:
 * 130-167); the reference's CUDA path has no Q8_K kernel (it feeds K-quants
 * Q8_0 blocks, src/cuda/kquant.cu:3-14), which is why its results differ from
 * its CPU path and these do not. */
ILL_API int ill_quant_q8_k(ill_dptr x, ill_dptr xq, ill_dptr xd, ill_dptr bsums, int64_t nblocks, ill_stream stream);

/* RMSNORM! (src/model.lisp:205-216) of N rows of X (D wide) by W, fused with the
 * activation quantizer: value = (x * scale) * w with scale = 1 / sqrt(float(sum
 * of squares in double / d + eps)), then quantized as ill_quant_q8_0 (KIND 0;
 * XSUM int32 per block or 0; F16_SCALE as there) or ill_quant_q8_k (KIND 1; XSUM
 * int16 per 16, required).  H, when not 0, also receives the normalized floats.
 * Replaces the rmsnorm_q8 launch (RMSNORM-Q8, src/cuda-dense.lisp:260-264;
 * src/cuda/dense.cu:144-160), which quantizes to Q8_0 only. */
ILL_API int ill_rmsnorm_q8(int kind, ill_dptr x, ill_dptr w, ill_dptr h, ill_dptr xq, ill_dptr xs, ill_dptr xsum, int d,
                           float eps, int64_t n, int f16_scale, ill_stream stream);

/* ill_quant_q8_k / ill_rmsnorm_q8 (kind 1) that also leave the blocks' fp16 forms for the tcgen05 products, as
 * ill_act_f16 would make them of the bytes (MAP 0): XH[n*cols] the quants as halves, XE[n*(cols/256)*64] the sums
 * of 16 as halves, 48 of each 64 zero.  One launch where the quantizer and ill_act_f16 are two. */
ILL_API int ill_quant_q8_k_f16(ill_dptr x, ill_dptr xq, ill_dptr xd, ill_dptr bsums, ill_dptr xh, ill_dptr xe, int64_t nblocks,
                               ill_stream stream);
ILL_API int ill_rmsnorm_q8k_f16(ill_dptr x, ill_dptr w, ill_dptr h, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr xh, ill_dptr xe,
                                int d, float eps, int64_t n, ill_stream stream);

/* ---- rows as floats --------------------------------------------------------- */

/* OUT[i*cols ..] = row ROW_IDS[i] (int32, on the device) of the FMT matrix W
 * dequantized, i < NROWS; with ROW_IDS = 0, rows FIRST_ROW .. FIRST_ROW+NROWS-1.
 * Bit-for-bit the reference's CPU dequantization (Q8MAT-ROW! src/tensor.lisp:
 * 354, KMAT-ROW! src/kquant.lisp:466, IQ2XXS-ROW-FLOATS! / Q2K-ROW-FLOATS!
 * src/iquant.lisp:161,217).  Replaces embed_q8 (src/cuda/dense.cu:53) and
 * embed_k (src/cuda/kquant.cu:202). */
ILL_API int ill_dequant_rows(int fmt, ill_dptr w, int cols, ill_dptr row_ids, int64_t first_row, int nrows,
                             ill_dptr out, ill_stream stream);

/* ---- matrix x vector -------------------------------------------------------- */

/* Y[t*rows + r] (+)= W[r] . X[t] (+ BIAS[r]) for N tokens (1 <= N <= 16):
 * token t's quants at XQ + t*cols, its scales at XS + t*(cols/32) (Q8_0) or
 * t*(cols/256) (others), its sums of 16 at XSUM + t*(cols/16) (int16; unused
 * for Q8_0 and IQ2_XXS and may be 0 then).  ACC != 0 adds into Y.  BIAS may
 * be 0.  Replaces mv_q8 (src/cuda/dense.cu:194), mv_k (src/cuda/kquant.cu:169)
 * and d4_mvq8 / d4_mvq8n (src/cuda/ds4f.cu:50,66) behind CMAT-MUL
 * (src/cuda-dense.lisp:220) and DK-Q8MV (src/cuda-ds4f.lisp:773).  XQ must be
 * 16-byte aligned and cols a multiple of 256 (32 for Q8_0).
 *
 * N > 16 is a prefill chunk: Q8_0, Q4_K and Q6_K take it in one launch on the
 * tensor cores' int8 path (any N), replacing mm_q8_mma2 (src/cuda/dense.cu:885)
 * and mm_q4k_mma / mm_q6k_mma (src/cuda/kquant.cu:316-466) behind CMAT-MUL-N;
 * that path wants XS (Q8_0: and cols a multiple of 128) or XSUM (others) 16-byte
 * aligned.  Otherwise ILL_ERR_UNSUPPORTED comes back for N > 16 -- also for N <= 16
 * when N tokens of COLS columns do not fit a CTA's shared memory -- and the caller
 * splits the tokens. */
ILL_API int ill_mv(int fmt, ill_dptr w, int rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr y,
                   ill_dptr bias, int acc, int n, ill_stream stream);

/* Three products sharing one token's activations in one launch: Yk = Wk . X
 * (+ Bk).  With W2 = 0 and ROWS2 = 0, two products.  Replaces mv_q8_3
 * (src/cuda/dense.cu:210) behind QKV-MUL (src/cuda-dense.lisp:309); also takes
 * the K-quant formats. */
ILL_API int ill_mv_3(int fmt, ill_dptr w0, ill_dptr w1, ill_dptr w2, int rows0, int rows1, int rows2, int cols,
                     ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr y0, ill_dptr y1, ill_dptr y2, ill_dptr b0,
                     ill_dptr b1, ill_dptr b2, ill_stream stream);

/* Y[r] = silu(G[r] . X) * (U[r] . X), silu(g) = g / (1 + exp(-g)), one token.
 * Replaces mv_q8_glu (src/cuda/dense.cu:230) and mv_k_glu (src/cuda/kquant.cu:
 * 183) behind GLU-MUL (src/cuda-dense.lisp:326). */
ILL_API int ill_mv_glu(int fmt, ill_dptr wg, ill_dptr wu, int rows, int cols, ill_dptr xq, ill_dptr xs,
                       ill_dptr xsum, ill_dptr y, ill_stream stream);

/* ---- a decoded token's chain of products in one launch ---------------------------- */

/* One product of the chain.  KIND ILL_OP_MV: Y (+)= W X' (+ BIAS), ACC != 0 adds
 * into Y; ILL_OP_GLU: Y = silu(W X') * (W2 X') (no ACC, no BIAS).  X' is the
 * product's activations, made from the COLS floats at X inside the launch:
 * RMSNORM! of them by NORM_W with EPS when NORM_W is given (as ill_rmsnorm_q8),
 * then quantized the way FMT's products take them (Q8_0 blocks for ILL_Q8_0, with
 * the scale rounded through fp16 when F16_SCALE; Q8_K super-blocks otherwise) --
 * bit for bit what ill_quant_q8_0 / ill_quant_q8_k / ill_rmsnorm_q8 write.  AFTER
 * != 0: the product reads (X) or adds into (Y) what an earlier product of the list
 * writes, so every earlier product is complete before it starts; products without
 * it may run beside their predecessors.  W, W2, X and NORM_W are 16-byte aligned. */
#define ILL_OP_MV 0
#define ILL_OP_GLU 1
typedef struct ill_decode_op {
  ill_dptr w, w2, x, norm_w, y, bias;
  int32_t fmt, kind, rows, cols;
  int32_t acc, after, f16_scale;
  float eps;
} ill_decode_op;

/* A token's products in one launch, in place of a launch per product and a launch
 * per quantization (CUDA-FORWARD-N, src/cuda-dense.lisp:380-432; the reference's
 * own note on what its ~1,700 launches a token cost: TODO.md:16-21).
 * ill_decode_plan turns the NOPS products at OPS (host memory) into the list the
 * kernel walks, written to PLAN (device memory the caller owns, 128-byte aligned,
 * ill_decode_plan_bytes(nops) bytes; it also holds the barrier the CTAs meet at),
 * and fills LAUNCH (ILL_DECODE_LAUNCH_WORDS ints the caller keeps beside PLAN; the
 * library keeps nothing itself).  It synchronises STREAM.  ill_decode_run enqueues
 * the token: one cooperative launch of one CTA per SM; it updates LAUNCH (the
 * barrier's arrivals are counted on from token to token).  The same PLAN runs any
 * number of tokens, one at a time, in the order ill_decode_run was called (two runs
 * of one PLAN must not overlap).  Results are the same bits ill_mv / ill_mv_glu give on the
 * same activations.  Rows too long for a lane's registers (more than 160 units of
 * 64 weights, 224 Q8_0 blocks) are ILL_ERR_UNSUPPORTED: use ill_mv for those.
 * After a time-out (ILL_ERR_DEVICE_WAIT from ill_device_status) plan again before
 * the next run: the barrier's count may be left mid-way. */
#define ILL_DECODE_LAUNCH_WORDS 16
ILL_API int64_t ill_decode_plan_bytes(int nops);
ILL_API int ill_decode_plan(const ill_decode_op* ops, int nops, ill_dptr plan, int64_t plan_bytes, int32_t* launch,
                            ill_stream stream);
ILL_API int ill_decode_run(ill_dptr plan, int32_t* launch, ill_stream stream);

/* ---- routed experts: one decoded token ------------------------------------------ */

/* Y[z*y_stride + r] = W_z[r] . X_z for each expert z < NZ: W_z's NROWS rows of
 * NCOLS weights start at PTRS[z] + ADD (PTRS: a device table of 64-bit device
 * addresses, the experts' slots; 16-byte aligned addresses and ADD); X_z is
 * token z of XQ/XS/XSUM when X_PER_EXPERT is 1, token 0 for every expert when
 * it is 0.  Replaces d4_mv_iq2_xxs / d4_mv_q2_k (src/cuda/ds4f.cu:769,837)
 * behind DK-FFN-TAIL (src/cuda-ds4f.lisp:908-956); activations are Q8_K, as
 * the CPU path's are (src/ds4f.lisp:1001,1021). */
ILL_API int ill_moe_mv(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, int nz, ill_dptr xq, ill_dptr xs,
                       ill_dptr xsum, int x_per_expert, ill_dptr y, int64_t y_stride, ill_stream stream);

/* MID[z*mid_stride + r] = silu(min(g, c)) * clamp(u, +-c) * WEIGHTS[z] with g =
 * G_z[r] . X, u = U_z[r] . X, G_z at PTRS[z] + GATE_ADD, U_z at PTRS[z] + UP_ADD
 * (CLAMP <= 1e-6: no clamping); FMT is ILL_IQ2_XXS or ILL_Q2_K.  One launch for
 * what the reference does with two d4_mv_iq2_xxs grids and d4_swiglu_w
 * (src/cuda-ds4f.lisp:937-939); the arithmetic is D4-ROUTED!'s
 * (src/ds4f.lisp:1012-1019). */
ILL_API int ill_moe_glu(int fmt, int ncols, int nrows, int64_t gate_add, int64_t up_add, ill_dptr ptrs, int nz,
                        ill_dptr xq, ill_dptr xs, ill_dptr xsum, int x_per_expert, float clamp, ill_dptr weights,
                        ill_dptr mid, int64_t mid_stride, ill_stream stream);

/* MID[i] = silu(min(G[i], c)) * clamp(U[i], +-c) * W[i / ff] for i < N (W = 0: no
 * weights).  Replaces d4_swiglu_w (src/cuda/ds4f.cu:645); quantize the result
 * with ill_quant_q8_0 / ill_quant_q8_k. */
ILL_API int ill_swiglu_w(int64_t n, int ff, float clamp, ill_dptr g, ill_dptr u, ill_dptr w, ill_dptr mid,
                         ill_stream stream);

/* ill_swiglu_w, ill_quant_q8_k and ill_act_f16 of the middle values in one
 * pass, for the chunk path: MH[r*ff + j] = fp16 of the Q8_K quant of row r's
 * j-th middle value, MS[r*(ff/256) + kb] its block scales, and with ME given
 * (Q2_K down weights) ME[(r*(ff/256) + kb)*64 + i] the sums of 16 as ill_act_f16
 * lays them out.  Bit for bit what the three calls produce; the middle values
 * and their int8 form are not written.  (The reference keeps d4_swiglu_w and
 * the quantizer apart, src/cuda-ds4f-prefill.lisp:348-349; fusing them is its own
 * open item, TODO.md:16-21.)  ROWS_DEV as for ill_ep_unpack (0: all ROWS). */
ILL_API int ill_swiglu_q8k_f16(int64_t rows, int ff, float clamp, ill_dptr g, ill_dptr u, ill_dptr w, ill_dptr mh,
                               ill_dptr me, ill_dptr ms, ill_dptr rows_dev, ill_stream stream);

/* MOE[t*d + r] = sum over slots s < NU, in slot order, of DOWN[row(t,s)*d + r]
 * (+ SHARED[t*d + r] unless 0); row(t,s) = MAP[t*nu + s], or t*nu + s when MAP
 * is 0.  Replaces d4_moe_sum (src/cuda/ds4f.cu:902) and d4_moe_sum_rows
 * (src/cuda/ds4f_chunk.cu:402). */
ILL_API int ill_moe_sum(int d, int nu, int64_t ntok, ill_dptr down, ill_dptr map, ill_dptr shared_, ill_dptr moe,
                        ill_stream stream);

/* ---- routed experts: a chunk of tokens -------------------------------------------- */

/* Per token: SEL[t*nu ..] the NU experts with the largest p + BIAS (BIAS may be
 * 0), the earlier expert first among equals, and WEIGHTS[t*nu ..] = p / max(sum
 * of the chosen p, 6.103515625e-5) * SCALE; p = sqrt(softplus(logit)) for MODE 0
 * (D4-ROUTE, src/ds4f.lisp:950-978), sigmoid(logit) for MODE 2 (G53-ROUTE,
 * src/glm53.lisp:360-379).  NE <= 512, NU <= 32.  Replaces d4_route
 * (src/cuda/ds4f_chunk.cu:420). */
ILL_API int ill_moe_route(int ne, int nu, int mode, float scale, int64_t ntok, ill_dptr logits, ill_dptr bias,
                          ill_dptr sel, ill_dptr weights, ill_stream stream);

/* Element types of the unquantized tensors ill_mv_dense takes. */
#define ILL_F32 0
#define ILL_F16 1
#define ILL_BF16 2

/* Y[t*y_stride + r] = W[r] . X[t] for the ROWS x COLS matrix W of F32 / F16 /
 * BF16 values (row-major, as in the file) and N tokens' float activations
 * X [n, cols] (one token, a few, or a prefill chunk: DK-F16MM,
 * src/cuda-ds4f-prefill.lisp:297); fp32 accumulate.  The router's logits and the other
 * small unquantized tensors between the quantized products: DK-MV16
 * (src/cuda-ds4f.lisp:767-771; d4_mv_f16 src/cuda/ds4f.cu:145, g53_mv_bf16,
 * d41_mv_f32 and their several-token forms).  The CPU path is F32MV!
 * (src/ds4f.lisp:256-276) on weights widened to float. */
ILL_API int ill_mv_dense(int type, ill_dptr w, int rows, int cols, ill_dptr x, ill_dptr y, int n, int64_t y_stride,
                         ill_stream stream);

/* Bytes of scratch ill_moe_group needs for ROWS (token, slot) rows and NE experts. */
ILL_API int64_t ill_moe_group_scratch_bytes(int64_t rows, int ne);

/* Groups the ROWS = tokens*NU (token, slot) rows by expert, an expert's rows in
 * token order (a stable counting sort: the result does not depend on
 * scheduling): COUNTS[e], BASES[e] (uint32 per expert); RMAP[place] = the row's
 * token; SMAP[t*nu + s] = the row's place; WROW[place] = W[t*nu + s] (WROW may
 * be 0).  SCRATCH: ill_moe_group_scratch_bytes.  Replaces d4_group_zero / count
 * / scan / scatter (src/cuda/ds4f_chunk.cu:476-508), whose order inside an
 * expert follows an atomic counter. */
ILL_API int ill_moe_group(int64_t rows, int ne, int nu, ill_dptr sel, ill_dptr w, ill_dptr scratch, ill_dptr counts,
                          ill_dptr bases, ill_dptr rmap, ill_dptr smap, ill_dptr wrow, ill_stream stream);

/* ROW_PTRS[place] = PTRS[e] for every place of expert e < NE as ill_moe_group counted them (COUNTS, BASES; TOTAL_ROWS
 * places in all): the table ill_moe_glu / ill_moe_mv take with NZ = TOTAL_ROWS and X_PER_EXPERT = 1, so that the
 * one-token kernels multiply a few tokens' rows expert by expert, an expert's rows next to each other (its weights
 * come from HBM once, the other rows find them in L2).  The several-token form of the routed experts on the matvec
 * path: DK-FFN-SMALL (src/cuda-ds4f-spec.lisp:31-132), whose d4_mv_iq2_xxs / d4_mv_q2_k take the same COUNTS and
 * BASES (src/cuda/ds4f.cu:769-772, 837).  Places past the last expert's get expert 0's matrix. */
ILL_API int ill_moe_row_ptrs(int ne, ill_dptr ptrs, ill_dptr counts, ill_dptr bases, int64_t total_rows, ill_dptr row_ptrs,
                             ill_stream stream);

/* ill_moe_group for callers that cannot allocate device memory and have none
 * to spare for scratch: a host whose whole device budget is committed at
 * start-up (illatio sizes its expert pool to all the memory that is left and
 * records every allocation so it can give the device up and come back), or one
 * that runs where an allocation would stall the device.  Same arguments and
 * results as ill_moe_group, without SCRATCH: the scratch is a fixed array inside
 * the library's device image (384 KB on every GPU that loads the library, held
 * until the process exits).  No counterpart in the reference.
 *   - Limits: ROWS <= ILL_GROUP_STATIC_MAX_ROWS and NE <=
 *     ILL_GROUP_STATIC_MAX_EXPERTS, else ILL_ERR_TOO_LARGE.
 *   - The first call on a device looks the array's address up (a host-side
 *     query, no allocation); make that first call outside any stream capture.
 *   - The function calls no cudaMalloc / cudaFree and no allocating routine.
 *   - All calls on a device share the one array.  A call reads nothing an
 *     earlier call left there, but two calls whose kernels overlap on the GPU
 *     (different streams) race: keep them in one stream or order them. */
#define ILL_GROUP_STATIC_MAX_ROWS 65536
#define ILL_GROUP_STATIC_MAX_EXPERTS 512
ILL_API int ill_moe_group_static(int64_t rows, int ne, int nu, ill_dptr sel, ill_dptr w, ill_dptr counts, ill_dptr bases,
                                 ill_dptr rmap, ill_dptr smap, ill_dptr wrow, ill_stream stream);

/* DST row r = SRC row MAP[r], rows of ROW_BYTES bytes: a multiple of 16 with
 * both 16-byte aligned, or a multiple of 4 with both 4-byte aligned.  Replaces
 * d4_gather_rows (src/cuda/ds4f_chunk.cu:393). */
ILL_API int ill_gather_rows(int64_t rows, int64_t row_bytes, ill_dptr src, ill_dptr map, ill_dptr dst,
                            ill_stream stream);

/* The Q8_K activations as the tensor cores take them, gathered into expert
 * order: XH[place*cols + k] = fp16(XQ[t*cols + k]) (the int8 quant, exact), t =
 * MAP[place] (MAP = 0: t = place).  With XE given (Q2_K weights need it), also
 * the sums of 16: XE[(place*(cols/256) + kb)*64 + g] = fp16(BSUMS[t*(cols/16) +
 * 16*kb + g]) for g < 16 (exact), the other 48 of each 64 zero.  XQ, XH, XE
 * 16-byte aligned.  (The reference's d4_mm_id rounds the unquantized floats to
 * fp16 instead, src/cuda/ds4f_mm.cu:1-20, and so drifts from its CPU path.) */
ILL_API int ill_act_f16(int64_t rows, int cols, ill_dptr xq, ill_dptr bsums, ill_dptr map, ill_dptr xh, ill_dptr xe,
                        ill_stream stream);

/* Expert parallelism: a (token, slot) row travels to the rank that holds its
 * expert as one piece, the token's Q8_K form and the slot's weight:
 *   [cols int8 quants][cols/256 float scales][cols/16 int16 sums][float weight]
 * padded to a multiple of 16 bytes = ill_ep_row_bytes(cols).  ill_ep_pack fills
 * PACKED[place] from token MAP[place] of XQ / XS / XSUM (ill_quant_q8_k) and
 * W[place] (the WROW of ill_moe_group).  ill_ep_unpack is ill_act_f16 on rows that
 * arrived packed: XH / XE as there, plus XD[place, kb] (the scales
 * ill_moe_mm_id wants, so that it needs no MAP) and W[place]; MAP[place] is the
 * arrival index of the row placed at `place` (the P2R of ill_ep_plan_rows; 0:
 * the same).  ROWS_DEV, when not 0, points at the number of rows in use (a
 * uint32 on the device, e.g. the TOTAL of ill_ep_plan_dev): places from there
 * up to ROWS are skipped.  No counterpart in the reference. */
ILL_API int64_t ill_ep_row_bytes(int cols);
ILL_API int ill_ep_pack(int64_t rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr w, ill_dptr map,
                        ill_dptr packed, ill_stream stream);
ILL_API int ill_ep_unpack(int64_t rows, int cols, ill_dptr packed, ill_dptr map, ill_dptr xh, ill_dptr xe, ill_dptr xd,
                          ill_dptr w, ill_dptr rows_dev, ill_stream stream);

/* The same exchange with slabs of a fixed size, so that the host never waits for
 * counts: every rank sends every rank CAP rows' worth (ill_ep_pack_cap: rank g's
 * rows, in place order, in slab g; PSLOT[place] = g*cap + index; *OVERFLOW is
 * set, and the rows past CAP dropped, if a slab is too small -- the caller then
 * repeats the chunk with exact sizes), and the per-expert counts travel as a
 * [world, per] table.  ill_ep_plan_dev turns the received table RC[s*per + e]
 * into the local experts' COUNTS / BASES, the two row orders (P2R over all
 * world*cap places, those past the last row pointing at slot 0), TOTAL[0], and
 * with PDST given where each place's result goes (for ill_moe_mm_id_peers), on
 * the device.  Only the rows a sender kept are planned (a source's first CAP in
 * its expert order), so the plan never names more than world*cap rows whatever RC
 * holds; when some were cut, *OVERFLOW (may be 0) is or-ed with 1.  No counterpart
 * in the reference. */
ILL_API int ill_ep_pack_cap(int64_t rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr w, ill_dptr map,
                            ill_dptr bases, int per, int world, int cap, ill_dptr packed, ill_dptr pslot, ill_dptr overflow,
                            ill_dptr peers, int rank, ill_stream stream);
/* With PEERS given (the address of every rank's receive buffer: peer memory)
 * ill_ep_pack_cap stores each row straight into slab RANK of its destination's
 * buffer and PACKED is not used; ill_ep_put_counts does the same for the table
 * of counts (row RANK of every rank's [world, per] table).  The dispatch then
 * needs no collective, only a barrier between the ranks' streams before the
 * receivers read.  OVERFLOW, when not 0, is cleared (the flag of the
 * ill_ep_pack_cap that follows in the stream). */
ILL_API int ill_ep_put_counts(int world, int per, int rank, ill_dptr counts, ill_dptr peers, ill_dptr overflow,
                              ill_stream stream);
ILL_API int ill_ep_plan_dev(int world, int per, int cap, int rank, ill_dptr rc, ill_dptr counts, ill_dptr bases, ill_dptr p2r,
                            ill_dptr r2p, ill_dptr pdst, ill_dptr total, ill_dptr overflow, ill_stream stream);

/* ---- expert parallelism without a collective library: peer mappings and meetings ------------
 * A host that runs one process per GPU (as illatio runs one Lisp thread per device,
 * src/cuda-ds4f.lisp:594-618) needs two things of its peers: their buffers' addresses,
 * and a way for the ranks' streams to meet.  Both are here, so that the chunk needs no
 * NCCL, no torch and no host synchronisation.  No counterpart in the reference, whose
 * second device exchanges activations through pinned host memory.
 *
 * ill_ep_ipc_export gives the 64-byte CUDA IPC handle of the allocation that holds BUF (a
 * cuMemAlloc'd buffer of the caller's) and BUF's offset inside it; the host passes both to
 * its peers by any means it has.  ill_ep_ipc_open maps a peer's buffer into this process
 * (peer access is enabled on first use) and returns its address here; ill_ep_ipc_close
 * unmaps it.  A rank does not open its own handle: it uses its own address.
 *
 * A meeting is made of flags: every rank owns ill_ep_flags_bytes() bytes of zeroed device
 * memory that its peers have mapped, FLAG_PEERS is a device table of the WORLD addresses
 * (this rank's own at [RANK]), FLAGS this rank's own array.  Meeting number EPOCH (1, 2, ...
 * counted by the caller, the same on every rank) in SLOT (0..3): the rank stores EPOCH into
 * every peer's flags, after a system-wide fence, and waits until every peer's EPOCH has
 * arrived in its own.  The wait is bounded: WAIT_NS nanoseconds (0: two seconds), after
 * which the kernel records a code in the status word (ill_device_status) and goes on
 * without the meeting -- ill_ep_plan_dev_sync then plans no rows, ill_moe_sum_sync sums
 * nothing; nothing hangs and nothing traps.  ill_ep_barrier is the meeting alone (one
 * block); ill_ep_plan_dev_sync is ill_ep_plan_dev after a meeting in slot 0 (this rank's
 * rows and counts are in its peers' buffers; theirs are in its own once they have all said
 * so); ill_moe_sum_sync is ill_moe_sum after a meeting in slot 1, with row(t, s) =
 * MAP2[MAP[t*nu + s]] when MAP2 is given (OVF_EPOCH / OVF_FLAG: see ill_ep_dispatch; both
 * may be 0).  Two meetings a chunk order everything: a peer
 * cannot overwrite a buffer this rank still reads, because it passes the chunk's second
 * meeting only after this rank has enqueued everything before its own. */
#define ILL_EP_IPC_HANDLE_BYTES 64
ILL_API int ill_ep_ipc_export(ill_dptr buf, unsigned char* handle, int64_t* offset);
ILL_API int ill_ep_ipc_open(const unsigned char* handle, int64_t offset, ill_dptr* out);
ILL_API int ill_ep_ipc_close(ill_dptr mapped, int64_t offset);
ILL_API int64_t ill_ep_flags_bytes(void);
ILL_API int ill_ep_barrier(ill_dptr flag_peers, ill_dptr flags, int world, int rank, int slot, uint32_t epoch, int64_t wait_ns,
                           ill_stream stream);
/* An all-gather by peer stores (the row-split head's logits; no counterpart in the reference, which
 * keeps the head on one device): NBYTES of SRC go to DST_PEERS[p] + DST_OFF of every rank p
 * (DST_PEERS: a device table of WORLD mapped addresses, this rank's own included; an address
 * equal to SRC is skipped, so SRC may be this rank's block inside its own buffer), then the
 * ranks meet in SLOT (see above): when the call's kernel has ended without a status code, every
 * peer's block is complete in this rank's buffer.  SRC, NBYTES, DST_OFF multiples of 4 (16 for
 * the fast path).  One call at a time a device.  The caller alternates two buffers (or holds
 * another meeting) before a block is overwritten that a peer may still be reading. */
ILL_API int ill_peer_put(ill_dptr src, int64_t nbytes, ill_dptr dst_peers, int64_t dst_off, ill_dptr flag_peers, ill_dptr flags,
                         int world, int rank, int slot, uint32_t epoch, int64_t wait_ns, ill_stream stream);
/* ill_mv for one token with the all-gather in its epilogue (the row-split head at batch 1): row r's result goes to
 * Y_PEERS[p] + 4 * (Y_OFF + r) of every rank p (a device table of WORLD mapped float buffers, this rank's own
 * included) instead of to a Y, and the CTA that finishes last holds the ranks' meeting in SLOT -- one launch where
 * ill_mv + ill_peer_put are two.  The same caveats as ill_peer_put (one such call at a time a device; alternate
 * two buffers).  ILL_ERR_UNSUPPORTED for shapes the one-token kernel does not take whole (then: ill_mv and
 * ill_peer_put). */
ILL_API int ill_mv_peers(int fmt, ill_dptr w, int rows, int cols, ill_dptr xq, ill_dptr xs, ill_dptr xsum, ill_dptr y_peers,
                         int64_t y_off, ill_dptr bias, ill_dptr flag_peers, ill_dptr flags, int world, int rank, int slot,
                         uint32_t epoch, int64_t wait_ns, ill_stream stream);
ILL_API int ill_ep_plan_dev_sync(int world, int per, int cap, int rank, ill_dptr rc, ill_dptr counts, ill_dptr bases, ill_dptr p2r,
                                 ill_dptr r2p, ill_dptr pdst, ill_dptr total, ill_dptr overflow, ill_dptr flag_peers, ill_dptr flags,
                                 uint32_t epoch, int64_t wait_ns, ill_stream stream);
ILL_API int ill_moe_sum_sync(int d, int nu, int64_t ntok, ill_dptr down, ill_dptr map, ill_dptr map2, ill_dptr shared_, ill_dptr moe,
                             ill_dptr flag_peers, ill_dptr flags, int world, int rank, uint32_t epoch, int64_t wait_ns,
                             ill_dptr ovf_epoch, ill_dptr ovf_flag, ill_stream stream);

/* The dispatch of an expert-parallel chunk in one launch: ill_quant_q8_k, ill_ep_put_counts
 * and ill_ep_pack_cap (peer form) together.  X holds the NTOK tokens' activations as floats
 * [tokens, cols] (16-byte aligned).  Token t is quantized once -- the same bits as
 * ill_quant_q8_k -- and its packed row stored, for each of its NU slots s, in slab RANK of
 * the rank that holds the slot's expert (PEERS_ROWS), with the slot's weight: the row's
 * place among the (token, slot) rows is SMAP[t*nu + s] and its weight W[place], as
 * ill_moe_group leaves them (its SMAP, WROW, and its per-expert BASES / COUNTS); this rank's
 * rows per expert go into row RANK of every rank's table (PEERS_RC).  A slab too small raises
 * *OVERFLOW to EPOCH (>= 1, the chunk's number; the word is never cleared --
 * ill_ep_plan_dev_sync raises it the same way, and ill_moe_sum_sync turns "equals this
 * chunk's number" into 0 / 1 at *OVF_FLAG when given OVF_EPOCH = this word).  Needs
 * NTOK >= ceil(world*per / 128), else ILL_ERR_UNSUPPORTED (use the three calls); NU <= 32.
 * No counterpart in the reference. */
ILL_API int ill_ep_dispatch(int64_t ntok, int nu, int cols, ill_dptr x, ill_dptr w, ill_dptr smap, ill_dptr bases, ill_dptr counts,
                            int per, int world, int cap, int rank, ill_dptr peers_rows, ill_dptr peers_rc, ill_dptr pslot,
                            ill_dptr overflow, uint32_t epoch, ill_stream stream);

/* Two matrices of every expert against the same rows in one launch (gate and up:
 * W_e at PTRS[e] + ADD into Y, at PTRS[e] + ADD2 into Y2; no YMAP).  The same
 * results as two calls of ill_moe_mm_id; one launch fills the SMs better when a
 * rank holds few experts. */
ILL_API int ill_moe_mm_id2(int fmt, int ncols, int nrows, int64_t add, int64_t add2, ill_dptr ptrs, ill_dptr counts,
                           ill_dptr bases, int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map,
                           ill_dptr y, ill_dptr y2, int64_t y_stride, ill_stream stream);

/* ill_moe_mm_id with the combine of an expert-parallel chunk fused into it: the
 * row computed for `place` is stored straight into the memory of the rank that
 * owns its token, YPEERS[r] being the address of rank r's Y (peer memory: a
 * symmetric allocation, every rank's the same shape) and YDST[place] = r << 24 |
 * row of that Y (the PDST of ill_ep_plan_dev, RANK the caller's).  Plain stores
 * over NVLink, tile by tile as the products finish, instead of an all-to-all
 * after them; the owner may read its Y once every rank's call has completed (a
 * barrier between the ranks' streams).  No TMA and no multicast touch peer
 * memory.  No counterpart in the reference. */
ILL_API int ill_moe_mm_id_peers(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases,
                                int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr ydst,
                                ill_dptr ypeers, int64_t y_stride, ill_stream stream);

/* CMAT-MUL-N for a prefill chunk on the 5th-generation tensor cores: Y[t*rows + r] (+)= W[r] . X[t] for N tokens
 * and a ROWS x COLS matrix of Q4_K or Q6_K blocks -- the kernel of ill_moe_mm_id with the matrix as its one expert
 * and no tables on the device.  XH / XE / XD as ill_act_f16 leaves them for the chunk's Q8_K activations (MAP 0):
 * quants and sums of 16 as fp16 integers (XE: Q4_K only, else 0), and the block scales.  The weights go in as
 * integers exact in fp16 (Q4_K: scale * q <= 945; Q6_K: scale * (q - 32) as an even and an odd part) and a block's
 * sum is taken in fp32 in tensor memory, exact up to 2^24: it could only round if nearly every weight and
 * activation of a block sat at its maximum.  W 16-byte aligned (Q4_K), ROWS a multiple of 4.
 * ILL_ERR_UNSUPPORTED for the other formats: ill_mv takes chunks of Q8_0 (and of these two) on the int8 mma.sync
 * path.  Replaces mm_q4k_mma / mm_q6k_mma (src/cuda/kquant.cu:316-466) behind CMAT-MUL-N (src/cuda-dense.lisp:250-255). */
ILL_API int ill_mm_chunk(int fmt, ill_dptr w, int rows, int cols, ill_dptr xh, ill_dptr xe, ill_dptr xd, int64_t n, ill_dptr y,
                         int acc, ill_stream stream);
/* The same for two matrices of one shape against the same chunk (a gated FFN's gate and up) in one launch:
 * Y = W X, Y2 = W2 X.  Twice the tiles for the kernel's persistent CTAs to share. */
ILL_API int ill_mm_chunk2(int fmt, ill_dptr w, ill_dptr w2, int rows, int cols, ill_dptr xh, ill_dptr xe, ill_dptr xd, int64_t n,
                          ill_dptr y, ill_dptr y2, ill_stream stream);

/* The routed experts' product for a chunk: for each expert e < NE and each row
 * `place` in [BASES[e], BASES[e] + COUNTS[e]): Y[place*y_stride + n] = W_e[n] .
 * X[place], n < NROWS, W_e the FMT (ILL_IQ2_XXS, ILL_Q2_K; also ILL_Q4_K, ILL_Q6_K) matrix at PTRS[e]
 * + ADD, X the Q8_K activations XH (+ XE for Q2_K / Q4_K) of ill_act_f16 with block
 * scales XD[t*(ncols/256) + kb], t = MAP[place] (MAP = 0: t = place).  COUNTS /
 * BASES are read on the device (no host synchronisation); TOTAL_ROWS is the
 * number of rows of XH and Y.  With YMAP given, row `place` is written to row
 * YMAP[place] of Y instead (expert parallelism: the rows leave in the order they
 * arrived).
 *
 * tcgen05 MMA, tiles of 128 weight rows x up to 128 rows of X: the operands are
 * the integers of both sides as fp16 (exact; the weights' go straight from the
 * dequantizing warps into tensor memory), accumulated per 256-wide block in
 * tensor memory (fp32, two buffers), and each block's sum is scaled by d_w * d_x
 * in fp32 as it is drained -- the arithmetic of the reference's CPU kernels (src/avx2.lisp:
 * 77-150), so results agree with them to fp32 rounding.  Replaces
 * d4_mm_id_iq2_xxs / d4_mm_id_q2_k (src/cuda/ds4f_mm.cu:229-257) behind
 * DK-FFN-ROUTED-CHUNK (src/cuda-ds4f-prefill.lisp:345-351). */
ILL_API int ill_moe_mm_id(int fmt, int ncols, int nrows, int64_t add, ill_dptr ptrs, ill_dptr counts, ill_dptr bases,
                          int ne, int64_t total_rows, ill_dptr xh, ill_dptr xe, ill_dptr xd, ill_dptr map, ill_dptr ymap,
                          ill_dptr y, int64_t y_stride, ill_stream stream);

/* Expert parallelism: the two row orders of a rank that receives rows from
 * several sources.  Rows arrive source by source, each source's rows grouped by
 * expert; the products want them expert by expert.  Segment i (one source, one
 * expert) is SEG_LEN[i] rows that arrive at SEG_ARRIVAL[i] .. and are placed at
 * SEG_PLACE[i] ..: fills P2R[place] = arrival index and R2P[arrival] = place
 * (uint32).  The three tables (int32, NSEG each) come from the host, which knows
 * every rank's counts after one small exchange.  No counterpart in the
 * reference, whose experts never leave their GPU. */
ILL_API int ill_ep_plan_rows(int nseg, ill_dptr seg_arrival, ill_dptr seg_place, ill_dptr seg_len, ill_dptr p2r,
                             ill_dptr r2p, ill_stream stream);

#ifdef __cplusplus
}
#endif
#endif
