"""Host side of the dense decode path: the reference's src/cuda-dense.lisp,
mirrored name for name over the C ABI.

The reference drives its kernels from Lisp (`launch`, src/cuda.lisp:323); no
Lisp implementation is available to run, so this module plays the part of the
Lisp caller: the same operators (UPLOAD-GMAT, QUANT-Q8, CMAT-MUL, QKV-MUL,
GLU-MUL, EMBED), the same argument meaning, over libillatio_b200.so.  torch is
used only to own device memory and streams.

Differences from the reference's device layout, all invisible to callers of
these operators: matrices stay as raw GGUF blocks (no repack_q8 / repack_q6k),
and K-quant products take Q8_K activations as the CPU path does (`xs` is then
one float per 256 and `xsum` one int16 per 16 quants).
"""
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from .blocks import BLOCK_BYTES, BLOCK_WEIGHTS, NAMES, Q8_0, row_bytes


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


@dataclass
class CMat:
    """A matrix on the device (CMAT, src/cuda-dense.lisp:13-16): raw blocks."""
    name: str
    type: int
    rows: int
    cols: int
    qs: torch.Tensor  # uint8, rows * row_bytes

    @property
    def row_bytes(self):
        return row_bytes(self.type, self.cols)

    @property
    def nbytes(self):
        return self.rows * self.row_bytes


def cmat_kquant_p(w):
    return w.type != Q8_0


def upload_gmat(blocks, fmt, rows, cols, name="", device="cuda"):
    """UPLOAD-GMAT (src/cuda-dense.lisp:75-100): a tensor's raw blocks (uint8
    numpy array or tensor) to the device, as they are."""
    if cols % BLOCK_WEIGHTS[fmt]:
        raise ValueError("%s: %d columns is not a whole number of blocks" % (name, cols))
    t = torch.as_tensor(blocks).reshape(-1)
    if t.dtype != torch.uint8 or t.numel() != rows * row_bytes(fmt, cols):
        raise ValueError("%s: expected %d bytes of %s blocks" % (name, rows * row_bytes(fmt, cols), NAMES[fmt]))
    return CMat(name, fmt, rows, cols, t.to(device, non_blocking=True).contiguous())


@dataclass
class QAct:
    """Quantized activations of N tokens (the cctx's xq / xs / xsum)."""
    kind: str            # "q8" (Q8_0 blocks) or "q8k" (Q8_K super-blocks)
    xq: torch.Tensor     # int8 [n * cols]
    xs: torch.Tensor     # float32 per 32 (q8) or per 256 (q8k)
    xsum: torch.Tensor   # q8: int32 per 32 (or None); q8k: int16 per 16


def make_qact(n, kind, device="cuda", want_xsum=False):
    """Room for N activations in KIND (MAKE-QACT, src/kquant.lisp:506-510)."""
    if kind == "q8":
        return QAct(kind, torch.empty(n, dtype=torch.int8, device=device),
                    torch.empty(n // 32, dtype=torch.float32, device=device),
                    torch.empty(n // 32, dtype=torch.int32, device=device) if want_xsum else None)
    return QAct(kind, torch.empty(n, dtype=torch.int8, device=device),
                torch.empty(n // 256, dtype=torch.float32, device=device),
                torch.empty(n // 16, dtype=torch.int16, device=device))


def matrix_act_kind(w):
    """MATRIX-ACT-KIND (src/kquant.lisp:532-533)."""
    return "q8k" if cmat_kquant_p(w) else "q8"


def quant_q8(x, act, f16_scale=True):
    """X (float32, a whole number of blocks) quantized into ACT: the reference's
    quant_q8 launch (src/cuda-dense.lisp:366,417), in the kind ACT holds."""
    n = x.numel()
    if act.kind == "q8":
        _lib.call("ill_quant_q8_0", _ptr(x), _ptr(act.xq), _ptr(act.xs), _ptr(act.xsum), n // 32,
                  1 if f16_scale else 0, _stream())
    else:
        cf = getattr(act, "_cf", None)
        if cf is not None and cf.n * cf.cols == n:
            # ACT's fp16 form is in use by the tcgen05 products: renewed in the same launch
            _lib.call("ill_quant_q8_k_f16", _ptr(x), _ptr(act.xq), _ptr(act.xs), _ptr(act.xsum), _ptr(cf.xh), _ptr(cf.xe), n // 256,
                      _stream())
            cf.xd = act.xs
            act._cf_fresh = True
            return act
        _lib.call("ill_quant_q8_k", _ptr(x), _ptr(act.xq), _ptr(act.xs), _ptr(act.xsum), n // 256, _stream())
    act._cf_fresh = False
    return act


def rmsnorm_q8(x, w, act, d, eps, n=1, h=None, f16_scale=True):
    """RMSNORM-Q8 (src/cuda-dense.lisp:260-264): RMSNORM! of N rows of X (D wide) by
    W, quantized into ACT in the kind it holds; H, when given, also gets the floats."""
    cf = getattr(act, "_cf", None)
    if act.kind == "q8k" and cf is not None and cf.n == n and cf.cols == d:
        # ACT's fp16 form is in use by the tcgen05 products: renewed in the same launch
        _lib.call("ill_rmsnorm_q8k_f16", _ptr(x), _ptr(w), _ptr(h), _ptr(act.xq), _ptr(act.xs), _ptr(act.xsum), _ptr(cf.xh),
                  _ptr(cf.xe), d, float(eps), n, _stream())
        cf.xd = act.xs
        act._cf_fresh = True
        return act
    _lib.call("ill_rmsnorm_q8", 1 if act.kind == "q8k" else 0, _ptr(x), _ptr(w), _ptr(h), _ptr(act.xq), _ptr(act.xs),
              _ptr(act.xsum), d, float(eps), n, 1 if f16_scale else 0, _stream())
    act._cf_fresh = False
    return act


def cmat_mul(w, act, y, n=1, bias=None, acc=False):
    """CMAT-MUL (src/cuda-dense.lisp:220-248): Y = W X for N tokens (token t's X
    at t*cols, its Y at t*rows), or Y += it when ACC."""
    if ((w.type == 1 or (w.type == 2 and TC_Q6K)) and act.kind == "q8k" and n >= TC_MIN_TOKENS and w.rows >= TC_MIN_ROWS and w.rows % 4 == 0 and bias is None
            and w.qs.data_ptr() % 16 == 0 and act.xq.numel() == n * w.cols):
        # a prefill chunk of a Q4_K / Q6_K matrix: the tcgen05 kernel (the activations' fp16 form is made once per quantization)
        return cmat_mul_tc(w, _chunk_f16_of(act, n, w.cols), y, acc=acc)
    done = 0
    # Q8_0 / Q4_K / Q6_K take a whole chunk of tokens in one launch; the other formats up to 16 tokens --
    # fewer when their activations do not fit beside the stages
    kmax = n
    while done < n:
        k = min(kmax, n - done)
        sc = w.cols // (32 if act.kind == "q8" else 256)
        rc = _lib.status("ill_mv", w.type, _ptr(w.qs), w.rows, w.cols,
                         act.xq.data_ptr() + done * w.cols, act.xs.data_ptr() + 4 * done * sc,
                         0 if act.kind == "q8" else act.xsum.data_ptr() + 2 * done * (w.cols // 16),
                         y.data_ptr() + 4 * done * w.rows, _ptr(bias), 1 if acc else 0, k, _stream())
        if rc == 3 and k > 1:   # ILL_ERR_UNSUPPORTED: long rows, many tokens
            kmax = 16 if k > 16 else k // 2
            continue
        if rc:
            _lib.call("ill_mv", w.type, _ptr(w.qs), w.rows, w.cols, act.xq.data_ptr() + done * w.cols,
                      act.xs.data_ptr() + 4 * done * sc, 0 if act.kind == "q8" else act.xsum.data_ptr() + 2 * done * (w.cols // 16),
                      y.data_ptr() + 4 * done * w.rows, _ptr(bias), 1 if acc else 0, k, _stream())  # raises with the text
        done += k
    return y


_SIDE = {}


def _side_stream(device):
    """A second stream per device for products that may run beside the current stream's."""
    s = _SIDE.get(device)
    if s is None:
        s = _SIDE[device] = torch.cuda.Stream(device=device)
    return s


def qkv_mul(wq, wk, wv, act, q, k, v, bq=None, bk=None, bv=None, n=1):
    """QKV-MUL (src/cuda-dense.lisp:309-324): one launch when the three formats
    agree and there is one token, else three products."""
    if n == 1 and wq.type == wk.type == wv.type:
        _lib.call("ill_mv_3", wq.type, _ptr(wq.qs), _ptr(wk.qs), _ptr(wv.qs), wq.rows, wk.rows, wv.rows, wq.cols,
                  _ptr(act.xq), _ptr(act.xs), _ptr(act.xsum) if act.kind == "q8k" else 0,
                  _ptr(q), _ptr(k), _ptr(v), _ptr(bq), _ptr(bk), _ptr(bv), _stream())
    elif n == 1 and wq.type == wk.type:
        # Q4_K_M files keep V in Q6_K: Q and K in one launch, V in its own -- beside it, on a second
        # stream (both read the same activations; in a captured graph this is a fork and a join)
        cur = torch.cuda.current_stream()
        side = _side_stream(cur.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            cmat_mul(wv, act, v, n, bias=bv)
        _lib.call("ill_mv_3", wq.type, _ptr(wq.qs), _ptr(wk.qs), 0, wq.rows, wk.rows, 0, wq.cols,
                  _ptr(act.xq), _ptr(act.xs), _ptr(act.xsum) if act.kind == "q8k" else 0,
                  _ptr(q), _ptr(k), 0, _ptr(bq), _ptr(bk), 0, _stream())
        cur.wait_stream(side)
    else:
        cmat_mul(wq, act, q, n, bias=bq)
        cmat_mul(wk, act, k, n, bias=bk)
        cmat_mul(wv, act, v, n, bias=bv)


def glu_mul(g, u, act, fa, n=1, fb=None):
    """GLU-MUL (src/cuda-dense.lisp:326-339): silu(G x) * (U x) into FA."""
    if n == 1 and g.type == u.type:
        _lib.call("ill_mv_glu", g.type, _ptr(g.qs), _ptr(u.qs), g.rows, g.cols, _ptr(act.xq), _ptr(act.xs),
                  _ptr(act.xsum) if act.kind == "q8k" else 0, _ptr(fa), _stream())
        return fa
    if fb is None:
        fb = torch.empty_like(fa)
    cmat_mul(g, act, fa, n)
    cmat_mul(u, act, fb, n)
    fa.copy_((fa / (1.0 + torch.exp(-fa))) * fb)  # the reference's swiglu kernel; not on the decode path
    return fa


class ChunkF16:
    """A chunk's Q8_K activations as the tcgen05 product takes them (ill_act_f16): XH [n, cols] the quants as fp16
    (exact), XE [n, cols / 256, 64] the sums of 16 as fp16 (exact; 48 of each 64 zero), XD the block scales."""

    def __init__(self, n, cols, device="cuda"):
        self.n, self.cols = n, cols
        self.xh = torch.empty(n, cols, dtype=torch.float16, device=device)
        self.xe = torch.empty(n, cols // 256, 64, dtype=torch.float16, device=device)
        self.xd = None

    def fill(self, act):
        _lib.call("ill_act_f16", self.n, self.cols, _ptr(act.xq), _ptr(act.xsum), 0, _ptr(self.xh), _ptr(self.xe), _stream())
        self.xd = act.xs
        return self


def cmat_mul_tc(w, cf, y, acc=False):
    """CMAT-MUL-N for a prefill chunk on the 5th-generation tensor cores (ill_mm_chunk): Y[t*rows + r] (+)= W[r] . X[t]
    for the chunk CF (a ChunkF16 filled from the chunk's Q8_K activations) and a Q4_K or Q6_K matrix W.  Replaces
    mm_q4k_mma / mm_q6k_mma (src/cuda/kquant.cu:316-466) behind CMAT-MUL-N (src/cuda-dense.lisp:250-255)."""
    _lib.call("ill_mm_chunk", w.type, _ptr(w.qs), w.rows, w.cols, _ptr(cf.xh), _ptr(cf.xe), _ptr(cf.xd), cf.n, _ptr(y),
              1 if acc else 0, _stream())
    return y


def glu_mul_tc(g, u, act, n, fa, fb):
    """The gate and up products of a gated FFN over a prefill chunk in one launch of the tcgen05 kernel
    (ill_mm_chunk2): FA = G X, FB = U X for the chunk's Q8_K activations ACT.  Both matrices of one format and
    shape, and large enough for tc_takes()."""
    cf = _chunk_f16_of(act, n, g.cols)
    _lib.call("ill_mm_chunk2", g.type, _ptr(g.qs), _ptr(u.qs), g.rows, g.cols, _ptr(cf.xh), _ptr(cf.xe), _ptr(cf.xd), n, _ptr(fa),
              _ptr(fb), _stream())
    return fa, fb


def swiglu_chunk_f16(g, u, cf, clamp=3.0e38):
    """silu(G) * U over a chunk's [n, ff] gate and up products, quantized to Q8_K and left in CF (a ChunkF16 of n x ff)
    in the form the tcgen05 product takes -- the swiglu, quant_q8 and fp16 steps between a prefill chunk's up and
    down products in one launch (ill_swiglu_q8k_f16: each step's arithmetic, bit for bit)."""
    n, ff = cf.n, cf.cols
    if cf.xd is None or cf.xd.numel() != n * ff // 256:
        cf.xd = torch.empty(n * ff // 256, dtype=torch.float32, device=cf.xh.device)
    _lib.call("ill_swiglu_q8k_f16", n, ff, float(clamp), _ptr(g), _ptr(u), 0, _ptr(cf.xh), _ptr(cf.xe), _ptr(cf.xd), 0, _stream())
    return cf


def tc_takes(w, n):
    """Whether cmat_mul sends N tokens of matrix W to the tcgen05 kernel."""
    return ((w.type == 1 or (w.type == 2 and TC_Q6K)) and n >= TC_MIN_TOKENS and w.rows >= TC_MIN_ROWS and w.rows % 4 == 0
            and w.qs.data_ptr() % 16 == 0)


TC_MIN_TOKENS, TC_MIN_ROWS = 64, 2048   # below these the int8 mma.sync kernel is as fast or faster
# Q6_K on the tcgen05 path: scale * (q - 32) reaches 4064 and fp16 holds only even integers above 2048, so the kernel
# multiplies an even part and an odd part of every product (both exact).  False keeps Q6_K chunks on the int8 kernel.
TC_Q6K = True


def _chunk_f16_of(act, n, cols):
    """ACT's fp16 form for the tcgen05 product, made once per quantization of ACT (quant_q8 / rmsnorm_q8 mark it stale)."""
    cf = getattr(act, "_cf", None)
    if cf is None or cf.n != n or cf.cols != cols:
        cf = act._cf = ChunkF16(n, cols, device=act.xq.device)
        act._cf_fresh = False
    if not getattr(act, "_cf_fresh", False):
        cf.fill(act)
        act._cf_fresh = True
    return cf


def swiglu(g, u, out, ff, clamp=3.0e38):
    """OUT = silu(G) * U over whole rows of FF values (the reference's swiglu launch between the gate / up and the
    down products of a prefill chunk, src/cuda-dense.lisp:326-339); CLAMP as d4_swiglu_w clamps, off by default."""
    _lib.call("ill_swiglu_w", g.numel(), ff, float(clamp), _ptr(g), _ptr(u), 0, _ptr(out), _stream())
    return out


OP_MV, OP_GLU = 0, 1


def decode_op(w, x, y, w2=None, norm_w=None, eps=1e-6, bias=None, acc=False, after=True, f16_scale=True):
    """One product of a token's chain for DecodePlan: Y (+)= W X' (+ BIAS), or Y = silu(W X') * (W2 X') when W2 is
    given; X' = X (floats on the device) after RMSNORM! by NORM_W (when given) and the quantizer W's format takes.
    AFTER: the product reads or adds into what an earlier one of the chain writes."""
    import ctypes
    op = _lib.DecodeOp()
    op.w, op.w2, op.x, op.norm_w, op.y, op.bias = _ptr(w.qs), _ptr(w2.qs) if w2 is not None else 0, _ptr(x), _ptr(norm_w), _ptr(y), _ptr(bias)
    op.fmt, op.kind, op.rows, op.cols = w.type, OP_GLU if w2 is not None else OP_MV, w.rows, w.cols
    op.acc, op.after, op.f16_scale, op.eps = int(bool(acc)), int(bool(after)), int(bool(f16_scale)), float(eps)
    if w2 is not None and (w2.type, w2.rows, w2.cols) != (w.type, w.rows, w.cols):
        raise ValueError("a gated product's two matrices must agree in format and shape")
    return op


class DecodePlan:
    """A token's chain of products run as ONE launch (ill_decode_plan / ill_decode_run): what CUDA-FORWARD-N
    (src/cuda-dense.lisp:380-432) issues as a launch per product and per quantization.  OPS: decode_op()s in
    order.  The plan lives in device memory this object owns; run() enqueues one token on the current stream."""

    def __init__(self, ops, device="cuda"):
        import ctypes
        self.n = len(ops)
        arr = (_lib.DecodeOp * self.n)(*ops)
        nbytes = _lib.lib().ill_decode_plan_bytes(self.n)
        if nbytes <= 0:
            raise ValueError("a chain holds 1 to 1024 products")
        self.plan = torch.zeros(nbytes + 128, dtype=torch.uint8, device=device)
        self.base = (self.plan.data_ptr() + 127) // 128 * 128
        self.launch = (ctypes.c_int32 * 16)()
        with torch.cuda.device(self.plan.device):
            _lib.call("ill_decode_plan", arr, self.n, self.base, nbytes, self.launch, _stream())

    def run(self):
        _lib.call("ill_decode_run", self.base, self.launch, _stream())


def embed(emb, tokens, x):
    """EMBED (src/cuda-dense.lisp:302-307): rows TOKENS (int32 on the device) of
    EMB as floats in X."""
    _lib.call("ill_dequant_rows", emb.type, _ptr(emb.qs), emb.cols, _ptr(tokens), 0, tokens.numel(), _ptr(x),
              _stream())
    return x


def dequant_rows(w, first_row, nrows, out=None):
    """Rows FIRST_ROW.. of W as floats (the bit-exactness check point)."""
    if out is None:
        out = torch.empty(nrows, w.cols, dtype=torch.float32, device=w.qs.device)
    _lib.call("ill_dequant_rows", w.type, _ptr(w.qs), w.cols, 0, first_row, nrows, _ptr(out), _stream())
    return out


def device_status():
    """The device status word (0 = no kernel gave up a wait); synchronises."""
    import ctypes
    v = ctypes.c_uint(0)
    _lib.status("ill_device_status", ctypes.byref(v), _stream())
    return v.value
