"""Host side of the mixture-of-experts prefill path: DK-FFN-ROUTED-CHUNK of the
reference's src/cuda-ds4f-prefill.lisp (:315-356), mirrored over the C ABI.

The chunk's routing, grouping and products all run on the device with no host
synchronisation, as in the reference; the products run on tcgen05 tensor cores
over the Q8_K-quantized activations (so the results follow the reference's CPU
prefill, src/ds4f.lisp:1168-1239, within fp16 operand rounding).
"""
from dataclasses import dataclass

import torch

from . import _lib
from . import cuda_dense as D
from .blocks import Q2_K
from .cuda_ds4f import _DENSE_TYPES, ExpertPool, swiglu_w


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


@dataclass
class ChunkScratch:
    """The buffers of a chunk (the reference's PB scratch, src/cuda-ds4f-prefill.lisp:35-47)."""
    n: int
    rows: int
    sel: torch.Tensor
    w: torch.Tensor
    counts: torch.Tensor
    bases: torch.Tensor
    rmap: torch.Tensor
    smap: torch.Tensor
    wrow: torch.Tensor
    group: torch.Tensor
    xq: D.QAct
    xh: torch.Tensor
    xe: torch.Tensor
    g: torch.Tensor
    u: torch.Tensor
    mid: torch.Tensor
    midq: D.QAct
    mh: torch.Tensor
    me: torch.Tensor
    down: torch.Tensor
    moe: torch.Tensor


def make_chunk_scratch(pool, n, nu, device="cuda"):
    d, ff, ne = pool.d, pool.ff, pool.n_expert
    rows = n * nu
    i32 = dict(dtype=torch.int32, device=device)
    f32 = dict(dtype=torch.float32, device=device)
    return ChunkScratch(
        n, rows, torch.empty(n, nu, **i32), torch.empty(n, nu, **f32), torch.empty(ne, **i32), torch.empty(ne, **i32),
        torch.empty(rows, **i32), torch.empty(rows, **i32), torch.empty(rows, **f32),
        torch.empty(_lib.lib().ill_moe_group_scratch_bytes(rows, ne), dtype=torch.uint8, device=device),
        D.make_qact(n * d, "q8k", device=device), torch.empty(rows, d, dtype=torch.float16, device=device),
        torch.empty(rows, d // 256, 64, dtype=torch.float16, device=device) if pool.gate_fmt == Q2_K else None,
        torch.empty(rows, ff, **f32), torch.empty(rows, ff, **f32), torch.empty(rows, ff, **f32),
        D.make_qact(rows * ff, "q8k", device=device), torch.empty(rows, ff, dtype=torch.float16, device=device),
        torch.empty(rows, ff // 256, 64, dtype=torch.float16, device=device) if pool.down_fmt == Q2_K else None,
        torch.empty(rows, d, **f32), torch.empty(n, d, **f32))


def act_f16(act, cols, rows, rmap, xh, xe):
    """The Q8_K activations ACT as fp16 integers in expert order (and the sums of 16)."""
    _lib.call("ill_act_f16", rows, cols, _ptr(act.xq), _ptr(act.xsum), _ptr(rmap), _ptr(xh), _ptr(xe), _stream())


def mm_id(pool, fmt, ncols, nrows, add, sc, xh, xe, xd, rmap, y):
    """d4_mm_id_<fmt> (src/cuda-ds4f-prefill.lisp:345-347); every expert is resident."""
    _lib.call("ill_moe_mm_id", fmt, ncols, nrows, add, _ptr(pool.ptrs_all), _ptr(sc.counts), _ptr(sc.bases),
              pool.n_expert, sc.rows, _ptr(xh), _ptr(xe), _ptr(xd), _ptr(rmap), 0, _ptr(y), nrows, _stream())


def dk_ffn_routed_chunk(pool, norms, logits, nu, clamp, sc, mode=2, bias=None, scale=1.0, shared=None, fused=True):
    """DK-FFN-ROUTED-CHUNK (src/cuda-ds4f-prefill.lisp:315-356): the chunk's N
    tokens (NORMS [n, d] floats, LOGITS [n, ne] router logits) through their
    routed experts; returns MOE [n, d] (plus SHARED [n, d] when given)."""
    n, d = norms.shape
    ff, ne = pool.ff, pool.n_expert
    st = _stream()
    _lib.call("ill_moe_route", ne, nu, mode, float(scale), n, _ptr(logits), _ptr(bias), _ptr(sc.sel), _ptr(sc.w), st)
    _lib.call("ill_moe_group", sc.rows, ne, nu, _ptr(sc.sel), _ptr(sc.w), _ptr(sc.group), _ptr(sc.counts),
              _ptr(sc.bases), _ptr(sc.rmap), _ptr(sc.smap), _ptr(sc.wrow), st)
    D.quant_q8(norms, sc.xq)                                       # each token's Q8_K, once
    act_f16(sc.xq, d, sc.rows, sc.rmap, sc.xh, sc.xe)
    if fused:  # gate and up in one launch
        _lib.call("ill_moe_mm_id2", pool.gate_fmt, d, ff, 0, pool.gate_bytes, _ptr(pool.ptrs_all), _ptr(sc.counts), _ptr(sc.bases),
                  pool.n_expert, sc.rows, _ptr(sc.xh), _ptr(sc.xe), _ptr(sc.xq.xs), _ptr(sc.rmap), _ptr(sc.g), _ptr(sc.u), ff, st)
    else:
        mm_id(pool, pool.gate_fmt, d, ff, 0, sc, sc.xh, sc.xe, sc.xq.xs, sc.rmap, sc.g)
        mm_id(pool, pool.gate_fmt, d, ff, pool.gate_bytes, sc, sc.xh, sc.xe, sc.xq.xs, sc.rmap, sc.u)
    if fused:  # the three steps below in one pass (same results bit for bit; sc.mid and sc.midq.xq stay unwritten)
        _lib.call("ill_swiglu_q8k_f16", sc.rows, ff, float(clamp), _ptr(sc.g), _ptr(sc.u), _ptr(sc.wrow), _ptr(sc.mh),
                  _ptr(sc.me), _ptr(sc.midq.xs), 0, st)
    else:
        swiglu_w(sc.g, sc.u, sc.wrow, sc.mid, ff, clamp)
        D.quant_q8(sc.mid, sc.midq)                                # per (token, slot) row, as the CPU path does
        act_f16(sc.midq, ff, sc.rows, None, sc.mh, sc.me)
    mm_id(pool, pool.down_fmt, ff, d, 2 * pool.gate_bytes, sc, sc.mh, sc.me, sc.midq.xs, None, sc.down)
    _lib.call("ill_moe_sum", d, nu, n, _ptr(sc.down), _ptr(sc.smap), _ptr(shared), _ptr(sc.moe), st)
    return sc.moe


def dk_ffn_small(pool, norms, logits, nu, clamp, sc, **kw):
    """DK-FFN-SMALL (src/cuda-ds4f-spec.lisp:31-132): the routed experts for a few tokens at once -- several decode
    sequences, or the positions of a speculative run -- with the rows grouped by expert so that an expert's weights
    are read once for all of its tokens.  The reference multiplies with its matvec kernels given COUNTS / BASES
    (src/cuda/ds4f.cu:769-772); here the grouping and the products are the chunk driver's: the tcgen05 kernel takes
    tiles of as few as 16 rows, and for the 2-bit expert formats it is the faster of the two forms (their matvecs
    are bound by instructions, not by the bytes they read).  Same arguments and result as dk_ffn_routed_chunk."""
    return dk_ffn_routed_chunk(pool, norms, logits, nu, clamp, sc, **kw)


def dk_ffn_small_mv(pool, norms, logits, nu, clamp, sc, mode=2, bias=None, scale=1.0, shared=None):
    """DK-FFN-SMALL on the matvec path, as the reference runs it (src/cuda-ds4f-spec.lisp:82-97): the rows grouped by
    expert, the tokens' FFN inputs gathered row by row (d4_gather_rows), then the one-token kernels with an expert's
    rows next to each other -- ill_moe_glu (gate, up, SwiGLU and the routing weight in one launch), the middle values'
    Q8_K, ill_moe_mv for down -- and the sum in slot order.  Same arguments and result as dk_ffn_routed_chunk (whose
    scratch it uses, plus a table of a pointer a row and the gathered rows, made on first use)."""
    n, d = norms.shape
    ff, ne = pool.ff, pool.n_expert
    st = _stream()
    if not hasattr(sc, "row_ptrs"):
        sc.row_ptrs = torch.empty(sc.rows, dtype=torch.int64, device=norms.device)
        sc.xrows = torch.empty(sc.rows, d, dtype=torch.float32, device=norms.device)
        sc.xrowq = D.make_qact(sc.rows * d, "q8k", device=norms.device)
    _lib.call("ill_moe_route", ne, nu, mode, float(scale), n, _ptr(logits), _ptr(bias), _ptr(sc.sel), _ptr(sc.w), st)
    _lib.call("ill_moe_group", sc.rows, ne, nu, _ptr(sc.sel), _ptr(sc.w), _ptr(sc.group), _ptr(sc.counts),
              _ptr(sc.bases), _ptr(sc.rmap), _ptr(sc.smap), _ptr(sc.wrow), st)
    _lib.call("ill_moe_row_ptrs", ne, _ptr(pool.ptrs_all), _ptr(sc.counts), _ptr(sc.bases), sc.rows, _ptr(sc.row_ptrs), st)
    _lib.call("ill_gather_rows", sc.rows, 4 * d, _ptr(norms), _ptr(sc.rmap), _ptr(sc.xrows), st)
    D.quant_q8(sc.xrows, sc.xrowq)
    _lib.call("ill_moe_glu", pool.gate_fmt, d, ff, 0, pool.gate_bytes, _ptr(sc.row_ptrs), sc.rows, _ptr(sc.xrowq.xq),
              _ptr(sc.xrowq.xs), _ptr(sc.xrowq.xsum), 1, float(clamp), _ptr(sc.wrow), _ptr(sc.mid), ff, st)
    D.quant_q8(sc.mid, sc.midq)
    _lib.call("ill_moe_mv", pool.down_fmt, ff, d, 2 * pool.gate_bytes, _ptr(sc.row_ptrs), sc.rows, _ptr(sc.midq.xq),
              _ptr(sc.midq.xs), _ptr(sc.midq.xsum), 1, _ptr(sc.down), d, st)
    _lib.call("ill_moe_sum", d, nu, n, _ptr(sc.down), _ptr(sc.smap), _ptr(shared), _ptr(sc.moe), st)
    return sc.moe


class HeadScratch:
    """The buffers of DK-FFN-HEAD-CHUNK for up to N tokens: NORM2 [n, d] floats and their Q8_0 quantization, the
    router's LOGITS [n, ne], the shared expert's gate / up [n, ff], the middle values' quantization, SOUT [n, d]."""

    def __init__(self, n, d, ff, ne, device="cuda"):
        f = dict(dtype=torch.float32, device=device)
        self.n, self.d, self.ff, self.ne = n, d, ff, ne
        self.norm2, self.logits = torch.empty(n, d, **f), torch.empty(n, ne, **f)
        self.sg, self.su, self.sout = torch.empty(n, ff, **f), torch.empty(n, ff, **f), torch.empty(n, d, **f)
        self.nq, self.mq = D.make_qact(n * d, "q8", device=device), D.make_qact(n * ff, "q8", device=device)


def dk_ffn_head_chunk(cur, norm_w, eps, router, sh_gate, sh_up, sh_down, clamp, hs):
    """DK-FFN-HEAD-CHUNK (src/cuda-ds4f-prefill.lisp:285-303) past its hyper-connection step: CUR [n, d] -> RMSNorm
    (NORM2) -> the router's logits (ROUTER: an unquantized [ne, d] tensor) and the shared expert
    (SH_GATE / SH_UP / SH_DOWN: Q8_0 matrices; d4_swiglu_w with weights of one between them) over the whole chunk.
    Returns (norm2, logits, sout): what DK-FFN-ROUTED-CHUNK takes as NORMS, LOGITS and SHARED."""
    n, d = cur.shape
    ne = router.shape[0]
    norm2, logits, sout = hs.norm2[:n], hs.logits[:n], hs.sout[:n]
    sg, su = hs.sg[:n], hs.su[:n]
    D.rmsnorm_q8(cur, norm_w, hs.nq, d, eps, n=n, h=norm2, f16_scale=False)     # DK-RMS and DK-Q8MM's quantization of NORM2
    _lib.call("ill_mv_dense", _DENSE_TYPES[router.dtype], _ptr(router), ne, d, _ptr(norm2), _ptr(logits), n, ne, _stream())
    D.cmat_mul(sh_gate, hs.nq, sg, n)
    D.cmat_mul(sh_up, hs.nq, su, n)
    _lib.call("ill_swiglu_w", n * hs.ff, hs.ff, float(clamp), _ptr(sg), _ptr(su), 0, _ptr(sg), _stream())
    D.quant_q8(sg, hs.mq, f16_scale=False)
    D.cmat_mul(sh_down, hs.mq, sout, n)
    return norm2, logits, sout
