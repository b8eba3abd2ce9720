"""Host side of the mixture-of-experts decode path: the reference's
src/cuda-ds4f.lisp (DK-Q8MV, DK-FFN-HEAD's shared expert, DK-FFN-TAIL) mirrored
over the C ABI.

On a B200 every expert is resident in HBM, so the reference's slot pool, LRU,
second-device tier, CPU share and read-through (src/cuda-ds4f.lisp:367-750) have
nothing to do: a "slot" is simply an expert's `gate | up | down` block in one
buffer (the layout D4-HOST-EXPERTS builds, src/cuda-ds4f.lisp:162-166) and every
lookup hits.  Routing is done on the device (ill_moe_route) instead of on the
CPU after a download of the logits (src/cuda-ds4f.lisp:991-999).
"""
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from . import cuda_dense as D
from .blocks import IQ2_XXS, Q2_K, Q8_0, row_bytes


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


@dataclass
class ExpertPool:
    """All experts of a layer in device memory: slot e = gate | up | down
    (DK-POOL with every expert held; src/cuda-ds4f.lisp:286-306)."""
    d: int
    ff: int
    gate_fmt: int
    down_fmt: int
    n_expert: int
    pool: torch.Tensor        # uint8 [n_expert * slot_bytes]
    slot_bytes: int
    gate_bytes: int           # bytes of gate (= bytes of up); down starts at 2 * gate_bytes
    down_bytes: int
    ptrs_all: torch.Tensor    # uint64 [n_expert]: device address of each slot

    def slot_ptrs(self, experts):
        """Device table of the slots' addresses for EXPERTS (a device int tensor)."""
        return self.ptrs_all[experts.to(torch.int64)]


def make_expert_pool(gate, up, down, d, ff, n_expert, gate_fmt=IQ2_XXS, down_fmt=Q2_K, device="cuda"):
    """Lay the three expert tensors (raw blocks, expert-major as in the GGUF:
    expert e's row r at (e*rows + r)*row_bytes, src/ds4f.lisp:1014-1015) out as
    one slot per expert, 256-byte aligned (src/cuda-ds4f.lisp:299)."""
    gb = ff * row_bytes(gate_fmt, d)
    db = d * row_bytes(down_fmt, ff)
    slot = (2 * gb + db + 255) // 256 * 256
    pool = torch.zeros(n_expert * slot, dtype=torch.uint8, device=device)
    pv = pool.view(n_expert, slot)
    pv[:, :gb] = torch.as_tensor(gate).to(device).view(n_expert, gb)
    pv[:, gb:2 * gb] = torch.as_tensor(up).to(device).view(n_expert, gb)
    pv[:, 2 * gb:2 * gb + db] = torch.as_tensor(down).to(device).view(n_expert, db)
    base = pool.data_ptr()
    ptrs = torch.tensor([base + e * slot for e in range(n_expert)], dtype=torch.int64, device=device)
    return ExpertPool(d, ff, gate_fmt, down_fmt, n_expert, pool, slot, gb, db, ptrs)


def dk_q8mv(w, x, y, q=None):
    """DK-Q8MV (src/cuda-ds4f.lisp:773-782): Y = W X for a Q8_0 W, X quantized as
    ds4 does (the block scale stays a float) unless Q has it already."""
    if q is None:
        q = D.make_qact(w.cols, "q8", device=x.device)
        D.quant_q8(x, q, f16_scale=False)
    D.cmat_mul(w, q, y, 1)
    return q


F32, F16, BF16 = 0, 1, 2
_DENSE_TYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def dk_mv16(w, x, y, n=1):
    """DK-MV16 (src/cuda-ds4f.lisp:767-771): Y = W X for an unquantized tensor W [rows, cols]
    (float32, float16 or bfloat16 on the device) and N tokens' float activations."""
    rows, cols = w.shape
    _lib.call("ill_mv_dense", _DENSE_TYPES[w.dtype], _ptr(w), rows, cols, _ptr(x), _ptr(y), n, rows, _stream())
    return y


def swiglu_w(g, u, w, mid, ff, clamp):
    """d4_swiglu_w (src/cuda-ds4f.lisp:939): MID = silu(min(G,c)) * clamp(U) * W[row]."""
    _lib.call("ill_swiglu_w", g.numel(), ff, float(clamp), _ptr(g), _ptr(u), _ptr(w), _ptr(mid), _stream())
    return mid


def dk_shared(sh_gate, sh_up, sh_down, norm, clamp, out):
    """The shared expert as DK-FFN-HEAD runs it (src/cuda-ds4f.lisp:900-906):
    D4-SHARED! (src/ds4f.lisp:1039-1048)."""
    ff = sh_gate.rows
    g = torch.empty(ff, device=norm.device)
    u = torch.empty(ff, device=norm.device)
    q = dk_q8mv(sh_gate, norm, g)
    dk_q8mv(sh_up, norm, u, q=q)
    mid = torch.empty(ff, device=norm.device)
    swiglu_w(g, u, None, mid, ff, clamp)
    dk_q8mv(sh_down, mid, out)
    return out


def route(logits, nu, mode=2, bias=None, scale=1.0):
    """D4-ROUTE / G53-ROUTE on the device for every row of LOGITS [n, ne]."""
    n, ne = logits.shape
    sel = torch.empty(n, nu, dtype=torch.int32, device=logits.device)
    w = torch.empty(n, nu, dtype=torch.float32, device=logits.device)
    _lib.call("ill_moe_route", ne, nu, mode, float(scale), n, _ptr(logits), _ptr(bias), _ptr(sel), _ptr(w), _stream())
    return sel, w


def dk_ffn_tail(pool, norm2, sel, w, clamp, shared=None, moe=None):
    """DK-FFN-TAIL (src/cuda-ds4f.lisp:908-956) for one token: the routed experts
    SEL (device int32 [k]) with weights W (device float [k]) on the FFN input
    NORM2, summed in SEL's order with the shared expert's output SHARED."""
    d, ff, k = pool.d, pool.ff, sel.numel()
    dev = norm2.device
    xq = D.make_qact(d, "q8k", device=dev)
    D.quant_q8(norm2, xq)
    ptrs = pool.slot_ptrs(sel)
    mid = torch.empty(k * ff, device=dev)
    _lib.call("ill_moe_glu", pool.gate_fmt, d, ff, 0, pool.gate_bytes, _ptr(ptrs), k, _ptr(xq.xq), _ptr(xq.xs),
              _ptr(xq.xsum), 0, float(clamp), _ptr(w), _ptr(mid), ff, _stream())
    midq = D.make_qact(k * ff, "q8k", device=dev)
    D.quant_q8(mid, midq)  # a slot's FF values are whole super-blocks: quantized apart (src/ds4f.lisp:1021-1022)
    bd = torch.empty(k * d, device=dev)
    _lib.call("ill_moe_mv", pool.down_fmt, ff, d, 2 * pool.gate_bytes, _ptr(ptrs), k, _ptr(midq.xq), _ptr(midq.xs),
              _ptr(midq.xsum), 1, _ptr(bd), d, _stream())
    if moe is None:
        moe = torch.empty(d, device=dev)
    _lib.call("ill_moe_sum", d, k, 1, _ptr(bd), 0, _ptr(shared), _ptr(moe), _stream())
    return moe, mid
