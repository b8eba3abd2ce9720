"""Expert parallelism and the row-split output head over the GPUs of one box.

The reference has no multi-GPU path of this kind: its second device holds a
fixed "tier" of experts and exchanges activations through pinned host memory
(D4-TIER-LAUNCH, src/cuda-ds4f.lisp:594-618), and "a model split across the
two GPUs" is an open item (TODO.md:112).  Here:

* Experts are placed expert-parallel: rank r of G holds experts
  [r*E/G, (r+1)*E/G) resident in its HBM.  A chunk's tokens are split evenly by
  position; every rank routes its own tokens, sends each (token, slot) row to
  the rank that owns the chosen expert (all-to-all over NVLink, NCCL), runs the
  indexed products for its experts, and sends the down rows back; the owner of
  a token adds its slots' rows in slot order, as D4_MOE_SUM_ROWS does.
  What travels is the token's Q8_K form (int8 quants, block scales, sums of 16:
  1.14 bytes a value) -- fewer bytes than bf16 and exactly what the products
  consume, so the result is bit-identical to the single-GPU path whatever G is.
  The down rows come back as fp32 so that the slot-order sum is unchanged.
* The output head (151936 rows) is split by rows; each rank multiplies its slice
  into its part of the logits buffer and one in-place all-gather completes it.

The index plumbing (which rows go where, where arrivals land) is written with
plain torch ops on whatever device the tensors live on, so it is tested on CPU
ranks over gloo; the products are the CUDA kernels.
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist


def expert_owner(experts, n_expert, world):
    """Rank that holds each expert: contiguous blocks of n_expert / world."""
    return experts // (n_expert // world)


@dataclass
class DispatchPlan:
    """Where a rank's grouped rows go and where the rows it receives land."""
    send_counts: list          # rows sent to each rank (host ints)
    recv_counts: list          # rows received from each rank (host ints)
    recv_expert_counts: torch.Tensor   # [world, local experts] rows from each source for each local expert
    counts: torch.Tensor       # [local experts] rows per local expert (int32)
    bases: torch.Tensor        # [local experts] first place of each local expert (int32)
    place_to_recv: torch.Tensor  # [total recv rows] arrival index of the row at each place (int32)
    recv_to_place: torch.Tensor  # inverse


def plan_dispatch(local_counts, world, group=None):
    """LOCAL_COUNTS: this rank's rows per expert (all E experts, int32/int64 on any
    device), its rows already sorted by expert.  Exchanges the counts (one small
    all-to-all) and builds the plan.  Rows arrive source by source, each source's
    rows in expert order; an expert's rows are placed source after source, so the
    place order is (expert, source, arrival order)."""
    E = local_counts.numel()
    per = E // world
    dev = local_counts.device
    lc = local_counts.to(torch.int64).view(world, per)          # [dest rank, its experts]
    if world > 1:
        rc = torch.empty_like(lc)                                # [source rank, my experts]
        dist.all_to_all_single(rc, lc.contiguous(), group=group)
    else:
        rc = lc.clone()
    send_counts = lc.sum(1).tolist()                             # host: the split sizes NCCL needs
    recv_counts = rc.sum(1).tolist()
    counts = rc.sum(0)                                           # per local expert
    bases = torch.cumsum(counts, 0) - counts
    # arrival index of (source s, expert e, i): offset of source s + offset of e inside s + i
    src_off = torch.cumsum(rc.sum(1), 0) - rc.sum(1)             # [world]
    in_src = torch.cumsum(rc, 1) - rc                            # [world, per]
    # place of (s, e, i): bases[e] + rows of e from sources before s + i
    before = torch.cumsum(rc, 0) - rc                            # [world, per]
    total = int(sum(recv_counts))
    seg_len = rc.reshape(-1)                                     # segments in arrival order: (s, e)
    seg_arrival = (src_off[:, None] + in_src).reshape(-1)
    seg_place = (bases[None, :] + before).reshape(-1)
    seg_id = torch.repeat_interleave(torch.arange(seg_len.numel(), device=dev), seg_len, output_size=total)
    within = torch.arange(total, device=dev) - torch.repeat_interleave(seg_arrival, seg_len, output_size=total)
    recv_to_place = (seg_place[seg_id] + within).to(torch.int32)  # arrival order is seg_arrival + within = arange
    place_to_recv = torch.empty(total, dtype=torch.int32, device=dev)
    place_to_recv[recv_to_place.long()] = torch.arange(total, dtype=torch.int32, device=dev)
    return DispatchPlan(send_counts, recv_counts, rc, counts.to(torch.int32), bases.to(torch.int32), place_to_recv,
                        recv_to_place)


def exchange_rows(rows, send_counts, recv_counts, group=None):
    """All-to-all of ROWS [n, ...] split by SEND_COUNTS; returns the received rows."""
    total = int(sum(recv_counts))
    out = torch.empty((total,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        # rows travel as bytes: NCCL has no 16-bit integer type, and the payload is opaque to it anyway
        src = rows.contiguous().view(rows.shape[0], -1).view(torch.uint8)
        dst = out.view(total, -1).view(torch.uint8)
        dist.all_to_all_single(dst, src, output_split_sizes=list(recv_counts), input_split_sizes=list(send_counts),
                               group=group)
    else:
        out.copy_(rows)
    return out


def moe_chunk_ep(norms, logits, nu, route_fn, quantize_fn, expert_fn, sum_fn, n_expert, group=None):
    """One chunk's routed experts over the ranks of GROUP; every rank passes its
    own tokens (NORMS [n, d], LOGITS [n, E]) and gets its tokens' output.

    The compute steps are callables so that the same plumbing runs the CUDA
    kernels on GPUs and stand-ins on CPU ranks in the tests:
      route_fn(logits) -> sel [n, nu] int, w [n, nu] float
      quantize_fn(norms) -> tuple of per-token row tensors (what a row carries)
      expert_fn(payload rows (tuple, arrival order), wrow, plan) -> down rows [recv rows, d] in arrival order
      sum_fn(down rows back in send order [n*nu, d], smap [n*nu]) -> [n, d]
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    n = norms.shape[0]
    sel, w = route_fn(logits)
    flat = sel.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)                     # this rank's rows grouped by expert, token order inside
    local_counts = torch.bincount(flat, minlength=n_expert)
    plan = plan_dispatch(local_counts, world, group)
    tok = (order // nu)
    payload = quantize_fn(norms)
    sent = tuple(exchange_rows(p[tok], plan.send_counts, plan.recv_counts, group) for p in payload)
    wrow = exchange_rows(w.reshape(-1)[order].contiguous(), plan.send_counts, plan.recv_counts, group)
    down = expert_fn(sent, wrow, plan)                           # arrival order
    back = exchange_rows(down, plan.recv_counts, plan.send_counts, group)  # rows return in the order they were sent
    smap = torch.empty_like(order)
    smap[order] = torch.arange(order.numel(), device=order.device)
    return sum_fn(back, smap.to(torch.int32), n)


# ---- the CUDA steps ----------------------------------------------------------------------

class CudaExperts:
    """This rank's experts and the CUDA steps of moe_chunk_ep."""

    def __init__(self, pool, nu, clamp, mode=2, scale=1.0):
        self.pool, self.nu, self.clamp, self.mode, self.scale = pool, nu, clamp, mode, scale

    def route(self, logits):
        from . import cuda_ds4f as M
        return M.route(logits, self.nu, mode=self.mode, scale=self.scale)

    def quantize(self, norms):
        from . import cuda_dense as D
        n, d = norms.shape
        act = D.make_qact(n * d, "q8k", device=norms.device)
        D.quant_q8(norms.contiguous(), act)
        return (act.xq.view(n, d), act.xs.view(n, d // 256), act.xsum.view(n, d // 16))

    def experts(self, payload, wrow, plan):
        """The local experts' gate / up / down on the arrived rows; rows back in arrival order."""
        from . import _lib
        from . import cuda_dense as D
        from .blocks import Q2_K
        from .cuda_ds4f import swiglu_w
        pool = self.pool
        d, ff = pool.d, pool.ff
        xq, xd, xbs = (p.contiguous() for p in payload)
        rows = xq.shape[0]
        dev = xq.device
        st = torch.cuda.current_stream().cuda_stream
        f32 = dict(dtype=torch.float32, device=dev)
        if rows == 0:
            return torch.empty(0, d, **f32)
        p2r = plan.place_to_recv
        xh = torch.empty(rows, d, dtype=torch.float16, device=dev)
        xe = torch.empty(rows, d // 256, 64, dtype=torch.float16, device=dev) if pool.gate_fmt == Q2_K else None
        ptr = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
        _lib.call("ill_act_f16", rows, d, ptr(xq), ptr(xbs), ptr(p2r), ptr(xh), ptr(xe), st)
        g, u = torch.empty(rows, ff, **f32), torch.empty(rows, ff, **f32)
        for add, y in ((0, g), (pool.gate_bytes, u)):
            _lib.call("ill_moe_mm_id", pool.gate_fmt, d, ff, add, ptr(pool.ptrs_all), ptr(plan.counts), ptr(plan.bases),
                      pool.n_expert, rows, ptr(xh), ptr(xe), ptr(xd), ptr(p2r), 0, ptr(y), ff, st)
        wplace = wrow[p2r.long()].contiguous()
        mid = torch.empty(rows, ff, **f32)
        swiglu_w(g, u, wplace, mid, ff, self.clamp)
        midq = D.make_qact(rows * ff, "q8k", device=dev)
        D.quant_q8(mid, midq)
        mh = torch.empty(rows, ff, dtype=torch.float16, device=dev)
        me = torch.empty(rows, ff // 256, 64, dtype=torch.float16, device=dev) if pool.down_fmt == Q2_K else None
        _lib.call("ill_act_f16", rows, ff, ptr(midq.xq), ptr(midq.xsum), 0, ptr(mh), ptr(me), st)
        down = torch.empty(rows, d, **f32)
        _lib.call("ill_moe_mm_id", pool.down_fmt, ff, d, 2 * pool.gate_bytes, ptr(pool.ptrs_all), ptr(plan.counts),
                  ptr(plan.bases), pool.n_expert, rows, ptr(mh), ptr(me), ptr(midq.xs), 0, 0, ptr(down), d, st)
        out = torch.empty_like(down)
        _lib.call("ill_gather_rows", rows, d * 4, ptr(down), ptr(plan.recv_to_place), ptr(out), st)
        return out

    def sum(self, back, smap, n):
        from . import _lib
        d = back.shape[1]
        moe = torch.empty(n, d, dtype=torch.float32, device=back.device)
        _lib.call("ill_moe_sum", d, self.nu, n, back.data_ptr(), smap.data_ptr(), 0, moe.data_ptr(),
                  torch.cuda.current_stream().cuda_stream)
        return moe

    def chunk(self, norms, logits, n_expert_total, group=None):
        return moe_chunk_ep(norms, logits, self.nu, self.route, self.quantize, self.experts, self.sum, n_expert_total,
                            group)


class EpScratch:
    """Buffers of CudaExperts.chunk_fast for chunks of up to N tokens a rank: nothing
    is allocated per chunk.  A rank may receive every row of the chunk (CAP)."""

    def __init__(self, pool, n, nu, n_expert_total, world, device="cuda"):
        from . import _lib
        from .blocks import Q2_K
        d, ff = pool.d, pool.ff
        rows, cap = n * nu, n * nu * world
        per = n_expert_total // world
        dev = dict(device=device)
        f32, i32, u8 = dict(dtype=torch.float32, **dev), dict(dtype=torch.int32, **dev), dict(dtype=torch.uint8, **dev)
        self.n, self.nu, self.rows, self.cap, self.per, self.world = n, nu, rows, cap, per, world
        self.sel, self.w = torch.empty(n, nu, **i32), torch.empty(n, nu, **f32)
        self.counts, self.bases = torch.empty(n_expert_total, **i32), torch.empty(n_expert_total, **i32)
        self.rmap, self.smap, self.wrow = torch.empty(rows, **i32), torch.empty(rows, **i32), torch.empty(rows, **f32)
        self.group = torch.empty(_lib.lib().ill_moe_group_scratch_bytes(rows, n_expert_total), **u8)
        self.cmat = torch.empty(world, n_expert_total, **i32)
        self.cmat_host = torch.empty(world, n_expert_total, dtype=torch.int32).pin_memory()
        nseg = world * per
        self.plan_host = torch.empty(3 * nseg + 2 * per, dtype=torch.int32).pin_memory()
        self.plan = torch.empty(3 * nseg + 2 * per, **i32)
        self.p2r, self.r2p = torch.empty(cap, **i32), torch.empty(cap, **i32)
        self.xq = torch.empty(n * d, dtype=torch.int8, **dev)
        self.xs, self.xsum = torch.empty(n * d // 256, **f32), torch.empty(n * d // 16, dtype=torch.int16, **dev)
        # the rows as they are sent (a token's Q8_K form and the slot's weight in one piece) and as they arrive
        self.row_bytes = _lib.lib().ill_ep_row_bytes(d)
        self.s_rows = torch.empty(rows, self.row_bytes, **u8)
        if world > 1:
            self.r_rows = torch.empty(cap, self.row_bytes, **u8)
            self.back = torch.empty(rows, d, **f32)
        self.xd = torch.empty(cap, d // 256, **f32)
        self.xh = torch.empty(cap, d, dtype=torch.float16, **dev)
        self.xe = torch.empty(cap, d // 256, 64, dtype=torch.float16, **dev) if pool.gate_fmt == Q2_K else None
        self.g, self.u = torch.empty(cap, ff, **f32), torch.empty(cap, ff, **f32)
        self.wplace = torch.empty(cap, **f32)
        self.ms = torch.empty(cap * ff // 256, **f32)
        self.mh = torch.empty(cap, ff, dtype=torch.float16, **dev)
        self.me = torch.empty(cap, ff // 256, 64, dtype=torch.float16, **dev) if pool.down_fmt == Q2_K else None
        self.down = torch.empty(cap, d, **f32)
        self.moe = torch.empty(n, d, **f32)


def host_plan(cm, me, per):
    """The plan of rank ME from every rank's rows per expert CM [world, E] (numpy):
    send and receive counts per rank, the rows and first place of each local
    expert, and per segment (source, local expert) where its rows arrive and where
    they are placed -- place order is (expert, source, order of arrival), as
    plan_dispatch has it."""
    import numpy as np
    world = cm.shape[0]
    cm = cm.astype(np.int64)
    send_counts = cm[me].reshape(world, per).sum(1)
    rc = cm[:, me * per:(me + 1) * per]
    recv_counts = rc.sum(1)
    counts = rc.sum(0)
    bases = np.cumsum(counts) - counts
    src_off = np.cumsum(recv_counts) - recv_counts
    in_src = np.cumsum(rc, 1) - rc
    before = np.cumsum(rc, 0) - rc
    return (send_counts, recv_counts, counts, bases, (src_off[:, None] + in_src).ravel(),
            (bases[None, :] + before).ravel(), rc.ravel())


def _a2a_bytes(dst, src, recv_counts, send_counts, group):
    """All-to-all of rows as bytes (NCCL has no 16-bit integer type, and the payload is opaque to it anyway)."""
    dist.all_to_all_single(dst.view(dst.shape[0], -1).view(torch.uint8), src.view(src.shape[0], -1).view(torch.uint8),
                           output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)


def chunk_fast(ex, sc, norms, logits, n_expert_total, group=None):
    """CudaExperts.chunk with every step a kernel of the library, no allocation and
    one host synchronisation (the ranks' rows per expert, which size the
    exchanges).  Same result, bit for bit."""
    import numpy as np
    from . import _lib
    pool = ex.pool
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    me = dist.get_rank(group) if dist.is_initialized() else 0
    n, d = norms.shape
    ff, nu, per = pool.ff, ex.nu, sc.per
    rows = n * nu
    E = n_expert_total
    st = torch.cuda.current_stream().cuda_stream
    ptr = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
    call = _lib.call
    call("ill_moe_route", E, nu, ex.mode, float(ex.scale), n, ptr(logits), 0, ptr(sc.sel), ptr(sc.w), st)
    call("ill_moe_group", rows, E, nu, ptr(sc.sel), ptr(sc.w), ptr(sc.group), ptr(sc.counts), ptr(sc.bases), ptr(sc.rmap),
         ptr(sc.smap), ptr(sc.wrow), st)
    if world > 1:
        dist.all_gather_into_tensor(sc.cmat.view(-1), sc.counts, group=group)
    else:
        sc.cmat.view(-1).copy_(sc.counts)
    sc.cmat_host.copy_(sc.cmat, non_blocking=True)
    # while the counts travel: what each row carries, in sending order
    call("ill_quant_q8_k", ptr(norms), ptr(sc.xq), ptr(sc.xs), ptr(sc.xsum), n * d // 256, st)
    call("ill_ep_pack", rows, d, ptr(sc.xq), ptr(sc.xs), ptr(sc.xsum), ptr(sc.wrow), ptr(sc.rmap), ptr(sc.s_rows), st)
    torch.cuda.current_stream().synchronize()
    send_counts, recv_counts, counts, bases, seg_a, seg_p, seg_l = host_plan(sc.cmat_host.numpy(), me, per)
    nseg = world * per
    ph = sc.plan_host.numpy()
    ph[0:nseg], ph[nseg:2 * nseg], ph[2 * nseg:3 * nseg] = seg_a, seg_p, seg_l
    ph[3 * nseg:3 * nseg + per], ph[3 * nseg + per:] = counts, bases
    sc.plan.copy_(sc.plan_host, non_blocking=True)
    total = int(recv_counts.sum())
    if total > sc.cap:
        raise ValueError("more rows than the scratch holds")
    lcounts, lbases = sc.plan[3 * nseg:3 * nseg + per], sc.plan[3 * nseg + per:]
    call("ill_ep_plan_rows", nseg, ptr(sc.plan), ptr(sc.plan) + 4 * nseg, ptr(sc.plan) + 8 * nseg, ptr(sc.p2r), ptr(sc.r2p), st)
    if world > 1:
        sl, rl = [int(x) for x in send_counts], [int(x) for x in recv_counts]
        dist.all_to_all_single(sc.r_rows[:total], sc.s_rows, output_split_sizes=rl, input_split_sizes=sl, group=group)
        r_rows = sc.r_rows
    else:
        r_rows = sc.s_rows
    if total:
        # the arrived rows as the products want them, expert by expert
        call("ill_ep_unpack", total, d, ptr(r_rows), ptr(sc.p2r), ptr(sc.xh), ptr(sc.xe), ptr(sc.xd), ptr(sc.wplace), 0, st)
        call("ill_moe_mm_id2", pool.gate_fmt, d, ff, 0, pool.gate_bytes, ptr(pool.ptrs_all), ptr(lcounts), ptr(lbases),
             pool.n_expert, total, ptr(sc.xh), ptr(sc.xe), ptr(sc.xd), 0, ptr(sc.g), ptr(sc.u), ff, st)
        call("ill_swiglu_q8k_f16", total, ff, float(ex.clamp), ptr(sc.g), ptr(sc.u), ptr(sc.wplace), ptr(sc.mh), ptr(sc.me),
             ptr(sc.ms), 0, st)
        # the down rows leave in the order their inputs arrived
        call("ill_moe_mm_id", pool.down_fmt, ff, d, 2 * pool.gate_bytes, ptr(pool.ptrs_all), ptr(lcounts), ptr(lbases),
             pool.n_expert, total, ptr(sc.mh), ptr(sc.me), ptr(sc.ms), 0, ptr(sc.p2r), ptr(sc.down), d, st)
    if world > 1:
        _a2a_bytes(sc.back, sc.down[:total], sl, rl, group)
        back = sc.back
    else:
        back = sc.down
    call("ill_moe_sum", d, nu, n, ptr(back), ptr(sc.smap), 0, ptr(sc.moe), st)
    return sc.moe


class EpCapScratch:
    """Buffers of chunk_capacity: exchanges of a fixed size, CAP rows from every rank to every rank."""

    def __init__(self, pool, n, nu, n_expert_total, world, cap=None, device="cuda", peer=False, group=None):
        """PEER (several ranks only; every rank must construct it at the same point): the buffer the down rows
        come back in is a symmetric allocation that every rank maps, so that the down product stores each row
        straight into its owner's memory instead of an all-to-all after it."""
        from . import _lib
        from .blocks import Q2_K
        d, ff = pool.d, pool.ff
        rows = n * nu
        per = n_expert_total // world
        if cap is None:  # half again the even share, and room for small chunks' spread
            cap = rows if world == 1 else min(rows, (rows // world * 3 // 2 + 63) // 64 * 64 + 64)
        tot = cap * world
        dev = dict(device=device)
        f32, i32, u8 = dict(dtype=torch.float32, **dev), dict(dtype=torch.int32, **dev), dict(dtype=torch.uint8, **dev)
        self.n, self.nu, self.rows, self.cap, self.tot, self.per, self.world = n, nu, rows, cap, tot, per, world
        self.sel, self.w = torch.empty(n, nu, **i32), torch.empty(n, nu, **f32)
        self.counts, self.bases = torch.empty(n_expert_total, **i32), torch.empty(n_expert_total, **i32)
        self.rmap, self.smap, self.wrow = torch.empty(rows, **i32), torch.empty(rows, **i32), torch.empty(rows, **f32)
        self.group = torch.empty(_lib.lib().ill_moe_group_scratch_bytes(rows, n_expert_total), **u8)
        self.rc = torch.empty(world, per, **i32)
        self.lcounts, self.lbases, self.total = torch.empty(per, **i32), torch.empty(per, **i32), torch.zeros(1, **i32)
        self.overflow = torch.zeros(1, **i32)
        self.ovf_epoch, self.ovf1 = torch.zeros(1, **i32), torch.zeros(1, **i32)  # the last chunk that overflowed; a spare flag
        self.pslot, self.smap2 = torch.empty(rows, **i32), torch.empty(rows, **i32)
        self.p2r, self.r2p = torch.zeros(tot, **i32), torch.zeros(tot, **i32)
        self.xq = torch.empty(n * d, dtype=torch.int8, **dev)
        self.xs, self.xsum = torch.empty(n * d // 256, **f32), torch.empty(n * d // 16, dtype=torch.int16, **dev)
        self.row_bytes = _lib.lib().ill_ep_row_bytes(d)
        self.s_rows = torch.zeros(tot, self.row_bytes, **u8)
        self.r_rows = torch.zeros(tot, self.row_bytes, **u8) if world > 1 else self.s_rows
        self.xh = torch.empty(tot, d, dtype=torch.float16, **dev)
        self.xe = torch.empty(tot, d // 256, 64, dtype=torch.float16, **dev) if pool.gate_fmt == Q2_K else None
        self.xd, self.wplace = torch.empty(tot, d // 256, **f32), torch.empty(tot, **f32)
        self.g, self.u = torch.zeros(tot, ff, **f32), torch.zeros(tot, ff, **f32)
        self.ms = torch.empty(tot * ff // 256, **f32)
        self.mh = torch.empty(tot, ff, dtype=torch.float16, **dev)
        self.me = torch.empty(tot, ff // 256, 64, dtype=torch.float16, **dev) if pool.down_fmt == Q2_K else None
        self.down = torch.zeros(tot, d, **f32)
        self.pdst = torch.zeros(tot, **i32)
        self.peers, self.peers_rows, self.peers_rc, self.peers_flags, self.flags = None, None, None, None, None
        self.epoch, self._mapped = 0, []
        if world > 1 and peer:
            # One buffer a rank holds everything its peers store into -- the rows that come back, the slabs of packed
            # rows, the table of counts, the flags the ranks meet at -- mapped into every peer through CUDA IPC
            # (ill_ep_ipc_export / ill_ep_ipc_open): plain peer pointers, no multicast, no collective library.
            import ctypes
            grp = group if group is not None else dist.group.WORLD
            me = dist.get_rank(grp)
            up = lambda v: (v + 255) // 256 * 256  # noqa: E731
            sizes = [tot * d * 4, tot * self.row_bytes, world * per * 4, int(_lib.lib().ill_ep_flags_bytes())]
            offs = [0]
            for sz in sizes:
                offs.append(offs[-1] + up(sz))
            self.shared = torch.zeros(offs[-1], dtype=torch.uint8, device=device)
            base = self.shared.data_ptr()
            handle = ctypes.create_string_buffer(64)
            off = ctypes.c_int64(0)
            with torch.cuda.device(self.shared.device):
                _lib.call("ill_ep_ipc_export", base, handle, ctypes.byref(off))
                torch.cuda.synchronize()
                every = [None] * world
                dist.all_gather_object(every, (handle.raw, off.value), group=grp)
                bases = []
                for r, (h, o) in enumerate(every):
                    if r == me:
                        bases.append(base)
                        continue
                    out = ctypes.c_uint64(0)
                    _lib.call("ill_ep_ipc_open", h, o, ctypes.byref(out))
                    self._mapped.append((out.value, o))
                    bases.append(out.value)
            table = lambda k: torch.tensor([b + offs[k] for b in bases], dtype=torch.int64, device=device)  # noqa: E731
            view = lambda k, dt, shape: self.shared[offs[k]:offs[k] + sizes[k]].view(dt).view(shape)  # noqa: E731
            self.back, self.peers = view(0, torch.float32, (tot, d)), table(0)
            self.r_rows, self.peers_rows = view(1, torch.uint8, (tot, self.row_bytes)), table(1)
            self.rc, self.peers_rc = view(2, torch.int32, (world, per)), table(2)
            self.flags, self.peers_flags = view(3, torch.int32, (-1,)), table(3)
            torch.cuda.synchronize()
            dist.barrier(group=grp)  # every rank's buffer is zeroed and mapped before anybody stores into one
        else:
            self.back = torch.zeros(tot, d, **f32) if world > 1 else self.down
        self.moe = torch.empty(n, d, **f32)

    def close(self):
        """Unmap the peers' buffers (call on every rank, after the last chunk has completed everywhere)."""
        for ptr_, off in self._mapped:
            _lib_close(ptr_, off)
        self._mapped = []


class PeerGather:
    """An all-gather without a collective library, for the row-split head: every rank holds two buffers of WORLD
    blocks of BLOCK_BYTES (they alternate, so a rank may still read one call's result while its peers store the
    next call's) and the flags the ranks meet at, all in one allocation that the peers map through CUDA IPC.  A rank
    writes its block in place (block(i) of its own buffer), and put() stores it into every peer's buffer and holds
    the meeting (ill_peer_put): when the stream has passed it, the whole buffer is complete on this rank."""

    def __init__(self, block_bytes, world, group=None, device="cuda"):
        import ctypes
        from . import _lib
        grp = group if group is not None else dist.group.WORLD
        self.world, self.rank = world, dist.get_rank(grp) if world > 1 else 0
        self.block = (block_bytes + 255) // 256 * 256
        fb = int(_lib.lib().ill_ep_flags_bytes())
        self.buf_bytes = self.block * world
        self.shared = torch.zeros(2 * self.buf_bytes + fb, dtype=torch.uint8, device=device)
        base = self.shared.data_ptr()
        bases, self._mapped = [base], []
        if world > 1:
            handle = ctypes.create_string_buffer(64)
            off = ctypes.c_int64(0)
            with torch.cuda.device(self.shared.device):
                _lib.call("ill_ep_ipc_export", base, handle, ctypes.byref(off))
                torch.cuda.synchronize()
                every = [None] * world
                dist.all_gather_object(every, (handle.raw, off.value), group=grp)
                bases = []
                for r, (h, o) in enumerate(every):
                    if r == self.rank:
                        bases.append(base)
                        continue
                    out = ctypes.c_uint64(0)
                    _lib.call("ill_ep_ipc_open", h, o, ctypes.byref(out))
                    self._mapped.append((out.value, o))
                    bases.append(out.value)
        self.peers = [torch.tensor([b + i * self.buf_bytes for b in bases], dtype=torch.int64, device=device) for i in (0, 1)]
        self.peers_flags = torch.tensor([b + 2 * self.buf_bytes for b in bases], dtype=torch.int64, device=device)
        self.flags = self.shared[2 * self.buf_bytes:].view(torch.int32)
        self.epoch = 0
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=grp)  # every rank's buffer is zeroed and mapped before anybody stores into one

    def buffer(self, i):
        """Buffer I (0 or 1) as bytes [world, block]."""
        return self.shared[i * self.buf_bytes:(i + 1) * self.buf_bytes].view(self.world, self.block)

    def put(self, i, nbytes, wait_ns=0):
        """This rank's block of buffer I (its first NBYTES) into every peer's buffer I, and the meeting."""
        from . import _lib
        self.epoch += 1
        mine = self.shared.data_ptr() + i * self.buf_bytes + self.rank * self.block
        _lib.call("ill_peer_put", mine, nbytes, self.peers[i].data_ptr(), self.rank * self.block, self.peers_flags.data_ptr(),
                  self.flags.data_ptr(), self.world, self.rank, 2, self.epoch, wait_ns, torch.cuda.current_stream().cuda_stream)

    def mul_put(self, i, w, act, wait_ns=0):
        """One token's product of this rank's rows (W: its slice of the matrix) straight into block RANK of every
        rank's buffer I, and the meeting, in one launch (ill_mv_peers); ill_mv + put() where the kernel declines."""
        from . import _lib
        self.epoch += 1
        off = self.rank * self.block // 4
        rc = _lib.status("ill_mv_peers", w.type, w.qs.data_ptr(), w.rows, w.cols, act.xq.data_ptr(), act.xs.data_ptr(),
                         0 if act.kind == "q8" else act.xsum.data_ptr(), self.peers[i].data_ptr(), off, 0, self.peers_flags.data_ptr(),
                         self.flags.data_ptr(), self.world, self.rank, 2, self.epoch, wait_ns, torch.cuda.current_stream().cuda_stream)
        if rc == 3:
            from . import cuda_dense as D
            self.epoch -= 1
            D.cmat_mul(w, act, self.buffer(i)[self.rank][:w.rows * 4].view(torch.float32), 1)
            self.put(i, w.rows * 4, wait_ns)
        elif rc:
            raise _lib.IllatioError("ill_mv_peers", rc, _lib.lib().ill_error_string(rc).decode(), 0)

    def close(self):
        for ptr_, off in self._mapped:
            _lib_close(ptr_, off)
        self._mapped = []


def _lib_close(ptr_, off):
    from . import _lib
    _lib.status("ill_ep_ipc_close", ptr_, off)


def chunk_capacity(ex, sc, norms, logits, n_expert_total, group=None, wait_ns=0):
    """The chunk with exchanges of a fixed size (sc.cap rows from every rank to every
    rank): nothing on the host depends on the routing, so the whole chunk is
    enqueued without a synchronisation.  Returns (moe, overflow): OVERFLOW is a
    device flag, set when some slab was too small -- the result is then void and
    the caller repeats the chunk with chunk_fast.  Otherwise the same bits as
    chunk_fast.  With peer buffers (EpCapScratch(peer=True)) the chunk uses no collective at all: rows and counts
    are stored into the owners' buffers, results into the tokens' owners', and the ranks' streams meet twice at
    flags in peer memory, inside the plan and the sum kernels (WAIT_NS: how long a meeting waits, 0 = two seconds;
    a meeting that times out shows in device_status() and the chunk's result is void)."""
    from . import _lib
    pool = ex.pool
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    n, d = norms.shape
    ff, nu, per, cap, tot = pool.ff, ex.nu, sc.per, sc.cap, sc.tot
    rows = n * nu
    E = n_expert_total
    st = torch.cuda.current_stream().cuda_stream
    ptr = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
    call = _lib.call
    call("ill_moe_route", E, nu, ex.mode, float(ex.scale), n, ptr(logits), 0, ptr(sc.sel), ptr(sc.w), st)
    call("ill_moe_group", rows, E, nu, ptr(sc.sel), ptr(sc.w), ptr(sc.group), ptr(sc.counts), ptr(sc.bases), ptr(sc.rmap),
         ptr(sc.smap), ptr(sc.wrow), st)
    me = dist.get_rank(group) if dist.is_initialized() else 0
    if sc.peers is not None:
        # the dispatch without a collective, in one launch: every token is quantized once and its packed row stored
        # straight into the slabs of its slots' owners over NVLink, and the counts go into the owners' tables; then the ranks meet
        sc.epoch += 1
        if n >= (world * per + 127) // 128:
            call("ill_ep_dispatch", n, nu, d, ptr(norms), ptr(sc.wrow), ptr(sc.smap), ptr(sc.bases), ptr(sc.counts), per, world, cap,
                 me, ptr(sc.peers_rows), ptr(sc.peers_rc), ptr(sc.pslot), ptr(sc.ovf_epoch), sc.epoch, st)
        else:  # fewer tokens than it takes blocks to carry the counts: the three steps apart
            call("ill_quant_q8_k", ptr(norms), ptr(sc.xq), ptr(sc.xs), ptr(sc.xsum), n * d // 256, st)
            call("ill_ep_put_counts", world, per, me, ptr(sc.counts), ptr(sc.peers_rc), 0, st)
            sc.ovf1.zero_()
            call("ill_ep_pack_cap", rows, d, ptr(sc.xq), ptr(sc.xs), ptr(sc.xsum), ptr(sc.wrow), ptr(sc.rmap), ptr(sc.bases), per,
                 world, cap, 0, ptr(sc.pslot), ptr(sc.ovf1), ptr(sc.peers_rows), me, st)
    else:
        call("ill_quant_q8_k", ptr(norms), ptr(sc.xq), ptr(sc.xs), ptr(sc.xsum), n * d // 256, st)
        sc.overflow.zero_()
        if world > 1:  # my rows per expert, to each expert's rank: [world, per] both ways
            dist.all_to_all_single(sc.rc.view(-1), sc.counts, group=group)
        else:
            sc.rc.view(-1).copy_(sc.counts)
        call("ill_ep_pack_cap", rows, d, ptr(sc.xq), ptr(sc.xs), ptr(sc.xsum), ptr(sc.wrow), ptr(sc.rmap), ptr(sc.bases), per,
             world, cap, ptr(sc.s_rows), ptr(sc.pslot), ptr(sc.overflow), 0, me, st)
        if world > 1:
            dist.all_to_all_single(sc.r_rows, sc.s_rows, group=group)
    if sc.peers is not None:
        # the ranks meet at the start of the plan kernel (flags in peer memory, a bounded wait): the slabs and the
        # table of counts are complete once every peer has said that its stores are out
        call("ill_ep_plan_dev_sync", world, per, cap, me, ptr(sc.rc), ptr(sc.lcounts), ptr(sc.lbases), ptr(sc.p2r), ptr(sc.r2p),
             ptr(sc.pdst), ptr(sc.total), ptr(sc.ovf_epoch), ptr(sc.peers_flags), ptr(sc.flags), sc.epoch, wait_ns, st)
    else:
        call("ill_ep_plan_dev", world, per, cap, me, ptr(sc.rc), ptr(sc.lcounts), ptr(sc.lbases), ptr(sc.p2r), ptr(sc.r2p),
             ptr(sc.pdst), ptr(sc.total), ptr(sc.overflow), st)
    # the element-wise steps stop at the rows in use (sc.total, written by the plan), not at the slabs' capacity
    call("ill_ep_unpack", tot, d, ptr(sc.r_rows), ptr(sc.p2r), ptr(sc.xh), ptr(sc.xe), ptr(sc.xd), ptr(sc.wplace), ptr(sc.total),
         st)
    call("ill_moe_mm_id2", pool.gate_fmt, d, ff, 0, pool.gate_bytes, ptr(pool.ptrs_all), ptr(sc.lcounts), ptr(sc.lbases),
         pool.n_expert, tot, ptr(sc.xh), ptr(sc.xe), ptr(sc.xd), 0, ptr(sc.g), ptr(sc.u), ff, st)  # gate and up in one launch
    call("ill_swiglu_q8k_f16", tot, ff, float(ex.clamp), ptr(sc.g), ptr(sc.u), ptr(sc.wplace), ptr(sc.mh), ptr(sc.me), ptr(sc.ms),
         ptr(sc.total), st)
    if sc.peers is not None:
        # the combine fused into the down product: rows go straight to their owners over NVLink; the ranks meet
        # again at the start of the sum (every owner's rows are in before it adds them), which also looks each
        # (token, slot) row up where it came back: at its slot of the slab it left in
        call("ill_moe_mm_id_peers", pool.down_fmt, ff, d, 2 * pool.gate_bytes, ptr(pool.ptrs_all), ptr(sc.lcounts),
             ptr(sc.lbases), pool.n_expert, tot, ptr(sc.mh), ptr(sc.me), ptr(sc.ms), 0, ptr(sc.pdst), ptr(sc.peers), d, st)
        call("ill_moe_sum_sync", d, nu, n, ptr(sc.back), ptr(sc.smap), ptr(sc.pslot), 0, ptr(sc.moe), ptr(sc.peers_flags),
             ptr(sc.flags), world, me, sc.epoch, wait_ns, ptr(sc.ovf_epoch), ptr(sc.overflow), st)
        if n < (world * per + 127) // 128:
            sc.overflow.bitwise_or_(sc.ovf1)
        return sc.moe, sc.overflow
    call("ill_moe_mm_id", pool.down_fmt, ff, d, 2 * pool.gate_bytes, ptr(pool.ptrs_all), ptr(sc.lcounts), ptr(sc.lbases),
         pool.n_expert, tot, ptr(sc.mh), ptr(sc.me), ptr(sc.ms), 0, ptr(sc.p2r), ptr(sc.down), d, st)
    if world > 1:
        dist.all_to_all_single(sc.back, sc.down, group=group)
    # a (token, slot) row's result is at its slot of the slab it left in
    call("ill_gather_rows", rows, 4, ptr(sc.pslot), ptr(sc.smap), ptr(sc.smap2), st)
    call("ill_moe_sum", d, nu, n, ptr(sc.back), ptr(sc.smap2), 0, ptr(sc.moe), st)
    return sc.moe, sc.overflow


def head_rows(rows, world, rank):
    """[first, end) of the output head's rows on RANK: equal slices (the last takes the remainder)."""
    per = rows // world
    first = rank * per
    return first, (rows if rank == world - 1 else first + per)


def head_mul_allgather(w_slice, act, logits, rows, group=None):
    """The row-split output head: this rank's slice of the matrix times the
    (replicated) activations into its part of LOGITS, then one in-place all-gather.
    ROWS must divide evenly by the world size."""
    from . import cuda_dense as D
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    first, end = head_rows(rows, world, rank)
    D.cmat_mul(w_slice, act, logits[first:end], 1)
    if world > 1:
        dist.all_gather_into_tensor(logits, logits[first:end], group=group)
    return logits
