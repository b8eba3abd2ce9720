"""The failure paths that must never become a fault or a hang: a bounded device wait that runs out,
an expert number out of range in the grouping, and exchange slabs that are too small.

None of these tests faults, traps or hangs the GPU: the wait is on a barrier nothing arrives at and
gives up after a millisecond; bad inputs are skipped and recorded in the status word; canary words
around the buffers show that nothing was written outside them.
"""
import ctypes

import numpy as np
import pytest
import torch

from illatio_b200 import _lib
from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from illatio_b200 import cuda_ds4f_prefill as P
from illatio_b200 import ep as EP
from illatio_b200 import microbench_moe as MB
from gpu_util import dev_act, to_dev

pytestmark = pytest.mark.gpu


def _status():
    v = ctypes.c_uint(0)
    rc = _lib.status("ill_device_status", ctypes.byref(v), None)
    return rc, v.value


def test_bounded_wait_runs_out_and_the_device_stays_usable(cuda_lib):
    assert torch.cuda.is_available()
    assert _status() == (0, 0)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0[0].record()
    _lib.call("ill_test_wait_timeout", 1_000_000, flag.data_ptr(), None)   # one millisecond
    t0[1].record()
    torch.cuda.synchronize()
    assert flag.item() == 1
    assert 0.5 < t0[0].elapsed_time(t0[1]) < 200.0   # it waited about the limit, not the two-second default
    rc, word = _status()
    assert rc == 5 and word == 0x800                  # ILL_ERR_DEVICE_WAIT, the test's own code
    assert _status() == (0, 0)                        # reading clears it
    # the next call works
    wb = B.synth_matrix(B.Q4_K, 64, 512, seed=1)
    w = D.upload_gmat(wb, B.Q4_K, 64, 512)
    y = torch.zeros(64, device="cuda")
    D.cmat_mul(w, dev_act(B.Q4_K, np.ones(512, np.float32)), y, 1)
    assert torch.isfinite(y).all() and y.abs().sum().item() > 0
    assert _status() == (0, 0)
    assert _lib.status("ill_test_wait_timeout", 10, 0, None) == 1   # limits outside 1 us .. 100 ms are refused


def test_meeting_of_ranks_gives_up_when_a_peer_never_arrives(cuda_lib):
    """The flag barrier of the expert-parallel path, on one GPU: a world of two whose second rank never
    signals.  The meeting waits its millisecond, records the barrier's code and returns; once the missing
    flag is there the same meeting passes."""
    nbytes = _lib.lib().ill_ep_flags_bytes()
    mine = torch.zeros(nbytes // 4, dtype=torch.int32, device="cuda")
    other = torch.zeros(nbytes // 4, dtype=torch.int32, device="cuda")     # stands for the absent rank's flags
    peers = torch.tensor([mine.data_ptr(), other.data_ptr()], dtype=torch.int64, device="cuda")
    slot, epoch = 2, 1
    _lib.call("ill_ep_barrier", peers.data_ptr(), mine.data_ptr(), 2, 0, slot, epoch, 1_000_000, None)
    torch.cuda.synchronize()
    assert _status() == (5, 0x700)
    assert mine[slot * 64 + 0].item() == epoch and other[slot * 64 + 0].item() == epoch   # this rank did signal both
    mine[slot * 64 + 1] = epoch                                                           # the peer's flag, late
    _lib.call("ill_ep_barrier", peers.data_ptr(), mine.data_ptr(), 2, 0, slot, epoch, 1_000_000, None)
    torch.cuda.synchronize()
    assert _status() == (0, 0)
    # the sum that follows a failed meeting adds nothing and leaves its output alone
    d, nu, n = 256, 2, 3
    down = torch.ones(n * nu, d, device="cuda")
    moe = torch.full((n, d), -7.0, device="cuda")
    _lib.call("ill_moe_sum_sync", d, nu, n, down.data_ptr(), 0, 0, 0, moe.data_ptr(), peers.data_ptr(), mine.data_ptr(), 2, 0,
              epoch + 1, 1_000_000, 0, 0, None)
    torch.cuda.synchronize()
    assert _status() == (5, 0x700) and (moe == -7.0).all()
    assert _lib.status("ill_ep_barrier", peers.data_ptr(), mine.data_ptr(), 65, 0, 0, 1, 0, None) == 1   # more ranks than flags


def test_group_skips_and_flags_an_expert_out_of_range(cuda_lib):
    ne, nu, n = 8, 2, 700
    rng = np.random.default_rng(1)
    sel_h = np.stack([rng.choice(ne, size=nu, replace=False) for _ in range(n)]).astype(np.int32)
    bad = sel_h.copy()
    bad[123, 1] = ne + 5
    bad[699, 0] = -1
    rows = n * nu
    i32 = dict(dtype=torch.int32, device="cuda")
    w = torch.rand(rows, device="cuda")
    scratch = torch.empty(_lib.lib().ill_moe_group_scratch_bytes(rows, ne), dtype=torch.uint8, device="cuda")
    out = {}
    for name, s in (("good", sel_h), ("bad", bad)):
        counts, bases = torch.full((ne + 4,), -7, **i32), torch.full((ne + 4,), -7, **i32)
        rmap, smap = torch.full((rows + 4,), -7, **i32), torch.full((rows + 4,), -7, **i32)
        wrow = torch.full((rows + 4,), -7.0, device="cuda")
        _lib.call("ill_moe_group", rows, ne, nu, to_dev(s).data_ptr(), w.data_ptr(), scratch.data_ptr(), counts.data_ptr(),
                  bases.data_ptr(), rmap.data_ptr(), smap.data_ptr(), wrow.data_ptr(), None)
        torch.cuda.synchronize()
        out[name] = [t.cpu().numpy() for t in (counts, bases, rmap, smap, wrow)]
        for t, k in zip(out[name], (ne, ne, rows, rows, rows)):
            assert (t[k:] == -7).all(), "wrote past a buffer"
        rc, word = _status()
        assert (rc, word) == ((0, 0) if name == "good" else (5, 0x600))
    # the two bad rows are in no expert's count; every other row keeps a place inside the table
    assert out["bad"][0][:ne].sum() == rows - 2
    assert (out["bad"][3][:rows] < rows).all() and (out["bad"][3][:rows] >= 0).all()


def test_slab_overflow_stays_inside_the_buffers(cuda_lib):
    """A slab five rows short (a world of one): the flag goes up, the plan names only the rows that were
    kept, and nothing is written past p2r / pdst / g / u / down."""
    cfg = dict(d=1024, ff=512, ne=8, nu=2, gate_fmt=B.IQ2_XXS, zipf=0.0)
    pool = MB.make_pool(cfg, seed=3)
    g = torch.Generator(device="cuda").manual_seed(1)
    n = 300
    norms = torch.randn(n, cfg["d"], device="cuda", generator=g)
    logits = torch.randn(n, cfg["ne"], device="cuda", generator=g)
    ce = EP.CudaExperts(pool, cfg["nu"], 10.0)
    cap = n * cfg["nu"] - 5
    small = EP.EpCapScratch(pool, n, cfg["nu"], cfg["ne"], 1, cap=cap)
    # the buffers the plan and the products index by place, re-made with canary rows after them
    PAD = 8
    def padded(t, fill):
        big = torch.full((t.shape[0] + PAD,) + tuple(t.shape[1:]), fill, dtype=t.dtype, device=t.device)
        return big, big[:t.shape[0]]
    bigs = {}
    for name, fill in (("p2r", -7), ("pdst", -7), ("g", -7.0), ("u", -7.0), ("down", -7.0)):
        bigs[name], view = padded(getattr(small, name), fill)
        setattr(small, name, view)
    small.back = small.down
    _, flag = EP.chunk_capacity(ce, small, norms, logits, cfg["ne"])
    torch.cuda.synchronize()
    assert flag.item() == 1
    assert small.total.item() == cap and small.lcounts.sum().item() == cap
    for name, big in bigs.items():
        assert (big[-PAD:] == -7).all(), "%s was written past its end" % name
    assert _status() == (0, 0)
    # with room for every row the same scratch shape gives the chunk driver's result
    sc = P.make_chunk_scratch(pool, n, cfg["nu"])
    want = P.dk_ffn_routed_chunk(pool, norms, logits, cfg["nu"], 10.0, sc).clone()
    full = EP.EpCapScratch(pool, n, cfg["nu"], cfg["ne"], 1)
    moe, flag = EP.chunk_capacity(ce, full, norms, logits, cfg["ne"])
    assert flag.item() == 0 and torch.equal(moe, want)
