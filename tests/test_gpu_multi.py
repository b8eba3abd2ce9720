"""Expert parallelism on GPUs.  With one GPU: the expert-parallel driver run as a
world of one must give the single-GPU chunk driver's result bit for bit.  With
two or more GPUs (run under a multi-GPU box): two ranks over NCCL against the
one-rank result."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from illatio_b200 import cuda_ds4f as M
from illatio_b200 import cuda_ds4f_prefill as P
from illatio_b200 import ep as EP
from illatio_b200 import microbench_moe as MB

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(d=1024, ff=512, ne=8, nu=2, gate_fmt=B.IQ2_XXS, zipf=0.0)


def test_world_of_one_equals_chunk_driver(cuda_lib):
    pool = MB.make_pool(CFG, seed=3)
    g = torch.Generator(device="cuda").manual_seed(1)
    n = 300
    norms = torch.randn(n, CFG["d"], device="cuda", generator=g)
    logits = torch.randn(n, CFG["ne"], device="cuda", generator=g)
    sc = P.make_chunk_scratch(pool, n, CFG["nu"])
    want = P.dk_ffn_routed_chunk(pool, norms, logits, CFG["nu"], 10.0, sc).clone()
    ce = EP.CudaExperts(pool, CFG["nu"], 10.0)
    got = ce.chunk(norms, logits, CFG["ne"])
    assert torch.equal(got, want)
    # the path without allocations or torch index arithmetic, twice over the same scratch
    esc = EP.EpScratch(pool, n, CFG["nu"], CFG["ne"], 1)
    for _ in range(2):
        assert torch.equal(EP.chunk_fast(ce, esc, norms, logits, CFG["ne"]), want)
    # exchanges of a fixed size: the same bits without a host synchronisation; a slab too small raises the flag
    csc = EP.EpCapScratch(pool, n, CFG["nu"], CFG["ne"], 1)
    for _ in range(2):
        moe, flag = EP.chunk_capacity(ce, csc, norms, logits, CFG["ne"])
        assert torch.equal(moe, want) and flag.item() == 0
    small = EP.EpCapScratch(pool, n, CFG["nu"], CFG["ne"], 1, cap=n * CFG["nu"] - 5)
    _, flag = EP.chunk_capacity(ce, small, norms, logits, CFG["ne"])
    assert flag.item() == 1
    assert D.device_status() == 0


def test_plan_rows_and_gather_words(cuda_lib):
    from illatio_b200 import _lib
    rng = np.random.default_rng(5)
    world, per = 3, 4
    cm = rng.integers(0, 9, size=(world, world * per))
    cm[1, :] = 0  # a source with nothing to send
    send, recv, counts, bases, seg_a, seg_p, seg_l = EP.host_plan(cm, 2, per)
    total = int(recv.sum())
    tab = torch.tensor(np.concatenate([seg_a, seg_p, seg_l]).astype(np.int32), device="cuda")
    nseg = world * per
    p2r = torch.full((total,), -1, dtype=torch.int32, device="cuda")
    r2p = torch.full((total,), -1, dtype=torch.int32, device="cuda")
    _lib.call("ill_ep_plan_rows", nseg, tab.data_ptr(), tab.data_ptr() + 4 * nseg, tab.data_ptr() + 8 * nseg,
              p2r.data_ptr(), r2p.data_ptr(), None)
    p2r, r2p = p2r.cpu().numpy(), r2p.cpu().numpy()
    # arrival order: source, then expert; place order: expert, then source
    arrival = [(s, e, i) for s in range(world) for e in range(per) for i in range(cm[s, 2 * per + e])]
    place = sorted(range(total), key=lambda a: (arrival[a][1], arrival[a][0], arrival[a][2]))
    assert np.array_equal(p2r, np.array(place)) and np.array_equal(r2p[p2r], np.arange(total))
    assert np.array_equal(counts, cm[:, 2 * per:3 * per].sum(0)) and send.sum() == cm[2].sum()
    src = torch.arange(total * 3, dtype=torch.float32, device="cuda").view(total, 3)  # rows of 12 bytes
    dst = torch.empty_like(src)
    m = torch.as_tensor(p2r.astype(np.int32), device="cuda")
    _lib.call("ill_gather_rows", total, 12, src.data_ptr(), m.data_ptr(), dst.data_ptr(), None)
    assert torch.equal(dst, src[m.long()])


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from illatio_b200 import blocks as B, ep as EP, microbench_moe as MB, cuda_ds4f_prefill as P, cuda_dense as D
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
cfg = dict(d=1024, ff=512, ne=8, nu=2, gate_fmt=B.IQ2_XXS, zipf=0.0)
full = MB.make_pool(cfg, seed=3)
per = cfg["ne"] // world
mine = MB.make_pool(cfg, n_local=per, first=rank * per, seed=3)
# the local experts must be the same bytes as the full layer's
assert torch.equal(mine.pool.view(per, -1), full.pool.view(cfg["ne"], -1)[rank * per:(rank + 1) * per])
g = torch.Generator(device="cuda").manual_seed(1)
n = 300
norms = torch.randn(n, cfg["d"], device="cuda", generator=g)
logits = torch.randn(n, cfg["ne"], device="cuda", generator=g)
sc = P.make_chunk_scratch(full, n, cfg["nu"])
want = P.dk_ffn_routed_chunk(full, norms, logits, cfg["nu"], 10.0, sc)
lo, hi = rank * n // world, (rank + 1) * n // world
ce = EP.CudaExperts(mine, cfg["nu"], 10.0)
got = ce.chunk(norms[lo:hi].contiguous(), logits[lo:hi].contiguous(), cfg["ne"])
esc = EP.EpScratch(mine, hi - lo, cfg["nu"], cfg["ne"], world)
fast = [EP.chunk_fast(ce, esc, norms[lo:hi].contiguous(), logits[lo:hi].contiguous(), cfg["ne"]).clone() for _ in range(2)]
for peer in (False, True):  # the combine as an all-to-all, and fused into the down product over peer memory
    csc = EP.EpCapScratch(mine, hi - lo, cfg["nu"], cfg["ne"], world, peer=peer)
    for _ in range(3):
        moe, flag = EP.chunk_capacity(ce, csc, norms[lo:hi].contiguous(), logits[lo:hi].contiguous(), cfg["ne"])
        fast.append(moe.clone())
        assert flag.item() == 0
ok = torch.equal(got, want[lo:hi]) and all(torch.equal(f, want[lo:hi]) for f in fast) and D.device_status() == 0
# slabs too small: every token routed to rank 0's experts, so rank 0 is sent more rows than a slab holds.  The
# flags go up, the plan names only the rows that were kept, canary rows after the buffers stay untouched.
skew = logits[lo:hi].clone()
skew[:, :per] += 100.0
for peer in (False, True):
    osc = EP.EpCapScratch(mine, hi - lo, cfg["nu"], cfg["ne"], world, cap=64, peer=peer)
    bigs = {}
    for name in ("p2r", "pdst", "g", "u", "down"):
        t = getattr(osc, name)
        big = torch.full((t.shape[0] + 8,) + tuple(t.shape[1:]), -7, dtype=t.dtype, device=t.device)
        bigs[name] = big
        setattr(osc, name, big[:t.shape[0]])
    _, flag = EP.chunk_capacity(ce, osc, norms[lo:hi].contiguous(), skew, cfg["ne"])
    torch.cuda.synchronize()
    dist.barrier()
    ok = ok and flag.item() == 1 and osc.total.item() <= world * 64 and osc.lcounts.sum().item() == osc.total.item()
    ok = ok and all((b[-8:] == -7).all().item() for b in bigs.values()) and D.device_status() == 0
# the row-split head: each rank multiplies its rows, stores its logits into every peer's buffer (ill_peer_put) and
# meets them; every rank then holds the product of the whole matrix, bit for bit
rows, cols = 3000, 1024
wfull = B.synth_matrix_torch(B.Q6_K, rows, cols, seed=5)
rb = B.row_bytes(B.Q6_K, cols)
first, end = EP.head_rows(rows, world, rank)
wmine = D.CMat("slice", B.Q6_K, end - first, cols, wfull[first * rb:end * rb].clone())
act = D.quant_q8(torch.randn(cols, device="cuda", generator=g), D.make_qact(cols, "q8k"))
whole = torch.empty(rows, device="cuda")
D.cmat_mul(D.CMat("head", B.Q6_K, rows, cols, wfull), act, whole, 1)
pg = EP.PeerGather((rows - (world - 1) * (rows // world)) * 4, world)
for it in range(8):   # both buffers; the product and the stores as two launches, then fused into one
    i = it & 1
    if it < 4:
        D.cmat_mul(wmine, act, pg.buffer(i)[rank][:(end - first) * 4].view(torch.float32), 1)
        pg.put(i, (end - first) * 4)
    else:
        pg.mul_put(i, wmine, act)
    torch.cuda.synchronize()
    parts = []
    for r in range(world):
        f, e = EP.head_rows(rows, world, r)
        parts.append(pg.buffer(i)[r][:(e - f) * 4].view(torch.float32))
    ok = ok and torch.equal(torch.cat(parts), whole) and D.device_status() == 0
    dist.barrier()
    pg.buffer(i).zero_()
    torch.cuda.synchronize()
    dist.barrier()
pg.close()
if not ok:
    print("rank", rank, "max abs difference", (got - want[lo:hi]).abs().max().item(), file=sys.stderr)
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if flag.item() == 1 else 1)
"""


def test_two_ranks_equal_one_rank(cuda_lib, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
