"""Expert-parallel dispatch / combine plumbing on two CPU ranks over gloo.

The products are stand-ins (a row times a number that depends on the expert),
so the test checks that every (token, slot) row reaches the rank that owns its
expert, is computed by that expert, returns to its token and is summed in slot
order -- against the same arithmetic done in one process.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from illatio_b200 import ep

E, NU, D_, N_PER = 8, 3, 5, 11


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(rank):
    g = torch.Generator().manual_seed(100 + rank)
    norms = torch.randn(N_PER, D_, generator=g)
    logits = torch.randn(N_PER, E, generator=g)
    if rank == 1:
        logits[:, 0] += 5.0  # a hot expert: uneven counts
    return norms, logits


def _route(logits):
    w, sel = torch.topk(torch.sigmoid(logits), NU, dim=1)
    return sel, w / w.sum(1, keepdim=True)


def _expected(norms, logits):
    sel, w = _route(logits)
    out = torch.zeros_like(norms)
    for s in range(NU):  # slot order
        out = out + norms * ((sel[:, s] + 1).float() * w[:, s])[:, None]
    return out


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        norms, logits = _inputs(rank)
        per = E // world

        def experts(payload, wrow, plan):
            (x,) = payload
            # the expert of each arrived row, from the plan alone
            expert_of_place = torch.repeat_interleave(torch.arange(per), plan.counts.long())
            e_global = expert_of_place[plan.recv_to_place.long()] + rank * per
            assert plan.bases.tolist() == (torch.cumsum(plan.counts, 0) - plan.counts).tolist()
            assert sorted(plan.place_to_recv.tolist()) == list(range(x.shape[0]))
            return x * ((e_global + 1).float() * wrow)[:, None]

        def summed(back, smap, n):
            rows = back[smap.long()].view(n, NU, -1)
            out = torch.zeros(n, back.shape[1])
            for s in range(NU):
                out = out + rows[:, s]
            return out

        got = ep.moe_chunk_ep(norms, logits, NU, _route, lambda x: (x,), experts, summed, E)
        # the plan the GPU drivers derive on the host from every rank's counts is the one plan_dispatch exchanges for
        sel, _ = _route(logits)
        mine = torch.bincount(sel.reshape(-1).long(), minlength=E)
        allc = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allc, mine)
        plan = ep.plan_dispatch(mine, world)
        send, recv, counts, bases, seg_a, seg_p, seg_l = ep.host_plan(torch.stack(allc).numpy(), rank, per)
        assert send.tolist() == plan.send_counts and recv.tolist() == plan.recv_counts
        assert counts.tolist() == plan.counts.tolist() and bases.tolist() == plan.bases.tolist()
        p2r = [0] * int(recv.sum())
        for a, pl, n in zip(seg_a, seg_p, seg_l):
            for i in range(int(n)):
                p2r[int(pl) + i] = int(a) + i
        assert p2r == plan.place_to_recv.tolist()
        q.put((rank, torch.allclose(got, _expected(norms, logits), atol=1e-6), None))
    except Exception as exc:  # report instead of hanging the other rank
        q.put((rank, False, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_dispatch_and_combine_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, ok, err in results:
        assert ok, "rank %d: %s" % (rank, err)


def test_plan_single_rank_is_identity_grouping():
    counts = torch.tensor([2, 0, 3, 1])
    plan = ep.plan_dispatch(counts, 1)
    assert plan.send_counts == [6] and plan.recv_counts == [6]
    assert plan.counts.tolist() == [2, 0, 3, 1] and plan.bases.tolist() == [0, 2, 2, 5]
    assert plan.place_to_recv.tolist() == list(range(6)) and plan.recv_to_place.tolist() == list(range(6))


def test_head_rows_cover_the_vocabulary():
    for world in (1, 2, 4, 8):
        spans = [ep.head_rows(151936, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 151936
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
