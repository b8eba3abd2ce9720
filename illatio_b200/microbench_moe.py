"""One mixture-of-experts layer, timed: `python -m illatio_b200.microbench_moe --config c4 --tokens 4096`.

c4: hidden 4096, 256 experts of FFN 2048, top-6, IQ2_XXS gate/up, Q2_K down.
c5: hidden 5120, 288 experts of FFN 1536, top-8, Q2_K throughout, Zipf(1.1) popularity.
Prints the chunk's time, tokens/s, and the time of each step.
"""
import argparse
import json

import numpy as np
import torch

from . import blocks as B
from . import cuda_dense as D
from . import cuda_ds4f as M
from . import cuda_ds4f_prefill as P

CONFIGS = {
    "c4": dict(d=4096, ff=2048, ne=256, nu=6, gate_fmt=B.IQ2_XXS, zipf=0.0),
    "c5": dict(d=5120, ff=1536, ne=288, nu=8, gate_fmt=B.Q2_K, zipf=1.1),
}


def expert_seed(seed, tensor, expert):
    """The seed expert EXPERT's tensor (0 gate, 1 up, 2 down) is drawn from: any slice of the layer, on any rank,
    is the same bytes."""
    return seed + 1000003 * tensor + expert


def interleaved_experts(ne, world, rank):
    """Expert placement that spreads popular experts over the ranks: rank r holds experts r, r + world, ...
    (a skewed router, e.g. Zipf popularity by expert number, then loads the ranks evenly).  The products see the
    rank's experts as local numbers 0 .. ne/world - 1 in this order; the router's rows are permuted to match when
    the model is loaded (virtual_order), which costs nothing per token."""
    return list(range(rank, ne, world))


def virtual_order(ne, world):
    """Expert numbers in the order the ranks hold them with interleaved placement: entry v is the expert that is
    rank v // (ne/world)'s local expert v % (ne/world)."""
    return [e for r in range(world) for e in interleaved_experts(ne, world, r)]


def make_pool(cfg, n_local=None, first=0, seed=0, device="cuda", experts=None):
    """Experts FIRST .. FIRST+N_LOCAL-1 of the layer (or the listed EXPERTS), drawn on the device."""
    d, ff, ne = cfg["d"], cfg["ff"], cfg["ne"]
    n_local = ne if n_local is None else n_local
    if experts is None:
        experts = list(range(first, first + n_local))
    n_local = len(experts)
    gb = ff * B.row_bytes(cfg["gate_fmt"], d)
    db = d * B.row_bytes(B.Q2_K, ff)
    slot = (2 * gb + db + 255) // 256 * 256
    pool = torch.zeros(n_local * slot, dtype=torch.uint8, device=device)
    pv = pool.view(n_local, slot)
    for i, (fmt, rows, cols, off, nb) in enumerate([(cfg["gate_fmt"], ff, d, 0, gb), (cfg["gate_fmt"], ff, d, gb, gb),
                                                    (B.Q2_K, d, ff, 2 * gb, db)]):
        for e, real in enumerate(experts):  # one stream of numbers per (tensor, expert)
            m = B.synth_matrix_torch(fmt, rows, cols, seed=expert_seed(seed, i, real), device=device)
            pv[e, off:off + nb] = m
    base = pool.data_ptr()
    ptrs = torch.tensor([base + e * slot for e in range(n_local)], dtype=torch.int64, device=device)
    return M.ExpertPool(d, ff, cfg["gate_fmt"], B.Q2_K, n_local, pool, slot, gb, db, ptrs)


def router_logits(cfg, n, seed=0, device="cuda"):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    logits = torch.randn(n, cfg["ne"], device=device, generator=g)
    if cfg["zipf"]:
        # expert popularity ~ 1 / rank^1.1: added to the logits as log-popularity
        p = 1.0 / torch.arange(1, cfg["ne"] + 1, device=device, dtype=torch.float32) ** cfg["zipf"]
        logits = logits + torch.log(p / p.sum()) - torch.log(p / p.sum()).mean()
    return logits


def run(config, tokens, iters=5, device="cuda"):
    cfg = CONFIGS[config]
    pool = make_pool(cfg, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(1)
    norms = torch.randn(tokens, cfg["d"], device=device, generator=g)
    logits = router_logits(cfg, tokens, device=device)
    sc = P.make_chunk_scratch(pool, tokens, cfg["nu"], device=device)
    for _ in range(2):
        P.dk_ffn_routed_chunk(pool, norms, logits, cfg["nu"], 10.0, sc)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        P.dk_ffn_routed_chunk(pool, norms, logits, cfg["nu"], 10.0, sc)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    counts = sc.counts.cpu().numpy()
    flop = 2.0 * tokens * cfg["nu"] * 3 * cfg["d"] * cfg["ff"]
    return {"config": config, "tokens": tokens, "ms": ms, "tok_per_s": tokens / ms * 1e3, "tflops": flop / ms / 1e9,
            "rows_per_expert_max": int(counts.max()), "rows_per_expert_mean": float(counts.mean()),
            "status": D.device_status()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c4")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    print(json.dumps(run(a.config, a.tokens, a.iters)))


if __name__ == "__main__":
    main()
