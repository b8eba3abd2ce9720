"""One product shape, timed cold: `python -m illatio_b200.microbench --fmt q4_k --rows 151936 --cols 2560`.

Runs the matvec (or the fused gate/up product with --glu) over COPIES distinct
copies of the matrix in turn, so every launch reads its weights from HBM, and
prints microseconds per launch and weight GB/s.  Small enough to capture under
a profiler: --iters 1 --copies 1 launches the kernel once after one warm-up.
"""
import argparse
import json

import torch

from . import blocks as B
from . import cuda_dense as D


def run(fmt, rows, cols, n=1, glu=False, copies=2, iters=10, warmup=2, graph=False):
    dev = torch.device("cuda")
    mats = [D.CMat("w", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=5 + i, device=dev))
            for i in range(copies * (2 if glu else 1))]
    x = torch.randn(n * cols, device=dev)
    act = D.make_qact(n * cols, D.matrix_act_kind(mats[0]), device=dev)
    D.quant_q8(x, act)
    y = torch.empty(n * rows, device=dev)

    def one(i):
        if glu:
            D.glu_mul(mats[2 * (i % copies)], mats[2 * (i % copies) + 1], act, y)
        else:
            D.cmat_mul(mats[i % copies], act, y, n)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:  # the launches back to back in one CUDA graph: no host launch cost between them
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(iters):
                    one(i)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            one(i)
        e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    nbytes = mats[0].nbytes * (2 if glu else 1)
    return {"fmt": B.NAMES[fmt], "rows": rows, "cols": cols, "n": n, "glu": glu, "MB": nbytes / 1e6, "us": us,
            "GBps": nbytes / us / 1e3, "status": D.device_status()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fmt", default="q4_k")
    ap.add_argument("--rows", type=int, default=151936)
    ap.add_argument("--cols", type=int, default=2560)
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--glu", action="store_true")
    ap.add_argument("--copies", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--graph", action="store_true")
    a = ap.parse_args()
    print(json.dumps(run(B.BY_NAME[a.fmt], a.rows, a.cols, a.n, a.glu, a.copies, a.iters, a.warmup, a.graph)))


if __name__ == "__main__":
    main()
