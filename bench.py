#!/usr/bin/env python
"""bench.py -- quantized matvec weight GB/s on the Qwen3-4B Q4_K_M decode shapes.

One "step" is every in-scope kernel of one decoded token of the Qwen3-4B
architecture (36 layers; Q/K/O/gate/up in Q4_K, V/down in Q6_K, a Q6_K output
head of 151936 rows): activation quantization and the dequant-fused matrix x
vector products, in the order the reference's CUDA-FORWARD-N issues them
(src/cuda-dense.lisp:380-432), on seeded synthetic blocks.  Attention, RoPE and
normalisation are not part of the path and are not run.

  value     weight bytes of a step / device time of a step, weights resident
            in HBM, every step reading all 2.6 GB cold (far larger than L2)
  e2e       the same through host buffers: the token's activations go up from
            pinned memory and the logits come back, inside the timed region
  roofline  the Q4_K gate/up product (the kernel most of the bytes go through)
  formats   each of the five formats on one large matrix, cold

Usage: python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

Q8_0, Q4_K, Q6_K, Q2_K, IQ2_XXS = range(5)
HIDDEN, QDIM, KVDIM, FFN, VOCAB, LAYERS = 2560, 4096, 1024, 9728, 151936, 36
WORKLOAD = "qwen3-4b Q4_K_M single-token decode (configs[1]): 36 layers + 151936-row Q6_K head"
# (name, fmt, rows, cols)
LAYER_MATS = [("q", Q4_K, QDIM, HIDDEN), ("k", Q4_K, KVDIM, HIDDEN), ("v", Q6_K, KVDIM, HIDDEN),
              ("o", Q4_K, HIDDEN, QDIM), ("gate", Q4_K, FFN, HIDDEN), ("up", Q4_K, FFN, HIDDEN),
              ("down", Q6_K, HIDDEN, FFN)]
HEAD = ("head", Q6_K, VOCAB, HIDDEN)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    """Measured dense bf16 / fp16 TFLOP/s of this pool's B200s (the burst figure), else the fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes():
    from illatio_b200.blocks import matrix_bytes
    per_layer = sum(matrix_bytes(f, r, c) for _, f, r, c in LAYER_MATS)
    return per_layer * LAYERS + matrix_bytes(HEAD[1], HEAD[2], HEAD[3]), per_layer


# ------------------------------------------------------------------ reference arm

def run_reference(args, rank, world):
    """The reference's CPU path (its C restatement, oracle/) on the host cores:
    a step is one layer's seven products plus their activation quantization."""
    if rank != 0:
        return
    from oracle import oracle as O
    from illatio_b200 import blocks as B
    O.build()
    cores = len(os.sched_getaffinity(0))
    mats = [(n, f, r, c, B.synth_matrix(f, r, c, seed=10 + i)) for i, (n, f, r, c) in enumerate(LAYER_MATS)]
    rng = np.random.default_rng(0)
    xs = {c: rng.standard_normal(c).astype(np.float32) for c in (HIDDEN, QDIM, FFN)}
    nbytes = sum(m[4].size for m in mats)

    def step():
        for _, f, r, c, w in mats:
            act = O.quantize_act(f, xs[c])
            O.matvec(f, w, r, c, act, threads=cores)

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = nbytes / dt / 1e9
    sample = "one layer of the workload (7 products, %.1f MB of blocks) per step, portable-order C port, rows split over %d threads" % (nbytes / 1e6, cores)
    print(json.dumps({
        "impl": "reference", "metric": "quant matvec weight GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 dots, fp32 accumulate",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ our arm

def cpu_baseline_sample(seconds=10.0):
    """The oracle timed on this box's host cores on one layer of the workload."""
    from oracle import oracle as O
    from illatio_b200 import blocks as B
    O.build()
    cores = len(os.sched_getaffinity(0))
    mats = [(f, r, c, B.synth_matrix(f, r, c, seed=10 + i)) for i, (_, f, r, c) in enumerate(LAYER_MATS)]
    rng = np.random.default_rng(0)
    xs = {c: rng.standard_normal(c).astype(np.float32) for c in (HIDDEN, QDIM, FFN)}
    nbytes = sum(m[3].size for m in mats)

    def step():
        for f, r, c, w in mats:
            O.matvec(f, w, r, c, O.quantize_act(f, xs[c]), threads=cores)

    step()
    t0 = time.perf_counter()
    reps = 0
    while True:
        step()
        reps += 1
        if time.perf_counter() - t0 > seconds or reps >= 100000:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "one layer of the workload (%.1f MB of blocks), %d repetitions, %.1f s" % (nbytes / 1e6, reps, dt * reps)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-formats", action="store_true", help="skip the per-format sweep")
    ap.add_argument("--no-moe", action="store_true", help="skip the mixture-of-experts layer")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from illatio_b200 import _lib
    from illatio_b200 import blocks as B
    from illatio_b200 import cuda_dense as D

    _lib.lib()  # fails loudly if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)

    # ---- the model's matrices (random-init, seeded), resident in HBM
    layers = []
    for li in range(LAYERS):
        layers.append({n: D.CMat(n, f, r, c, B.synth_matrix_torch(f, r, c, seed=1000 * li + i + 7919 * rank, device=dev))
                       for i, (n, f, r, c) in enumerate(LAYER_MATS)})
    head = D.CMat("head", HEAD[1], HEAD[2], HEAD[3], B.synth_matrix_torch(HEAD[1], HEAD[2], HEAD[3], seed=99 + rank, device=dev))
    total_bytes, per_layer_bytes = weight_bytes()

    g = torch.Generator(device=dev)
    g.manual_seed(1 + rank)
    x = torch.randn(HIDDEN, device=dev, generator=g)             # the token's hidden state
    att = torch.randn(QDIM, device=dev, generator=g)              # stands for the attention output
    act_d = D.make_qact(HIDDEN, "q8k", device=dev)
    act_q = D.make_qact(QDIM, "q8k", device=dev)
    act_f = D.make_qact(FFN, "q8k", device=dev)
    q = torch.empty(QDIM, device=dev)
    k = torch.empty(KVDIM, device=dev)
    v = torch.empty(KVDIM, device=dev)
    fa = torch.empty(FFN, device=dev)
    h = torch.zeros(HIDDEN, device=dev)
    logits = torch.empty(VOCAB, device=dev)
    x_host = torch.randn(HIDDEN).pin_memory()
    logits_host = torch.empty(VOCAB).pin_memory()
    launches_per_step = [0]

    # The reference fuses the quantization of the attention / FFN inputs into kernels that are
    # not on this path (rmsnorm_q8, attn_merge: src/cuda-dense.lisp:264,356); here the token's
    # hidden state is quantized once per step and stands for each layer's normed input, and the
    # attention output is quantized before the timed region.  The quantization after the gated
    # product is the reference's own stand-alone quant_q8 launch (src/cuda-dense.lisp:417).
    D.quant_q8(att, act_q)

    def token_step():
        n = 0
        D.quant_q8(x, act_d); n += 1
        for L in layers:
            D.qkv_mul(L["q"], L["k"], L["v"], act_d, q, k, v); n += 2
            D.cmat_mul(L["o"], act_q, h, 1, acc=True); n += 1
            D.glu_mul(L["gate"], L["up"], act_d, fa); n += 1
            D.quant_q8(fa, act_f); n += 1
            D.cmat_mul(L["down"], act_f, h, 1, acc=True); n += 1
        D.cmat_mul(head, act_d, logits, 1); n += 1
        launches_per_step[0] = n

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # eager warm-up, then one CUDA graph of a step (removes host launch cost from the device number)
    for _ in range(args.warmup):
        h.zero_()
        token_step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            token_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for _ in range(args.warmup):
        graph.replay()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-timed region: K steps, weights resident
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps

    # ---- end to end: activations up from pinned memory, logits back, every step
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        x.copy_(x_host, non_blocking=True)
        graph.replay()
        logits_host.copy_(logits, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps

    # ---- the dominant kernel alone: the Q4_K gate/up product of every layer, back to back in one
    # CUDA graph (36 launches, each on its own layer's matrices: cold), timed with events
    glu_bytes = 2 * B.matrix_bytes(Q4_K, FFN, HIDDEN) + HIDDEN * (1 + 4 / 256 + 2 / 16) + 4 * FFN
    D.quant_q8(x, act_d)
    torch.cuda.synchronize()
    ggraph = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(ggraph, stream=side):
            for L in layers:
                D.glu_mul(L["gate"], L["up"], act_d, fa)
    torch.cuda.synchronize()
    for _ in range(3):
        ggraph.replay()
    torch.cuda.synchronize()
    reps = 10
    e0.record()
    for _ in range(reps):
        ggraph.replay()
    e1.record()
    torch.cuda.synchronize()
    glu_us = e0.elapsed_time(e1) * 1e3 / (reps * LAYERS)

    # ---- each format on one large matrix, cold (two copies, alternating, each larger than L2)
    formats = {}
    if not args.no_formats:
        for fmt, rows, cols in ((Q8_0, VOCAB, 896), (Q4_K, VOCAB, 2560), (Q6_K, VOCAB, 5120), (Q2_K, VOCAB, 5120),
                                (IQ2_XXS, VOCAB, 4096)):
            ms_ = [D.CMat("sweep", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=5 + i, device=dev))
                   for i in range(2)]
            xx = torch.randn(cols, device=dev, generator=g)
            act = D.make_qact(cols, D.matrix_act_kind(ms_[0]), device=dev)
            D.quant_q8(xx, act)
            y = torch.empty(rows, device=dev)
            for i in range(4):
                D.cmat_mul(ms_[i & 1], act, y, 1)
            torch.cuda.synchronize()
            e0.record()
            for i in range(10):
                D.cmat_mul(ms_[i & 1], act, y, 1)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 10
            nb = ms_[0].nbytes
            formats[B.NAMES[fmt]] = {"rows": rows, "cols": cols, "MB": nb / 1e6, "us": us, "GBps": nb / us / 1e3}
            del ms_
            torch.cuda.empty_cache()

    # free the sweep's matrices before the mixture-of-experts layer is built
    torch.cuda.empty_cache()

    # ---- the sharded paths: (1) the row-split output head with an all-gather of the logits,
    # (2) one DeepSeek-V4-Flash-shaped MoE layer (configs[3]) over a 4096-token chunk, experts placed
    # expert-parallel (256 / N per rank), tokens split by position (strong scaling)
    from illatio_b200 import ep as EP
    from illatio_b200 import microbench_moe as MB
    first_row, end_row = EP.head_rows(VOCAB, world, rank)
    rb = B.row_bytes(HEAD[1], HIDDEN)
    head_slice = D.CMat("head_slice", HEAD[1], end_row - first_row, HIDDEN, head.qs[first_row * rb:end_row * rb])
    for _ in range(3):
        EP.head_mul_allgather(head_slice, act_d, logits, VOCAB)
    barrier()
    e0.record()
    for _ in range(20):
        EP.head_mul_allgather(head_slice, act_d, logits, VOCAB)
    e1.record()
    barrier()
    head_us = e0.elapsed_time(e1) * 1e3 / 20

    moe = None
    if not args.no_moe:
        cfg = MB.CONFIGS["c4"]
        n_tok = 4096
        per = cfg["ne"] // world
        pool = MB.make_pool(cfg, n_local=per, first=rank * per, seed=7, device=dev)
        gm = torch.Generator(device=dev)
        gm.manual_seed(11)  # the same chunk on every rank; each takes its slice of the tokens
        norms_all = torch.randn(n_tok, cfg["d"], device=dev, generator=gm)
        logits_all = MB.router_logits(cfg, n_tok, seed=12, device=dev)
        lo, hi = rank * n_tok // world, (rank + 1) * n_tok // world
        norms_l, logits_l = norms_all[lo:hi].contiguous(), logits_all[lo:hi].contiguous()
        del norms_all, logits_all
        ce = EP.CudaExperts(pool, cfg["nu"], 10.0)
        # A stream of independent chunks.  The exchanges have a fixed size (half again the even share of rows
        # from every rank to every rank), so nothing on the host waits for the routing; a slab that turned out
        # too small would raise a flag, checked after the timed region.  (ILL_EP_LANES=2 alternates the chunks
        # between two CUDA streams; measured, it gains nothing: the persistent product kernel holds every SM, so
        # the other stream's exchange kernels do not run beside it.)
        nlanes = int(os.environ.get("ILL_EP_LANES", "1"))
        exact = os.environ.get("ILL_EP_MODE", "capacity") == "exact"
        peer_combine = world > 1 and not exact and os.environ.get("ILL_EP_COMBINE", "peer") == "peer"
        mk = (lambda: EP.EpScratch(pool, hi - lo, cfg["nu"], cfg["ne"], world, device=dev)) if exact else \
             (lambda: EP.EpCapScratch(pool, hi - lo, cfg["nu"], cfg["ne"], world, device=dev, peer=peer_combine))
        try:
            lanes = [(torch.cuda.Stream(device=dev), mk()) for _ in range(nlanes)]
            made = 1
        except Exception as exc:  # no peer mapping on this box: the same exchanges over NCCL
            print("rank %d: symmetric memory unavailable (%s)" % (rank, exc), file=sys.stderr)
            made = 0
        if peer_combine:  # every rank takes the same path
            agree = torch.tensor([made], device=dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            if agree.item() == 0:
                peer_combine = False
                lanes = [(torch.cuda.Stream(device=dev), mk()) for _ in range(nlanes)]
        flags = []

        def run_chunks(k):
            main = torch.cuda.current_stream()
            for s_, _ in lanes:
                s_.wait_stream(main)
            for i in range(k):
                s_, esc = lanes[i % nlanes]
                with torch.cuda.stream(s_):
                    if exact:
                        EP.chunk_fast(ce, esc, norms_l, logits_l, cfg["ne"])
                    else:
                        flags.append(EP.chunk_capacity(ce, esc, norms_l, logits_l, cfg["ne"])[1].clone())
            for s_, _ in lanes:
                main.wait_stream(s_)

        run_chunks(4)
        barrier()
        reps = 12
        e0.record()
        run_chunks(reps)
        e1.record()
        barrier()
        moe_ms = e0.elapsed_time(e1) / reps
        mt = torch.tensor([moe_ms, head_us], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(mt, op=dist.ReduceOp.MAX)
        moe_ms, head_us = mt.tolist()
        flop = 2.0 * n_tok * cfg["nu"] * 3 * cfg["d"] * cfg["ff"]
        moe = {"workload": "configs[3]: hidden 4096, 256 experts of FFN 2048, top-6, IQ2_XXS gate/up, Q2_K down; one 4096-token chunk through the routed experts",
               "n_gpus": world, "experts_per_gpu": per, "tokens": n_tok, "ms_per_chunk": moe_ms, "chunks_in_flight": nlanes,
               "exchange_sizes": "exact (one host synchronisation a chunk)" if exact else "fixed slabs, no host synchronisation",
               "slab_overflows": int(sum(int(f.item()) for f in flags)),
               "combine": ("fused into the down product: stores into the owners' memory over NVLink" if peer_combine
                           else "NCCL all-to-all of fp32 rows" if world > 1 else "none (one GPU)"),
               "tok_per_s": n_tok / moe_ms * 1e3, "tflops": flop / moe_ms / 1e9, "scaling": "strong",
               "roofline": {"bound": "tensor", "achieved": flop / moe_ms / 1e9 / world, "peak": tensor_peak()[0],
                            "peak_source": tensor_peak()[1], "unit": "TFLOP/s per GPU, whole chunk (products and all the steps around them)",
                            "frac": flop / moe_ms / 1e9 / world / tensor_peak()[0]},
               "exchange": ("none (one GPU)" if world == 1 else
                            "peer stores over NVLink: packed Q8_K rows out (1.14 B/value), fp32 rows back from the down product's epilogue"
                            if peer_combine else "NCCL all-to-all of packed Q8_K rows out (1.14 B/value), fp32 rows back")}
        del pool, ce, lanes

    clocks = sampler.stop() if rank == 0 else None  # sampled over every timed region above
    status = D.device_status()
    tmax = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms, e2e_ms = tmax.tolist()
    if rank == 0:
        peak, which = peaks()
        value = world * total_bytes / (ms * 1e-3) / 1e9
        e2e = world * total_bytes / (e2e_ms * 1e-3) / 1e9
        achieved = glu_bytes / (glu_us * 1e-6) / 1e9
        for f in formats.values():
            f["frac_of_%s_hbm" % which] = f["GBps"] / peak
        out = {
            "metric": "quant matvec weight GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> int32 dots, fp32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "weight_bytes_per_step": total_bytes,
                       "l2": "every step reads 2.6 GB of distinct weights, far larger than the 126 MB L2",
                       "replicas": "each rank decodes its own token on its own copy (the decode products do not shard)",
                       "launch": "one CUDA graph of the step's %d kernel launches" % launches_per_step[0]},
            "frac_of_%s_hbm" % which: value / world / peak,
            "e2e": {"value": e2e, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": HIDDEN * 4,
                    "d2h_bytes_per_step": VOCAB * 4},
            "gpu_launches": launches_per_step[0] * args.steps,
            "roofline": {"bound": "hbm", "kernel": "mvw_kernel<Q4_K, gated> (gate/up 2 x 9728x2560)",
                         "achieved": achieved, "peak": peak, "peak_source": which + " (MEASURED_PEAKS.json hbm_gbs)" if which == "measured" else which,
                         "unit": "GB/s", "frac": achieved / peak,
                         # dram__bytes_read + write of one launch, from the ncu capture summarised under profiles/
                         "traffic": 28059904.0,
                         "us_per_launch": glu_us, "algorithmic_bytes_per_launch": glu_bytes},
            "clocks": clocks, "formats": formats, "device_status": status,
            "head_rowsplit": {"rows_per_gpu": end_row - first_row, "us_per_token": head_us,
                              "GBps": B.matrix_bytes(HEAD[1], VOCAB, HIDDEN) / head_us / 1e3,
                              "collective": "in-place all-gather of fp32 logits" if world > 1 else "none (one GPU)"},
            "moe_prefill": moe,
        }
        if not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
