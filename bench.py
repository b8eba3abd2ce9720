#!/usr/bin/env python
"""bench.py -- quantized matvec weight GB/s on the Qwen3-4B Q4_K_M decode shapes, and the rest of the path's
configurations beside it.

One "step" is every in-scope kernel of one decoded token of the Qwen3-4B architecture (36 layers; Q/K/O/gate/up
in Q4_K, V/down in Q6_K, a Q6_K output head of 151936 rows): activation quantization and the dequant-fused matrix
x vector products, in the order the reference's CUDA-FORWARD-N issues them (src/cuda-dense.lisp:380-432), on
seeded synthetic blocks.  Attention, RoPE and normalisation are not part of the path and are not run.

  value / ms_per_step  weight bytes of a step / device time of a step, weights resident in HBM, every step
                       reading all 2.6 GB cold (far larger than L2); one replica per GPU (the decode products do
                       not shard), so across N this key is weak scaling of independent copies
  e2e                  the same through host buffers: the token's activations go up from pinned memory and the
                       logits come back, inside the timed region
  roofline             the Q4_K gate/up product (the kernel most of the bytes go through)
  formats              each of the five formats on one 151936-row matrix, cold
  configs              the other configurations: c1 (Q8_0 0.5B token), c2_chain (the 4B token with RMSNorm and
                       every quantization fused, product by product and as one launch), c2_prefill_512, c3 (Q6_K
                       27B-scale matrices at batch 1 / 4 / 16), c4_decode (one token through an MoE layer)
  sharded              THE CURVES THAT SCALE WITH N: moe_prefill (c4, one 4096-token chunk, experts placed
                       expert-parallel), c5 (288 experts, Zipf: 64-sequence decode and an 8192-token prefill),
                       head_rowsplit (the 151936 x 5120 Q6_K head split by rows) -- each with `vs_1gpu` (the same
                       work timed on rank 0 alone in the same run) and `parity` (checked against the CPU oracle or
                       the one-GPU product, outside the timed regions)

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
C1 = dict(hidden=896, qdim=896, kvdim=128, ffn=4864, vocab=151936, layers=24)
EPS = 1e-6


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


def profiled_traffic(name):
    """dram bytes read + written per launch, from the JSON beside the ncu summary under profiles/ (None if absent)."""
    p = os.path.join(ROOT, "profiles", name)
    if not os.path.exists(p):
        return None
    d = json.load(open(p))
    return float(d["dram_bytes_read"]) + float(d["dram_bytes_written"])


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


# ------------------------------------------------------------------ the CPU legs (the oracle, timed)

def cpu_layer_gbs(fast, seconds, cores):
    """One layer of the workload (its seven products and their activation quantization) on the host cores:
    FAST = the AVX2 row dots on pinned threads, else the portable loops.  (GB/s, repetitions, seconds, bytes)."""
    from oracle import oracle as O
    from illatio_b200 import blocks as B
    O.build()
    mats = [(f, r, c, B.synth_matrix(f, r, c, seed=10 + i)) for i, (_, f, r, c) in enumerate(LAYER_MATS)]
    rng = np.random.default_rng(0)
    xs = {c: rng.standard_normal(c).astype(np.float32) for c in (HIDDEN, QDIM, FFN)}
    nbytes = sum(m[3].size for m in mats)
    prev = O.set_fast(fast)
    try:
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
    finally:
        O.set_fast(prev)
    return nbytes / dt / 1e9, reps, dt * reps, nbytes


def cpu_moe_layer(seconds, cores):
    """One token through the c4 layer's routed experts (6 of them) on the host cores, AVX2 on pinned threads:
    the reference's own CPU fast path for these formats (src/avx2.lisp:77-150; "80 us an expert across the cores")."""
    from oracle import oracle as O
    from illatio_b200 import blocks as B
    d, ff, nu = 4096, 2048, 6
    gate, up = (B.synth_matrix(B.IQ2_XXS, nu * ff, d, seed=s) for s in (41, 42))
    down = B.synth_matrix(B.Q2_K, nu * d, ff, seed=43)
    x = np.random.default_rng(1).standard_normal(d).astype(np.float32)
    sel, w = np.arange(nu, dtype=np.int32), np.full(nu, 1.0 / nu, np.float32)
    nbytes = gate.size + up.size + down.size
    out = {}
    for name, fast in (("avx2_pinned", True), ("portable", False)):
        if fast and not O.simd_available():
            continue
        prev = O.set_fast(fast)
        try:
            O.moe_routed(d, ff, B.IQ2_XXS, B.Q2_K, gate, up, down, x, sel, w, 10.0, threads=cores)
            t0, reps = time.perf_counter(), 0
            while time.perf_counter() - t0 < seconds:
                O.moe_routed(d, ff, B.IQ2_XXS, B.Q2_K, gate, up, down, x, sel, w, 10.0, threads=cores)
                reps += 1
            dt = (time.perf_counter() - t0) / reps
        finally:
            O.set_fast(prev)
        out[name] = {"us_per_token_layer": dt * 1e6, "GBps": nbytes / dt / 1e9, "us_per_expert": dt * 1e6 / nu}
    out["sample"] = "6 experts (IQ2_XXS gate / up, Q2_K down, %.1f MB) of one token, %d threads" % (nbytes / 1e6, cores)
    return out


def run_reference(args, rank, world):
    """The reference's CPU path (its C restatement, oracle/) on the host cores: a step is one layer's seven
    products plus their activation quantization.  The line's value is the fast form -- AVX2 integer dots on a
    pool of pinned threads, how the reference runs its own CPU share -- and the portable loops are timed beside it."""
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    cores = len(os.sched_getaffinity(0))
    fast = O.simd_available()
    budget = max(2.0, min(20.0, 0.5 * args.steps))
    gbs, reps, secs, nbytes = cpu_layer_gbs(fast, budget, cores)
    port_gbs = cpu_layer_gbs(False, 3.0, cores)[0] if fast else gbs
    sample = ("one layer of the workload (7 products, %.1f MB of blocks) per step, %s, rows split over %d threads"
              % (nbytes / 1e6, "AVX2 row dots on pinned threads" if fast else "portable-order C port", cores))
    print(json.dumps({
        "impl": "reference", "metric": "quant matvec weight GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": nbytes / gbs / 1e6, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 dots, fp32 accumulate",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample, "repetitions": reps, "seconds": secs},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                         "portable_scalar_GBps": port_gbs},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ helpers of the GPU arm

def graph_of(fn, torch):
    """FN captured in a CUDA graph (after one eager run)."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return g


def time_us(fn, reps, torch, warm=3):
    """Microseconds per call of FN, CUDA events on the current stream."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def build_chain_model(D, B, torch, dev, dims, layers, fmt_main, fmt_alt, seed):
    """The in-scope products of a dense transformer with the attention stood in for by its query vector: per
    layer q / k / v <- rmsnorm(h); h += o(q); fa <- glu(rmsnorm(h)); h += down(fa); then the head on rmsnorm(h)."""
    hidden, qdim, kvdim, ffn, vocab = dims
    g = torch.Generator(device=dev)
    g.manual_seed(seed)

    def mat(fmt, rows, cols, s):
        return D.CMat("m", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=s, device=dev))
    m = {"dims": dims, "layers": []}
    for li in range(layers):
        s = 100 * li + seed
        m["layers"].append(dict(q=mat(fmt_main, qdim, hidden, s + 1), k=mat(fmt_main, kvdim, hidden, s + 2),
                                v=mat(fmt_alt, kvdim, hidden, s + 3), o=mat(fmt_main, hidden, qdim, s + 4),
                                gate=mat(fmt_main, ffn, hidden, s + 5), up=mat(fmt_main, ffn, hidden, s + 6),
                                down=mat(fmt_alt, hidden, ffn, s + 7),
                                nw1=torch.rand(hidden, device=dev, generator=g) + 0.5,
                                nw2=torch.rand(hidden, device=dev, generator=g) + 0.5))
    m["head"] = mat(fmt_alt, vocab, hidden, seed + 99)
    m["nwf"] = torch.rand(hidden, device=dev, generator=g) + 0.5
    f = dict(dtype=torch.float32, device=dev)
    m["h"], m["q"], m["k"], m["v"] = torch.empty(hidden, **f), torch.empty(qdim, **f), torch.empty(kvdim, **f), torch.empty(kvdim, **f)
    m["fa"], m["logits"] = torch.empty(ffn, **f), torch.empty(vocab, **f)
    m["x0"] = torch.randn(hidden, device=dev, generator=g)
    m["bytes"] = sum(w.nbytes for L in m["layers"] for w in L.values() if isinstance(w, D.CMat)) + m["head"].nbytes
    return m


def chain_ops(D, m):
    ops = []
    for L in m["layers"]:
        ops += [D.decode_op(L["q"], m["h"], m["q"], norm_w=L["nw1"], eps=EPS, after=True),
                D.decode_op(L["k"], m["h"], m["k"], norm_w=L["nw1"], eps=EPS, after=False),
                D.decode_op(L["v"], m["h"], m["v"], norm_w=L["nw1"], eps=EPS, after=False),
                D.decode_op(L["o"], m["q"], m["h"], acc=True, after=True),
                D.decode_op(L["gate"], m["h"], m["fa"], w2=L["up"], norm_w=L["nw2"], eps=EPS, after=True),
                D.decode_op(L["down"], m["fa"], m["h"], acc=True, after=True)]
    ops.append(D.decode_op(m["head"], m["h"], m["logits"], norm_w=m["nwf"], eps=EPS, after=True))
    return ops


def chain_per_product(D, m, acts):
    """The same chain, a launch per product and per quantization (RMSNorm fused with the quantizer)."""
    hidden, qdim, kvdim, ffn, vocab = m["dims"]
    n = 0
    for L in m["layers"]:
        a = D.rmsnorm_q8(m["h"], L["nw1"], acts[("h", D.matrix_act_kind(L["q"]))], hidden, EPS)
        D.cmat_mul(L["q"], a, m["q"], 1)
        D.cmat_mul(L["k"], a, m["k"], 1)
        n += 3
        if D.matrix_act_kind(L["v"]) != a.kind:
            a = D.rmsnorm_q8(m["h"], L["nw1"], acts[("h", D.matrix_act_kind(L["v"]))], hidden, EPS)
            n += 1
        D.cmat_mul(L["v"], a, m["v"], 1)
        D.cmat_mul(L["o"], D.quant_q8(m["q"], acts[("q", D.matrix_act_kind(L["o"]))]), m["h"], 1, acc=True)
        a = D.rmsnorm_q8(m["h"], L["nw2"], acts[("h", D.matrix_act_kind(L["gate"]))], hidden, EPS)
        D.glu_mul(L["gate"], L["up"], a, m["fa"])
        D.cmat_mul(L["down"], D.quant_q8(m["fa"], acts[("fa", D.matrix_act_kind(L["down"]))]), m["h"], 1, acc=True)
        n += 7
    a = D.rmsnorm_q8(m["h"], m["nwf"], acts[("h", D.matrix_act_kind(m["head"]))], hidden, EPS)
    D.cmat_mul(m["head"], a, m["logits"], 1)
    return n + 2


def chain_leg(D, B, torch, dev, dims, layers, fmt_main, fmt_alt, seed, peak, name):
    """A token's chain both ways, timed; and that the two give the same logits."""
    m = build_chain_model(D, B, torch, dev, dims, layers, fmt_main, fmt_alt, seed)
    hidden, qdim, kvdim, ffn, vocab = dims
    acts = {(k, kind): D.make_qact(n, kind, device=dev) for k, n in (("h", hidden), ("q", qdim), ("fa", ffn)) for kind in ("q8", "q8k")}
    launches = [0]

    def per_product():
        m["h"].copy_(m["x0"])
        launches[0] = chain_per_product(D, m, acts) + 1
    plan = D.DecodePlan(chain_ops(D, m), device=dev)

    def one_launch():
        m["h"].copy_(m["x0"])
        plan.run()
    per_product()
    torch.cuda.synchronize()
    want = m["logits"].clone()
    m["logits"].zero_()
    one_launch()
    torch.cuda.synchronize()
    same = bool(torch.equal(m["logits"], want)) and bool(torch.isfinite(want).all())
    g = graph_of(per_product, torch)
    us_pp = time_us(g.replay, 10, torch)
    us_one = time_us(one_launch, 10, torch)
    out = {"workload": name, "weight_MB": m["bytes"] / 1e6,
           "per_product": {"us_per_token": us_pp, "GBps": m["bytes"] / us_pp / 1e3, "frac_of_hbm": m["bytes"] / us_pp / 1e3 / peak,
                           "launches": launches[0], "how": "one CUDA graph of the token's launches"},
           "one_launch": {"us_per_token": us_one, "GBps": m["bytes"] / us_one / 1e3, "frac_of_hbm": m["bytes"] / us_one / 1e3 / peak,
                          "launches": 1, "products": plan.n, "how": "ill_decode_run: one cooperative launch, a barrier between dependent products"},
           "parity": {"one_launch_equals_per_product_bits": same}}
    del m, plan, g
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-formats", action="store_true", help="skip the per-format sweep")
    ap.add_argument("--no-moe", action="store_true", help="skip the mixture-of-experts legs")
    ap.add_argument("--no-configs", action="store_true", help="skip the c1 / c2_chain / c3 / c4_decode legs")
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
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    peak, which = peaks()
    tpeak, twhich = tensor_peak()
    cores = len(os.sched_getaffinity(0))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(vals):
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

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
    # (configs.c2_chain runs the same token with the norms and every quantization inside.)
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

    # eager warm-up, then one CUDA graph of a step (removes host launch cost from the device number)
    for _ in range(args.warmup):
        h.zero_()
        token_step()
    graph = graph_of(token_step, torch)
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

    def all_glu():
        for L in layers:
            D.glu_mul(L["gate"], L["up"], act_d, fa)
    ggraph = graph_of(all_glu, torch)
    glu_us = time_us(ggraph.replay, 10, torch) / LAYERS
    del ggraph

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
            it = [0]

            def one():
                D.cmat_mul(ms_[it[0] & 1], act, y, 1)
                it[0] += 1
            us = time_us(one, 10, torch, warm=4)
            nb = ms_[0].nbytes
            formats[B.NAMES[fmt]] = {"rows": rows, "cols": cols, "MB": nb / 1e6, "us": us, "GBps": nb / us / 1e3,
                                     "frac_of_%s_hbm" % which: nb / us / 1e3 / peak}
            del ms_
            torch.cuda.empty_cache()

    clocks = sampler.stop() if rank == 0 else None  # sampled over the headline's timed regions and the kernels above
    ms, e2e_ms = max_over_ranks([ms, e2e_ms])
    # the headline's buffers are done with: make room for the other configurations
    del layers, head, graph
    torch.cuda.empty_cache()

    # ---- the other configurations, one GPU's worth each (rank 0 reports; every rank runs them, replicas)
    configs = {}
    if not args.no_configs:
        configs["c2_chain"] = chain_leg(D, B, torch, dev, (HIDDEN, QDIM, KVDIM, FFN, VOCAB), LAYERS, Q4_K, Q6_K, 1 + rank, peak,
                                        "configs[1] with RMSNorm and every activation quantization inside: q/k/v <- norm(h); h += o(q); "
                                        "fa <- glu(norm(h)); h += down(fa); head(norm(h))")
        configs["c1_token"] = chain_leg(D, B, torch, dev, (C1["hidden"], C1["qdim"], C1["kvdim"], C1["ffn"], C1["vocab"]), C1["layers"],
                                        Q8_0, Q8_0, 3 + rank, peak, "configs[0]: qwen2.5-0.5b, all Q8_0, one token (same chain)")
        configs["c2_prefill_512"] = prefill_leg(D, B, torch, dev, (HIDDEN, QDIM, KVDIM, FFN, VOCAB), LAYERS, Q4_K, Q6_K, 5 + rank, 512,
                                                tensor_peak())
        configs["c3_q6k_sweep"] = c3_sweep(D, B, torch, dev, peak, which)
        configs["c4_decode"] = c4_decode(D, B, torch, dev, peak)
        configs["c4_ffn_head_chunk"] = c4_head_chunk(D, B, torch, dev, 4096, tensor_peak())

    # ---- the sharded paths
    sharded = {}
    if not args.no_moe:
        from illatio_b200 import ep as EP
        from illatio_b200 import microbench_moe as MB
        sharded["head_rowsplit"] = head_rowsplit(D, B, EP, torch, dist, dev, rank, world, peak, barrier, max_over_ranks)
        sharded["moe_prefill"] = moe_leg(D, B, EP, MB, torch, dist, dev, rank, world, cores, "c4", 4096, tpeak, twhich, barrier,
                                         max_over_ranks, interleave=False)
        sharded["c5_prefill"] = moe_leg(D, B, EP, MB, torch, dist, dev, rank, world, cores, "c5", 8192, tpeak, twhich, barrier,
                                        max_over_ranks, interleave=True)
        sharded["c5_decode_64"] = moe_leg(D, B, EP, MB, torch, dist, dev, rank, world, cores, "c5", 64, tpeak, twhich, barrier,
                                          max_over_ranks, interleave=True, check=False)

    status = D.device_status()
    if rank == 0:
        value = world * total_bytes / (ms * 1e-3) / 1e9
        e2e = world * total_bytes / (e2e_ms * 1e-3) / 1e9
        achieved = glu_bytes / (glu_us * 1e-6) / 1e9
        out = {
            "metric": "quant matvec weight GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> int32 dots, fp32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "weight_bytes_per_step": total_bytes,
                       "l2": "every step reads 2.6 GB of distinct weights, far larger than the 126 MB L2",
                       "replicas": "each rank decodes its own token on its own copy (the decode products do not shard): across N "
                                   "`value` is weak scaling of independent copies.  The curves that scale with N are under `sharded`: "
                                   "moe_prefill.tok_per_s, c5_prefill.tok_per_s and head_rowsplit.n1.us_per_token, each with vs_1gpu and parity",
                       "launch": "one CUDA graph of the step's %d kernel launches" % launches_per_step[0]},
            "frac_of_%s_hbm" % which: value / world / peak,
            "e2e": {"value": e2e, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": HIDDEN * 4,
                    "d2h_bytes_per_step": VOCAB * 4},
            "gpu_launches": launches_per_step[0] * args.steps,
            "roofline": {"bound": "hbm", "kernel": "mvw_kernel<Q4_K, gated> (gate/up 2 x 9728x2560)",
                         "achieved": achieved, "peak": peak,
                         "peak_source": which + " (MEASURED_PEAKS.json hbm_gbs)" if which == "measured" else which,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": profiled_traffic("mvw_q4k_glu_9728x2560.json"),
                         "us_per_launch": glu_us, "algorithmic_bytes_per_launch": glu_bytes},
            "clocks": clocks, "formats": formats, "device_status": status, "configs": configs, "sharded": sharded,
        }
        if not args.no_cpu:
            fast_ok = False
            try:
                from oracle import oracle as O
                O.build()
                fast_ok = O.simd_available()
            except Exception:
                pass
            pg, preps, psecs, nb = cpu_layer_gbs(False, 6.0, cores)
            out["cpu_baseline"] = {"value": pg, "unit": "GB/s", "cores": cores, "kind": "port",
                                   "sample": "one layer of the workload (%.1f MB of blocks), portable scalar loops, %d repetitions, %.1f s"
                                             % (nb / 1e6, preps, psecs)}
            if fast_ok:
                fg, freps, fsecs, _ = cpu_layer_gbs(True, 6.0, cores)
                out["cpu_baseline"]["avx2"] = {"value": fg, "unit": "GB/s", "cores": cores, "kind": "port",
                                               "sample": "the same layer, AVX2 row dots on a pool of pinned threads, %d repetitions, %.1f s" % (freps, fsecs)}
            out["cpu_baseline"]["c4_moe_layer"] = cpu_moe_layer(3.0, cores)
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------ configuration legs

def prefill_leg(D, B, torch, dev, dims, layers, fmt_main, fmt_alt, seed, n, tpeak):
    """configs[1] as prefill: a chunk of N tokens through every in-scope product of the model (the chain of
    chain_leg with N rows: RMSNorm fused with the quantizer, q / k / v / o, gate and up, SwiGLU, down), the head for
    the last token only; one CUDA graph.  Attention itself is out of scope and stood in for by the query rows."""
    m = build_chain_model(D, B, torch, dev, dims, layers, fmt_main, fmt_alt, seed)
    hidden, qdim, kvdim, ffn, vocab = dims
    f = dict(dtype=torch.float32, device=dev)
    h0 = torch.randn(n * hidden, **f)
    h, q, k, v = torch.empty(n * hidden, **f), torch.empty(n * qdim, **f), torch.empty(n * kvdim, **f), torch.empty(n * kvdim, **f)
    ga, ub = torch.empty(n * ffn, **f), torch.empty(n * ffn, **f)
    acts = {(name, kind): D.make_qact(n * width, kind, device=dev) for name, width in (("h", hidden), ("q", qdim), ("fa", ffn))
            for kind in ("q8", "q8k")}
    last = D.make_qact(hidden, D.matrix_act_kind(m["head"]), device=dev)
    launches = [0]
    down_tc = D.tc_takes(m["layers"][0]["down"], n) and D.matrix_act_kind(m["layers"][0]["down"]) == "q8k"
    mid_cf = D.ChunkF16(n, ffn, device=dev) if down_tc else None
    L0_ = m["layers"][0]
    glu_tc = D.tc_takes(L0_["gate"], n) and L0_["gate"].type == L0_["up"].type and D.matrix_act_kind(L0_["gate"]) == "q8k"

    def chunk():
        h.copy_(h0)
        for L in m["layers"]:
            a = D.rmsnorm_q8(h, L["nw1"], acts[("h", D.matrix_act_kind(L["q"]))], hidden, EPS, n=n)
            D.cmat_mul(L["q"], a, q, n)
            D.cmat_mul(L["k"], a, k, n)
            if D.matrix_act_kind(L["v"]) != a.kind:
                a = D.rmsnorm_q8(h, L["nw1"], acts[("h", D.matrix_act_kind(L["v"]))], hidden, EPS, n=n)
            D.cmat_mul(L["v"], a, v, n)
            D.cmat_mul(L["o"], D.quant_q8(q, acts[("q", D.matrix_act_kind(L["o"]))]), h, n, acc=True)
            a = D.rmsnorm_q8(h, L["nw2"], acts[("h", D.matrix_act_kind(L["gate"]))], hidden, EPS, n=n)
            if glu_tc:   # gate and up in one launch of the tcgen05 kernel
                D.glu_mul_tc(L["gate"], L["up"], a, n, ga, ub)
            else:
                D.cmat_mul(L["gate"], a, ga, n)
                D.cmat_mul(L["up"], a, ub, n)
            if down_tc:   # SwiGLU, Q8_K and the fp16 form in one launch, straight into the tcgen05 product
                D.cmat_mul_tc(L["down"], D.swiglu_chunk_f16(ga, ub, mid_cf), h, acc=True)
            else:
                D.swiglu(ga, ub, ga, ffn)
                D.cmat_mul(L["down"], D.quant_q8(ga, acts[("fa", D.matrix_act_kind(L["down"]))]), h, n, acc=True)
        D.cmat_mul(m["head"], D.rmsnorm_q8(h[(n - 1) * hidden:], m["nwf"], last, hidden, EPS), m["logits"], 1)
    from illatio_b200 import _lib as LIB
    counted, real_call, real_status = [0], LIB.call, LIB.status

    def counting(fn):
        def wrapped(name, *a):
            r = fn(name, *a)
            counted[0] += 1 if r == 0 else 0   # a refusal (the caller then splits the tokens) launched nothing
            return r
        return wrapped
    LIB.call, LIB.status = counting(real_call), counting(real_status)   # every kernel launch goes through one of the two
    try:
        chunk()
    finally:
        LIB.call, LIB.status = real_call, real_status
    launches[0] = counted[0] + 1   # + the copy of the hidden states
    torch.cuda.synchronize()
    finite = bool(torch.isfinite(m["logits"]).all()) and bool(torch.isfinite(h).all())
    # parity, outside the timed region: the chunk product of the first layer's gate matrix against the one-token
    # product (itself held to the CPU oracle by the tests) for three of the tokens
    L0 = m["layers"][0]
    a = D.rmsnorm_q8(h0, L0["nw2"], acts[("h", D.matrix_act_kind(L0["gate"]))], hidden, EPS, n=n)
    D.cmat_mul(L0["gate"], a, ga, n)
    worst = 0.0
    one = D.make_qact(hidden, a.kind, device=dev)
    y1 = torch.empty(ffn, **f)
    for t in (0, n // 2 + 1, n - 1):
        D.rmsnorm_q8(h0[t * hidden:(t + 1) * hidden], L0["nw2"], one, hidden, EPS)
        D.cmat_mul(L0["gate"], one, y1, 1)
        worst = max(worst, float(((ga[t * ffn:(t + 1) * ffn] - y1).abs().max() / y1.abs().max()).item()))
    g = graph_of(chunk, torch)
    us = time_us(g.replay, 3, torch)
    body = m["bytes"] - m["head"].nbytes
    weights = sum(w.rows * w.cols for L in m["layers"] for w in L.values() if isinstance(w, D.CMat))
    tops = 2.0 * weights * n / us / 1e6
    out = {"workload": "configs[1], a %d-token chunk through %d layers' products and the last token's head" % (n, layers),
           "tokens": n, "ms": us / 1e3, "tokens_per_s": n / us * 1e6, "launches": launches[0], "how": "one CUDA graph",
           "int8_TOPS": tops, "frac_of_bf16_tensor_peak": tops / tpeak[0] if tpeak and tpeak[0] else None,
           "weight_MB_read_once": body / 1e6,
           "kernel": "Q4_K matrices of 2048 rows and more: mm_id_kernel<Q4_K> (tcgen05, ill_mm_chunk; fp16 integer operands, the "
                     "activations' fp16 form made once per quantization by ill_act_f16); k (1024 rows) and the Q6_K matrices (v, down): "
                     "mmd_kernel (int8 mma.sync, 128 rows x 128 tokens a CTA)",
           "parity": {"finite": finite, "chunk_vs_one_token_max_rel": worst, "ok": finite and worst < 2e-6}}
    del m, g
    torch.cuda.empty_cache()
    return out


def c4_head_chunk(D, B, torch, dev, n, tpeak):
    """configs[3]'s chunk before its routing (DK-FFN-HEAD-CHUNK): RMSNorm with the Q8_0 quantizer, the router's
    logits (F16 [256, 4096]) and the shared Q8_0 expert over N tokens."""
    from illatio_b200 import cuda_ds4f_prefill as P
    from illatio_b200 import cuda_ds4f as M
    d, ff, ne, clamp = 4096, 2048, 256, 10.0
    ws = [D.CMat("sh", Q8_0, r, c, B.synth_matrix_torch(Q8_0, r, c, seed=90 + i, device=dev)) for i, (r, c) in enumerate(((ff, d), (ff, d), (d, ff)))]
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    router = (torch.randn(ne, d, device=dev, generator=g) * 0.05).to(torch.float16)
    cur = torch.randn(n, d, device=dev, generator=g)
    nw = torch.rand(d, device=dev, generator=g) + 0.5
    hs = P.HeadScratch(n, d, ff, ne, device=dev)

    def head():
        P.dk_ffn_head_chunk(cur, nw, EPS, router, ws[0], ws[1], ws[2], clamp, hs)
    head()
    torch.cuda.synchronize()
    # parity, outside the timed region: three tokens through the one-token drivers (DK-MV16, the shared expert as
    # DK-FFN-HEAD runs it), which the tests hold to the CPU oracle
    worst_l = worst_s = 0.0
    y1, l1 = torch.empty(d, device=dev), torch.empty(ne, device=dev)
    for t in (0, n // 2 + 1, n - 1):
        M.dk_mv16(router, hs.norm2[t], l1)
        M.dk_shared(ws[0], ws[1], ws[2], hs.norm2[t], clamp, y1)
        worst_l = max(worst_l, float(((hs.logits[t] - l1).abs().max() / l1.abs().max()).item()))
        worst_s = max(worst_s, float(((hs.sout[t] - y1).abs().max() / y1.abs().max()).item()))
    gr = graph_of(head, torch)
    us = time_us(gr.replay, 5, torch)
    macs = n * (3.0 * d * ff + ne * d)
    out = {"workload": "configs[3]: %d tokens, RMSNorm + router logits + shared Q8_0 expert (gate / up / down)" % n, "tokens": n,
           "ms": us / 1e3, "launches": 8, "how": "one CUDA graph", "TOPS": 2.0 * macs / us / 1e6,
           "frac_of_bf16_tensor_peak": 2.0 * macs / us / 1e6 / tpeak[0] if tpeak and tpeak[0] else None,
           "parity": {"logits_vs_one_token_max_rel": worst_l, "shared_vs_one_token_max_rel": worst_s,
                      "ok": worst_l < 1e-5 and worst_s < 1e-5}}
    del gr, ws, hs
    torch.cuda.empty_cache()
    return out


def c3_sweep(D, B, torch, dev, peak, which):
    """configs[2]: the Q6_K matrices of a 27B-scale model at batch 1, 4 and 16, cold (a rotation of copies whose
    total is larger than twice the L2)."""
    out = {"format": "q6_k", "protocol": "copies rotated so that every launch reads its weights from HBM"}
    for name, rows, cols in (("5120x5120", 5120, 5120), ("17408x5120", 17408, 5120), ("5120x17408", 5120, 17408),
                             ("151936x5120", 151936, 5120)):
        nb = B.matrix_bytes(Q6_K, rows, cols)
        copies = max(2, int(-(-300e6 // nb)))
        ms_ = [D.CMat("w", Q6_K, rows, cols, B.synth_matrix_torch(Q6_K, rows, cols, seed=70 + i, device=dev)) for i in range(copies)]
        res = {"MB": nb / 1e6, "copies": copies}
        for n in (1, 4, 16):
            xx = torch.randn(n * cols, device=dev)
            act = D.make_qact(n * cols, "q8k", device=dev)
            D.quant_q8(xx, act)
            y = torch.empty(n * rows, device=dev)

            def sweep():
                for w in ms_:
                    D.cmat_mul(w, act, y, n)
            gph = graph_of(sweep, torch)
            us = time_us(gph.replay, 5, torch) / copies
            res["n%d" % n] = {"us": us, "GBps": nb / us / 1e3, "frac_of_%s_hbm" % which: nb / us / 1e3 / peak}
            del gph
        out[name] = res
        del ms_
        torch.cuda.empty_cache()
    return out


def c4_decode(D, B, torch, dev, peak):
    """configs[3] as decode: one token through one MoE layer (router given; 6 routed experts of 256 + the shared
    Q8_0 expert), 16 tokens with different routings back to back; the shared expert rotates over six copies."""
    from illatio_b200 import cuda_ds4f as M
    from illatio_b200 import microbench_moe as MB
    cfg = MB.CONFIGS["c4"]
    d, ff, nu = cfg["d"], cfg["ff"], cfg["nu"]
    pool = MB.make_pool(cfg, seed=7, device=dev)
    shared = [[D.CMat("s", Q8_0, r, c, B.synth_matrix_torch(Q8_0, r, c, seed=500 + 3 * i + j, device=dev))
               for j, (r, c) in enumerate(((ff, d), (ff, d), (d, ff)))] for i in range(6)]
    T = 16
    gg = torch.Generator(device=dev)
    gg.manual_seed(21)
    norms = torch.randn(T, d, device=dev, generator=gg)
    logits = torch.randn(T, cfg["ne"], device=dev, generator=gg)
    sel, w = M.route(logits, nu, mode=2)
    sh_out, moe = torch.empty(d, device=dev), torch.empty(d, device=dev)

    def tokens():
        for t in range(T):
            sg, su, sd = shared[t % 6]
            M.dk_shared(sg, su, sd, norms[t], 10.0, sh_out)
            M.dk_ffn_tail(pool, norms[t], sel[t], w[t], 10.0, shared=sh_out, moe=moe)
    tokens()
    us_eager = time_us(tokens, 5, torch) / T
    # the same sixteen tokens as one CUDA graph: the routing, the experts' addresses and every buffer are on the
    # device, so the host's launch cost (and the allocator's) is off the path, as it is when illatio's Lisp host
    # enqueues from preallocated buffers
    g = graph_of(tokens, torch)
    us = time_us(g.replay, 5, torch) / T
    del g
    routed = nu * (2 * B.matrix_bytes(IQ2_XXS, ff, d) + B.matrix_bytes(Q2_K, d, ff))
    sh_bytes = 3 * B.matrix_bytes(Q8_0, ff, d)
    out = {"workload": "one token through the layer: shared expert (3 Q8_0 products) + 6 routed experts (IQ2_XXS gate / up fused, Q2_K down) + slot-order sum",
           "us_per_token_layer": us, "MB": (routed + sh_bytes) / 1e6, "GBps": (routed + sh_bytes) / us / 1e3,
           "frac_of_hbm": (routed + sh_bytes) / us / 1e3 / peak, "launches_per_token_layer": 12,
           "how": "16 tokens with different routings in one CUDA graph", "us_per_token_layer_eager": us_eager}
    del pool, shared
    torch.cuda.empty_cache()
    return out


def head_rowsplit(D, B, EP, torch, dist, dev, rank, world, peak, barrier, max_over_ranks):
    """configs[2]'s output head, 151936 x 5120 Q6_K, split by rows over the ranks, then an all-gather of the logits;
    batch 1, 4 and 16.  Copies of the rank's slice rotate so that the weights come from HBM.  The product
    and the collective are also timed apart.  Parity: the gathered logits against rank 0's product of the whole
    matrix (exact: a row's arithmetic does not depend on which rank multiplies it)."""
    rows, cols = VOCAB, 5120
    first, end = EP.head_rows(rows, world, rank)
    rb = B.row_bytes(Q6_K, cols)

    def slice_of(copy):
        # every rank draws the whole matrix's stream and keeps its rows: any split is the same matrix
        full = B.synth_matrix_torch(Q6_K, rows, cols, seed=880 + copy, device=dev)
        s = full[first * rb:end * rb].clone()
        del full
        return D.CMat("head_slice", Q6_K, end - first, cols, s)
    # as many copies of the rank's slice as it takes to exceed twice the L2 (two at N <= 2, eight at N = 8): every launch
    # reads its weights from HBM
    ncopies = max(2, int(-(-300e6 // ((end - first) * rb))))
    slices = [slice_of(i) for i in range(ncopies)]
    torch.cuda.empty_cache()
    out = {"matrix": "151936 x 5120 Q6_K (638 MB)", "rows_per_gpu": end - first,
           "collective": "in-place all-gather of fp32 logits (NCCL)" if world > 1 else "none (one GPU)",
           "GBps_is": "the whole matrix's bytes over the time of the slowest rank: an aggregate over the ranks"}
    nb = B.matrix_bytes(Q6_K, rows, cols)
    sl = end - first
    pg = EP.PeerGather(16 * (rows - (world - 1) * (rows // world)) * 4, world, device=dev) if world > 1 else None
    if pg is not None:
        out["collective"] = ("peer stores of the rank's logits into every peer's buffer and one flag meeting -- from the "
                             "product's own epilogue at batch 1 (ill_mv_peers), a second kernel at batch 4 / 16 (ill_peer_put); "
                             "NCCL's in-place all-gather timed beside it")
    for n in (1, 4, 16):
        xx = torch.randn(n * cols, device=dev, generator=torch.Generator(device=dev).manual_seed(5))
        act = D.make_qact(n * cols, "q8k", device=dev)
        D.quant_q8(xx, act)
        # the logits as [rank, token, the rank's rows]: every rank's product writes its own block, one in-place
        # all-gather fills the rest (token t's logits are the ranks' blocks [:, t, :] side by side)
        gathered = torch.zeros(world, n, end - first, device=dev)
        part = gathered[rank]
        it = [0]

        def product_only():
            w = slices[it[0] % ncopies]
            it[0] += 1
            D.cmat_mul(w, act, part, n)

        def gather_only():
            dist.all_gather_into_tensor(gathered, part)

        def both():
            product_only()
            if world > 1:
                gather_only()
        us_peer = us_put = None
        if pg is not None:
            mine = [pg.buffer(i)[rank][:n * sl * 4].view(torch.float32) for i in (0, 1)]

            def both_peer():
                i, w = it[0] & 1, slices[it[0] % ncopies]
                it[0] += 1
                if n == 1:   # the product stores into every rank's buffer itself and holds the meeting: one launch
                    pg.mul_put(i, w, act)
                else:
                    D.cmat_mul(w, act, mine[i], n)
                    pg.put(i, n * sl * 4)
            barrier()
            us_peer = time_us(both_peer, 20, torch)
            barrier()
            us_put = time_us(lambda: pg.put(0, n * sl * 4), 20, torch)
            barrier()
        barrier()
        us_both = time_us(both, 20, torch)
        barrier()
        us_prod = time_us(product_only, 20, torch)
        us_gather = 0.0
        if world > 1:
            barrier()
            us_gather = time_us(gather_only, 20, torch)
        us_both, us_prod, us_gather, us_peer_m, us_put_m = max_over_ranks([us_both, us_prod, us_gather, us_peer or 0.0, us_put or 0.0])
        us_nccl = us_both
        if pg is not None:
            us_both = min(us_peer_m, us_nccl)   # a host picks the faster of the two once, when it sets the head up
        res = {"us_per_token": us_both, "GBps": nb / us_both / 1e3, "us_product": us_prod, "us_all_gather": us_gather,
               "us_with_nccl_all_gather": us_nccl if pg is not None else None,
               "us_with_peer_stores": us_peer_m if pg is not None else None, "us_peer_stores_alone": us_put_m if pg is not None else None,
               "product_frac_of_hbm_per_gpu": (nb / world) / us_prod / 1e3 / peak}
        if n == 1:
            # parity and the one-GPU time, on rank 0 (the whole matrix, copy 0)
            it[0] = 0
            if pg is not None:
                both_peer()
                torch.cuda.synchronize()
                barrier()
                per = rows // world
                got = torch.cat([pg.buffer(0)[r][:(rows - r * per if r == world - 1 else per) * 4].view(torch.float32)
                                 for r in range(world)]).clone()
            else:
                both()
                torch.cuda.synchronize()
                got = gathered.reshape(-1).clone()
            vs = None
            ok = None
            if rank == 0:
                full = D.CMat("head", Q6_K, rows, cols, B.synth_matrix_torch(Q6_K, rows, cols, seed=880, device=dev))
                full2 = D.CMat("head", Q6_K, rows, cols, B.synth_matrix_torch(Q6_K, rows, cols, seed=881, device=dev))
                want = torch.empty(rows, device=dev)
                D.cmat_mul(full, act, want, 1)
                torch.cuda.synchronize()
                ok = bool(torch.equal(got, want))
                j = [0]

                def alone():
                    D.cmat_mul((full, full2)[j[0] & 1], act, want, 1)
                    j[0] += 1
                us1 = time_us(alone, 20, torch)
                vs = us1 / us_both
                res["us_one_gpu_same_run"] = us1
                del full, full2
                torch.cuda.empty_cache()
            barrier()
            res["vs_1gpu"] = vs
            res["parity"] = {"gathered_logits_equal_one_gpu_product": ok, "ranks": world}
        out["n%d" % n] = res
    if pg is not None:
        torch.cuda.synchronize()
        barrier()
        pg.close()
    del slices, pg
    torch.cuda.empty_cache()
    return out


def moe_leg(D, B, EP, MB, torch, dist, dev, rank, world, cores, cfg_name, n_tok, tpeak, twhich, barrier, max_over_ranks,
            interleave, check=True):
    """One chunk of N_TOK tokens through a layer's routed experts, experts placed expert-parallel over the ranks
    (tokens split by position): time, tokens/s, rows per rank, slab overflows; the same chunk on rank 0 alone
    (vs_1gpu); and 8 of every rank's tokens against the CPU oracle (parity)."""
    from illatio_b200 import cuda_ds4f_prefill as P
    cfg = MB.CONFIGS[cfg_name]
    ne, nu, d, ff = cfg["ne"], cfg["nu"], cfg["d"], cfg["ff"]
    per = ne // world
    seed = 7
    mine = MB.interleaved_experts(ne, world, rank) if interleave else list(range(rank * per, (rank + 1) * per))
    order = MB.virtual_order(ne, world) if interleave else list(range(ne))
    pool = MB.make_pool(cfg, seed=seed, device=dev, experts=mine)
    gm = torch.Generator(device=dev)
    gm.manual_seed(11)  # the same chunk on every rank; each takes its slice of the tokens
    norms_all = torch.randn(n_tok, d, device=dev, generator=gm)
    # the router's logits in the order the ranks hold the experts (its rows are permuted once, when a model is loaded)
    logits_all = MB.router_logits(cfg, n_tok, seed=12, device=dev)[:, torch.tensor(order, device=dev)].contiguous()
    lo, hi = rank * n_tok // world, (rank + 1) * n_tok // world
    norms_l, logits_l = norms_all[lo:hi].contiguous(), logits_all[lo:hi].contiguous()
    ce = EP.CudaExperts(pool, nu, 10.0)
    peer = world > 1 and os.environ.get("ILL_EP_COMBINE", "peer") == "peer"
    made = 1
    try:
        esc = EP.EpCapScratch(pool, hi - lo, nu, ne, world, device=dev, peer=peer)
    except Exception as exc:  # no peer mapping on this box: the same exchanges over NCCL
        print("rank %d: symmetric memory unavailable (%s)" % (rank, exc), file=sys.stderr)
        made = 0
    if peer:  # every rank takes the same path
        agree = torch.tensor([made], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if agree.item() == 0:
            peer = False
            esc = EP.EpCapScratch(pool, hi - lo, nu, ne, world, device=dev, peer=False)
    flags = []

    def chunk():
        flags.append(EP.chunk_capacity(ce, esc, norms_l, logits_l, ne)[1].clone())
    for _ in range(3):
        chunk()
    if world == 1:
        # one GPU has nothing to exchange: the timed chunk is the plain chunk driver (DK-FFN-ROUTED-CHUNK; the same bits,
        # without the slabs' pack / plan / unpack steps) -- the same thing `vs_1gpu` is measured against at N > 1
        sc1 = P.make_chunk_scratch(pool, n_tok, nu, device=dev)

        def chunk():  # noqa: F811
            P.dk_ffn_routed_chunk(pool, norms_l, logits_l, nu, 10.0, sc1)
        for _ in range(2):
            chunk()
    barrier()
    reps = 12 if n_tok >= 1024 else 40
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        chunk()
    e1.record()
    barrier()
    ms = max_over_ranks([e0.elapsed_time(e1) / reps])[0]
    overflows = int(sum(int(f.item()) for f in flags))
    rows_here = float(esc.total.item())
    rmax = max_over_ranks([rows_here])[0]
    rsum = torch.tensor([rows_here], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(rsum)
    flop = 2.0 * n_tok * nu * 3 * d * ff
    out = {"workload": "%s: hidden %d, %d experts of FFN %d, top-%d, %s gate/up, Q2_K down%s; one %d-token chunk through the routed experts"
                       % (cfg_name, d, ne, ff, nu, B.NAMES[cfg["gate_fmt"]], ", Zipf(1.1) popularity" if cfg["zipf"] else "", n_tok),
           "n_gpus": world, "experts_per_gpu": per, "tokens": n_tok, "ms_per_chunk": ms,
           "placement": "interleaved (rank r holds experts r, r + N, ...; the router's rows permuted to match at load time)" if interleave
                        else "contiguous blocks of experts",
           "rows_per_rank": {"max": rmax, "mean": rsum.item() / world, "slab_rows": esc.cap * world},
           "slab_overflows": overflows, "exchange_sizes": "fixed slabs, no host synchronisation",
           "exchange": ("none (one GPU)" if world == 1 else
                        "peer stores over NVLink: packed Q8_K rows out (1.14 B/value), fp32 rows back from the down product's epilogue"
                        if peer else "NCCL all-to-all of packed Q8_K rows out (1.14 B/value), fp32 rows back"),
           "tok_per_s": n_tok / ms * 1e3, "tflops": flop / ms / 1e9, "scaling": "strong",
           "roofline": {"bound": "tensor", "achieved": flop / ms / 1e9 / world, "peak": tpeak, "peak_source": twhich,
                        "unit": "TFLOP/s per GPU, whole chunk (products and all the steps around them)",
                        "frac": flop / ms / 1e9 / world / tpeak}}
    if n_tok < 1024:
        out["note"] = ("batched decode (DK-FFN-SMALL, src/cuda-ds4f-spec.lisp:31-132) through the chunk driver: tensor-core "
                       "products on the few rows an expert has, its weights read and unpacked once for all of them")
        if world == 1:
            # the same batch on the one-token kernels, an expert's rows next to each other (ill_moe_row_ptrs): the form the
            # reference runs, here the slower one (the 2-bit matvecs are bound by instructions, a row at a time)
            sc2 = P.make_chunk_scratch(pool, n_tok, nu, device=dev)

            def small_mv():
                P.dk_ffn_small_mv(pool, norms_l, logits_l, nu, 10.0, sc2)
            mv_us = time_us(small_mv, 20, torch)
            same = bool(torch.allclose(sc2.moe, sc1.moe, rtol=0, atol=2e-3 * float(sc1.moe.abs().max())))
            out["matvec_path"] = {"ms_per_chunk": mv_us / 1e3, "tok_per_s": n_tok / mv_us * 1e6, "launches": 9,
                                  "agrees_with_chunk_driver": same,
                                  "how": "route, group, row pointers, gather, Q8_K, ill_moe_glu, Q8_K, ill_moe_mv, sum"}
    got_l = esc.moe.clone()
    sel_l = esc.sel.clone()
    # ---- parity: 8 of this rank's tokens against the CPU oracle, which is given those tokens' experts only
    # (any expert's bytes can be drawn again from its seed)
    if check:
        from oracle import oracle as O
        O.build()
        rng = np.random.default_rng(100 + rank)
        toks = np.unique(np.concatenate([[0, hi - lo - 1], rng.integers(0, hi - lo, 6)]))
        lg = logits_l[torch.as_tensor(toks, device=dev)].cpu().numpy()
        osel, ow = O.route(lg, nu, mode=2)
        sel_h = sel_l[torch.as_tensor(toks, device=dev)].cpu().numpy()
        got = got_l[torch.as_tensor(toks, device=dev)].cpu().numpy()
        nm = norms_l[torch.as_tensor(toks, device=dev)].cpu().numpy()
        worst, checked = 0.0, 0
        threads = max(1, cores // world)
        for i in range(len(toks)):
            if not np.array_equal(sel_h[i], osel[i]):
                continue  # expf's last place swapped two near-equal experts: not this token
            parts = []
            for tensor, (fmt, rows, cols) in enumerate(((cfg["gate_fmt"], ff, d), (cfg["gate_fmt"], ff, d), (B.Q2_K, d, ff))):
                parts.append(np.concatenate([B.synth_matrix_torch(fmt, rows, cols, seed=MB.expert_seed(seed, tensor, order[int(v)]),
                                                                  device=dev).cpu().numpy() for v in osel[i]]))
            want = O.moe_routed(d, ff, cfg["gate_fmt"], B.Q2_K, parts[0], parts[1], parts[2], nm[i], np.arange(nu, dtype=np.int32),
                                ow[i], 10.0, threads=threads)
            worst = max(worst, float(np.abs(got[i] - want).max() / np.abs(want).max()))
            checked += 1
        worst, nchecked = max_over_ranks([worst, -float(checked)])
        tot = torch.tensor([float(checked)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tot)
        out["parity"] = {"max_rel_err": worst, "tokens_checked": int(tot.item()), "ranks": world, "bound": 2e-3,
                         "ok": bool(worst < 2e-3 and tot.item() >= 4 * world and overflows == 0)}
    barrier()
    esc.close()
    del esc, ce, pool
    torch.cuda.empty_cache()
    # ---- the same chunk on rank 0 alone, every expert on its GPU
    vs = None
    if world > 1:
        if rank == 0:
            full = MB.make_pool(cfg, seed=seed, device=dev, experts=order)
            sc = P.make_chunk_scratch(full, n_tok, nu, device=dev)

            def alone():
                P.dk_ffn_routed_chunk(full, norms_all, logits_all, nu, 10.0, sc)
            ms1 = time_us(alone, 6, torch) / 1e3
            vs = ms1 / ms
            out["ms_one_gpu_same_run"] = ms1
            del full, sc
            torch.cuda.empty_cache()
        barrier()
    else:
        vs = 1.0
    out["vs_1gpu"] = vs
    return out


if __name__ == "__main__":
    main()
