"""One small case of a dense kernel, run a few times and timed: the command a profiler is pointed at.

    python -m illatio_b200.microbench_dense mv   q6_k 151936 5120 4      # ill_mv: FORMAT ROWS COLS TOKENS
    python -m illatio_b200.microbench_dense glu  q4_k 9728 2560           # ill_mv_glu
    python -m illatio_b200.microbench_dense chain q|qb|head|glu           # ill_decode_run: a chain of products
                                                                          #   q: 36 Q4_K 4096x2560, no barriers; qb: the same
                                                                          #   with a barrier after each; head: two Q6_K
                                                                          #   151936x2560; glu: twelve gated Q4_K 9728x2560

Weights are synthetic blocks made on the device (blocks.synth_matrix_torch); a rotation of copies keeps every
launch's weights out of L2.  Prints the mean time a launch and the device status word.
"""
import sys

import torch

from . import blocks as B
from . import cuda_dense as D

FORMATS = {"q8_0": B.Q8_0, "q4_k": B.Q4_K, "q6_k": B.Q6_K, "q2_k": B.Q2_K, "iq2_xxs": B.IQ2_XXS}


def _mat(fmt, rows, cols, seed):
    return D.CMat("w", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=seed))


def _time(fn, launches, reps=3):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * launches)


def run_mv(fmt, rows, cols, n, glu=False):
    nb = B.matrix_bytes(fmt, rows, cols) * (2 if glu else 1)
    copies = max(2, int(300e6 // nb) + 1)
    ws = [(_mat(fmt, rows, cols, 2 * i), _mat(fmt, rows, cols, 2 * i + 1) if glu else None) for i in range(copies)]
    x = torch.randn(n * cols, device="cuda")
    act = D.quant_q8(x, D.make_qact(n * cols, D.matrix_act_kind(ws[0][0])))
    y = torch.empty(n * rows, device="cuda")

    def sweep():
        for w, u in ws:
            if glu:
                D.glu_mul(w, u, act, y)
            else:
                D.cmat_mul(w, act, y, n)
    us = _time(sweep, copies)
    print("%s %s %dx%d n=%d: %.1f us a launch, %.0f GB/s of weights, status %d"
          % ("glu" if glu else "mv", B.NAMES[fmt], rows, cols, n, us, nb / us / 1e3, D.device_status()))


def run_chain(case):
    x0 = torch.randn(2560, device="cuda")
    if case in ("q", "qb"):
        ws = [_mat(B.Q4_K, 4096, 2560, i) for i in range(36)]
        y = torch.empty(4096, device="cuda")
        ops = [D.decode_op(w, x0, y, after=(case == "qb")) for w in ws]
    elif case == "head":
        ws = [_mat(B.Q6_K, 151936, 2560, i) for i in range(2)]
        y = torch.empty(151936, device="cuda")
        ops = [D.decode_op(w, x0, y, after=False) for w in ws]
    elif case == "glu":
        ws = [(_mat(B.Q4_K, 9728, 2560, 2 * i), _mat(B.Q4_K, 9728, 2560, 2 * i + 1)) for i in range(12)]
        y = torch.empty(9728, device="cuda")
        ops = [D.decode_op(g, x0, y, w2=u, after=False) for g, u in ws]
    else:
        raise SystemExit("chain case: q, qb, head or glu")
    plan = D.DecodePlan(ops)
    us = _time(plan.run, 1, reps=1)
    print("chain %s: %d products, %.1f us a launch, status %d" % (case, len(ops), us, D.device_status()))


def main(argv):
    if len(argv) >= 2 and argv[0] == "chain":
        run_chain(argv[1])
    elif len(argv) >= 5 and argv[0] == "mv":
        run_mv(FORMATS[argv[1]], int(argv[2]), int(argv[3]), int(argv[4]))
    elif len(argv) >= 4 and argv[0] == "glu":
        run_mv(FORMATS[argv[1]], int(argv[2]), int(argv[3]), 1, glu=True)
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main(sys.argv[1:])
