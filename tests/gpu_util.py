"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D


def to_dev(a):
    return torch.as_tensor(np.ascontiguousarray(a)).cuda()


def dev_act(fmt, x, f16_scale=True):
    """Quantize X (numpy float32, n*cols) on the device in the kind FMT takes."""
    kind = "q8" if fmt == B.Q8_0 else "q8k"
    xd = to_dev(x.astype(np.float32).reshape(-1))
    act = D.make_qact(xd.numel(), kind, want_xsum=False)
    D.quant_q8(xd, act, f16_scale=f16_scale)
    return act


def act_to_host(act):
    xq = act.xq.cpu().numpy()
    xs = act.xs.cpu().numpy()
    bs = None
    if act.kind == "q8k":
        bs = act.xsum.cpu().numpy().astype(np.int32)
    return xq, xs, bs


def rel_errors(got, want, terms=None):
    """(max|d|/max|ref|, max per-row |d|/sum|terms| or None)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    a = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    b = None
    if terms is not None:
        b = (np.abs(got - want) / terms).max()
    return a, b


def sum_terms(oracle, fmt, w, rows, cols, act_host, n=1):
    """sum_j |w_rj| * |x_j| per (token, row): the scale of a row's rounding error."""
    xq, xs, _ = act_host
    per = 32 if fmt == B.Q8_0 else 256
    xf = np.abs(xq.astype(np.float64) * np.repeat(xs.astype(np.float64), per)).reshape(n, cols)
    wf = np.abs(oracle.dequant(fmt, w, rows, cols).astype(np.float64))
    return xf @ wf.T
