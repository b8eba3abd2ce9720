"""The chunk's routed-expert product (tcgen05) against the CPU oracle.

The oracle multiplies Q8_K activations with exact integer dots; the device
multiplies the same dequantized values rounded to fp16 (weights and
activations) with fp32 accumulation, so outputs agree to about 5e-4 of the
largest output -- inside the 2e-3 the path is specified to.
"""
import numpy as np
import pytest
import torch

from illatio_b200 import _lib
from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from illatio_b200 import cuda_ds4f as M
from illatio_b200 import cuda_ds4f_prefill as P
from gpu_util import rel_errors, to_dev

pytestmark = pytest.mark.gpu
TOL_SPEC = 2e-3


@pytest.fixture(autouse=True)
def _need_gpu(cuda_lib):
    assert torch.cuda.is_available()
    yield
    assert D.device_status() == 0


def _pool(d, ff, ne, gate_fmt, seed):
    gate = B.synth_matrix(gate_fmt, ne * ff, d, seed=seed + 1)
    up = B.synth_matrix(gate_fmt, ne * ff, d, seed=seed + 2)
    down = B.synth_matrix(B.Q2_K, ne * d, ff, seed=seed + 3)
    return (gate, up, down), M.make_expert_pool(gate, up, down, d, ff, ne, gate_fmt=gate_fmt)


@pytest.mark.parametrize("fmt,rows_w,cols,counts", [
    (B.IQ2_XXS, 256, 512, [5, 0, 130, 1]),      # empty expert, one row, a partial second tile
    (B.Q2_K, 384, 256, [128, 129, 0, 0, 3]),    # exact tile, tile + 1
    (B.IQ2_XXS, 200, 1024, [40]),               # weight rows not a multiple of the tile
])
def test_mm_id_matches_float64_product(oracle, fmt, rows_w, cols, counts):
    """One indexed product alone: Y = XH . dequant(W_e)^T against float64."""
    ne = len(counts)
    rb = B.row_bytes(fmt, cols)
    w = B.synth_matrix(fmt, ne * rows_w, cols, seed=len(counts))
    slot = (rows_w * rb + 255) // 256 * 256
    poolbuf = torch.zeros(ne * slot, dtype=torch.uint8, device="cuda")
    poolbuf.view(ne, slot)[:, :rows_w * rb] = to_dev(w).view(ne, rows_w * rb)
    ptrs = torch.tensor([poolbuf.data_ptr() + e * slot for e in range(ne)], dtype=torch.int64, device="cuda")
    total = sum(counts)
    rng = np.random.default_rng(1)
    x = rng.standard_normal((total, cols)).astype(np.float32)
    xq, xd, _ = oracle.quantize_q8k(x)
    xh = torch.empty(total, cols, dtype=torch.float16, device="cuda")
    _lib.call("ill_act_f16", total, cols, to_dev(xq).data_ptr(), to_dev(xd).data_ptr(), 0, xh.data_ptr(), None)
    xdeq = xq.reshape(total, cols).astype(np.float32) * np.repeat(xd, 256).reshape(total, cols)
    assert np.array_equal(xh.cpu().numpy(), xdeq.astype(np.float16))
    y = torch.full((total + 4, rows_w), 7.0, dtype=torch.float32, device="cuda")
    bases = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32)
    _lib.call("ill_moe_mm_id", fmt, cols, rows_w, 0, ptrs.data_ptr(), to_dev(np.array(counts, np.int32)).data_ptr(),
              to_dev(bases).data_ptr(), ne, total, xh.data_ptr(), y.data_ptr(), rows_w, None)
    got = y.cpu().numpy()
    assert (got[total:] == 7.0).all()
    wf = oracle.dequant(fmt, w, ne * rows_w, cols).astype(np.float64).reshape(ne, rows_w, cols)
    want = np.concatenate([xdeq[b:b + c].astype(np.float64) @ wf[e].T for e, (b, c) in enumerate(zip(bases, counts))])
    a, _ = rel_errors(got[:total], want)
    assert a < 1e-3, a


@pytest.mark.parametrize("d,ff,ne,nu,n,gate_fmt,clamp", [
    (512, 256, 8, 2, 300, B.IQ2_XXS, 10.0),
    (1024, 512, 6, 3, 257, B.Q2_K, 0.0),
])
def test_chunk_matches_oracle_small(oracle, d, ff, ne, nu, n, gate_fmt, clamp):
    (gate, up, down), pool = _pool(d, ff, ne, gate_fmt, seed=n)
    rng = np.random.default_rng(3)
    norms = rng.standard_normal((n, d)).astype(np.float32)
    logits = rng.standard_normal((n, ne)).astype(np.float32)
    sc = P.make_chunk_scratch(pool, n, nu)
    moe = P.dk_ffn_routed_chunk(pool, to_dev(norms), to_dev(logits), nu, clamp, sc)
    got = moe.cpu().numpy()
    osel, ow = oracle.route(logits, nu, mode=2)
    assert np.array_equal(sc.sel.cpu().numpy(), osel)
    want = np.stack([oracle.moe_routed(d, ff, gate_fmt, B.Q2_K, gate, up, down, norms[t], osel[t], ow[t], clamp, threads=4)
                     for t in range(n)])
    a, _ = rel_errors(got, want)
    assert a < TOL_SPEC, a
