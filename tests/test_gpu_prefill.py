"""The chunk's routed-expert product (tcgen05) against the CPU oracle.

Both sides multiply the same integers exactly (the device as fp16 operands of
tcgen05 MMAs, block by block) and scale each 256-wide block's sum by d_w * d_x
in fp32, so the products agree to fp32 rounding; across the whole layer the
only other difference is expf in the gate, whose last-place differences can
move a quantized middle value by one step now and then.
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
def test_mm_id_matches_oracle_rows(oracle, fmt, rows_w, cols, counts):
    """One indexed product alone: each valid row of Y against the oracle's row dots."""
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
    xq, xd, bs = oracle.quantize_q8k(x)
    dxq, dxd, dbs = to_dev(xq), to_dev(xd), to_dev(bs.astype(np.int16))  # named: they must outlive the launches
    xh = torch.empty(total, cols, dtype=torch.float16, device="cuda")
    xe = torch.full((total, cols // 256, 64), 9.0, dtype=torch.float16, device="cuda")
    _lib.call("ill_act_f16", total, cols, dxq.data_ptr(), dbs.data_ptr(), 0, xh.data_ptr(), xe.data_ptr(), None)
    assert np.array_equal(xh.cpu().numpy().astype(np.int32), xq.reshape(total, cols))
    xeh = xe.cpu().numpy()
    assert np.array_equal(xeh[:, :, :16].astype(np.int32), bs.reshape(total, cols // 256, 16)) and (xeh[:, :, 16:] == 0).all()
    y = torch.full((total + 4, rows_w), 7.0, dtype=torch.float32, device="cuda")
    bases = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32)
    dcounts, dbases = to_dev(np.array(counts, np.int32)), to_dev(bases)
    _lib.call("ill_moe_mm_id", fmt, cols, rows_w, 0, ptrs.data_ptr(), dcounts.data_ptr(), dbases.data_ptr(), ne, total,
              xh.data_ptr(), xe.data_ptr(), dxd.data_ptr(), 0, 0, y.data_ptr(), rows_w, None)
    got = y.cpu().numpy()
    assert (got[total:] == 7.0).all()
    want = np.empty((total, rows_w), np.float32)
    for e, (b, c) in enumerate(zip(bases, counts)):
        we = w[e * rows_w * rb:(e + 1) * rows_w * rb]
        for r in range(b, b + c):
            act = (xq[r * cols:(r + 1) * cols], xd[r * (cols // 256):(r + 1) * (cols // 256)],
                   bs[r * (cols // 16):(r + 1) * (cols // 16)])
            want[r] = oracle.matvec(fmt, we, rows_w, cols, act)[0]
    a, _ = rel_errors(got[:total], want)
    assert a < 1e-5, a


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
    assert a < TOL_SPEC and a < 2e-4, a


@pytest.mark.parametrize("gate_fmt", [B.IQ2_XXS, B.Q2_K])
def test_fused_middle_equals_three_steps(gate_fmt):
    """SwiGLU + Q8_K + operand conversion in one pass: the same bits as the three separate launches."""
    d, ff, ne, nu, n = 512, 512, 4, 2, 70
    _, pool = _pool(d, ff, ne, gate_fmt, seed=9)
    rng = np.random.default_rng(4)
    norms, logits = to_dev(rng.standard_normal((n, d)).astype(np.float32)), to_dev(rng.standard_normal((n, ne)).astype(np.float32))
    sc = P.make_chunk_scratch(pool, n, nu)
    apart = P.dk_ffn_routed_chunk(pool, norms, logits, nu, 7.0, sc, fused=False).clone()
    mh, me, ms = sc.mh.clone(), sc.me.clone(), sc.midq.xs.clone()
    sc.mh.zero_(), sc.me.fill_(3.0), sc.midq.xs.zero_()
    fused = P.dk_ffn_routed_chunk(pool, norms, logits, nu, 7.0, sc, fused=True)
    assert torch.equal(sc.mh, mh) and torch.equal(sc.me, me) and torch.equal(sc.midq.xs, ms)
    assert torch.equal(fused, apart)
