"""Parity of the decode path on a B200 against the CPU oracle, through the C ABI.

Bit-exact: activation quantizers, dequantized rows.  Products: the integer
block dots are exact on both sides, so outputs differ only by fp32 summation
order; the bound asserted is far inside the 2e-3 the path is specified to.
"""
import os

import numpy as np
import pytest
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from gpu_util import act_to_host, dev_act, rel_errors, sum_terms, to_dev

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FMTS = list(range(5))
TOL_SPEC = 2e-3      # max relative error the path is specified to (vs max|ref|)
TOL_TERMS = 2e-6     # per row, relative to sum|terms|: fp32 reassociation only


@pytest.fixture(autouse=True)
def _need_gpu(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield
    assert D.device_status() == 0


def test_quant_q8_0_bit_exact(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(32 * 4099).astype(np.float32)
    x[64:96] = 0.0
    x[96:128] = [0.5 * (i - 16) for i in range(32)]  # exact halves: ties to even
    x[128:160] *= 1e-30
    x[160:192] *= 1e30
    for f16 in (True, False):
        act = D.make_qact(x.size, "q8", want_xsum=True)
        D.quant_q8(to_dev(x), act, f16_scale=f16)
        q, s = oracle.quantize_q8_0(x, f16_scale=f16)
        assert np.array_equal(act.xq.cpu().numpy(), q)
        assert np.array_equal(act.xs.cpu().numpy().view(np.uint32), s.view(np.uint32))
        assert np.array_equal(act.xsum.cpu().numpy(), q.reshape(-1, 32).astype(np.int32).sum(1))


def test_quant_q8_k_bit_exact(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal(256 * 1031).astype(np.float32)
    x[256:512] = 0.0
    x[512] = 3.0
    x[513] = -3.0
    x[514:768] *= 0.1
    x[768:1024] *= 1e-20
    x[1024:1280] = np.round(x[1024:1280] * 4) / 4  # many equal magnitudes
    act = D.make_qact(x.size, "q8k")
    D.quant_q8(to_dev(x), act)
    q, d, bs = oracle.quantize_q8k(x)
    assert np.array_equal(act.xq.cpu().numpy(), q)
    assert np.array_equal(act.xs.cpu().numpy().view(np.uint32), d.view(np.uint32))
    assert np.array_equal(act.xsum.cpu().numpy().astype(np.int32), bs)


@pytest.mark.parametrize("kind,d,n", [("q8", 896, 1), ("q8k", 2560, 1), ("q8k", 5120, 5), ("q8", 4864, 3)])
def test_rmsnorm_q8_matches_oracle(oracle, kind, d, n):
    """RMSNorm fused with the quantizer: the normalized floats, the quants and the scales of the CPU routines."""
    rng = np.random.default_rng(d + n)
    x = (rng.standard_normal((n, d)) * rng.uniform(0.01, 30.0, (n, 1))).astype(np.float32)
    w = rng.standard_normal(d).astype(np.float32)
    act = D.make_qact(n * d, kind, want_xsum=True)
    h = torch.empty(n, d, device="cuda")
    D.rmsnorm_q8(to_dev(x), to_dev(w), act, d, 1e-6, n, h=h)
    want = np.stack([oracle.rmsnorm(x[t], w, 1e-6) for t in range(n)])
    assert np.array_equal(h.cpu().numpy().view(np.uint32), want.view(np.uint32))
    if kind == "q8":
        q, s = oracle.quantize_q8_0(want)
        assert np.array_equal(act.xsum.cpu().numpy(), q.reshape(-1, 32).astype(np.int32).sum(1))
    else:
        q, s, bs = oracle.quantize_q8k(want)
        assert np.array_equal(act.xsum.cpu().numpy().astype(np.int32), bs)
    assert np.array_equal(act.xq.cpu().numpy(), q)
    assert np.array_equal(act.xs.cpu().numpy().view(np.uint32), s.view(np.uint32))


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_rows_bit_exact_golden(fmt):
    z = np.load(os.path.join(GOLD, "dequant_%s.npz" % B.NAMES[fmt]))
    blk, want = z["blocks"], z["floats"]
    cols = B.BLOCK_WEIGHTS[fmt] * 4
    rows = blk.shape[0] // 4
    w = D.upload_gmat(blk.reshape(-1), fmt, rows, cols)
    got = D.dequant_rows(w, 0, rows).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.reshape(rows, cols).view(np.uint32))


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_rows_bit_exact_random_and_embed(oracle, fmt):
    rows, cols = 300, B.BLOCK_WEIGHTS[fmt] * 9
    wb = B.synth_matrix(fmt, rows, cols, seed=50 + fmt)
    w = D.upload_gmat(wb, fmt, rows, cols)
    want = oracle.dequant(fmt, wb, rows, cols)
    got = D.dequant_rows(w, 0, rows).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ids = np.array([5, 299, 0, 5, 123], np.int32)
    x = torch.empty(len(ids), cols, dtype=torch.float32, device="cuda")
    D.embed(w, to_dev(ids), x)
    assert np.array_equal(x.cpu().numpy().view(np.uint32), want[ids].view(np.uint32))


# (rows, cols): model shapes of the configurations plus ragged ones -- one
# block / super-block per row, one row, rows not a multiple of anything
SHAPES = {
    B.Q8_0: [(896, 896), (128, 896), (4864, 896), (896, 4864), (1, 32), (5, 64), (1031, 160)],
    B.Q4_K: [(4096, 2560), (1024, 2560), (2560, 4096), (1, 256), (3, 512), (777, 768),
             (11700, 2560)],  # past 16 MB the plan changes (eight lanes a row, five units a lane)
    B.Q6_K: [(1024, 2560), (2560, 9728), (5120, 5120), (1, 256), (5, 256), (333, 1280), (64, 17408)],
    B.Q2_K: [(4096, 2048), (1536, 5120), (5120, 1536), (1, 256), (7, 512)],
    B.IQ2_XXS: [(2048, 4096), (1, 256), (9, 512), (515, 1024)],
}


@pytest.mark.parametrize("fmt", FMTS)
def test_mv_matches_oracle(oracle, fmt):
    for k, (rows, cols) in enumerate(SHAPES[fmt]):
        wb = B.synth_matrix(fmt, rows, cols, seed=100 * fmt + k)
        x = np.random.default_rng(k).standard_normal(cols).astype(np.float32)
        w = D.upload_gmat(wb, fmt, rows, cols)
        act = dev_act(fmt, x)
        y = torch.full((rows + 8,), 7.0, dtype=torch.float32, device="cuda")  # canary words after the output
        D.cmat_mul(w, act, y, 1)
        ah = act_to_host(act)
        want = oracle.matvec(fmt, wb, rows, cols, ah, threads=4)[0]
        got = y.cpu().numpy()
        assert (got[rows:] == 7.0).all(), "wrote past the output"
        a, b = rel_errors(got[:rows], want, sum_terms(oracle, fmt, wb, rows, cols, ah)[0])
        assert a < TOL_SPEC and a < 1e-5, (B.NAMES[fmt], rows, cols, a)
        assert b < TOL_TERMS, (B.NAMES[fmt], rows, cols, b)


@pytest.mark.parametrize("fmt", FMTS)
def test_mv_unaligned_base_bias_acc(oracle, fmt):
    """The matrix at an odd byte offset inside a buffer; bias and accumulate."""
    rows, cols = 130, B.BLOCK_WEIGHTS[fmt] * 3
    wb = B.synth_matrix(fmt, rows, cols, seed=7 + fmt)
    for shift in (2, 6, 14):
        buf = torch.zeros(wb.size + 64, dtype=torch.uint8, device="cuda")
        buf[shift:shift + wb.size] = to_dev(wb)
        w = D.CMat("shifted", fmt, rows, cols, buf[shift:shift + wb.size])
        x = np.random.default_rng(shift).standard_normal(cols).astype(np.float32)
        act = dev_act(fmt, x)
        bias = np.random.default_rng(1).standard_normal(rows).astype(np.float32)
        y0 = np.random.default_rng(2).standard_normal(rows).astype(np.float32)
        y = to_dev(y0)
        D.cmat_mul(w, act, y, 1, bias=to_dev(bias), acc=True)
        want = oracle.matvec(fmt, wb, rows, cols, act_to_host(act), bias=bias)[0] + y0
        a, _ = rel_errors(y.cpu().numpy(), want)
        assert a < 1e-5, (B.NAMES[fmt], shift, a)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("n", [2, 4, 7, 16, 19])
def test_mv_several_tokens(oracle, fmt, n):
    rows, cols = 257, B.BLOCK_WEIGHTS[fmt] * 5
    wb = B.synth_matrix(fmt, rows, cols, seed=3 + fmt)
    x = np.random.default_rng(n).standard_normal(n * cols).astype(np.float32)
    w = D.upload_gmat(wb, fmt, rows, cols)
    act = dev_act(fmt, x)
    y = torch.zeros(n * rows, dtype=torch.float32, device="cuda")
    D.cmat_mul(w, act, y, n)
    want = oracle.matvec(fmt, wb, rows, cols, act_to_host(act), n=n)
    a, _ = rel_errors(y.cpu().numpy().reshape(n, rows), want)
    assert a < 1e-5, (B.NAMES[fmt], n, a)


@pytest.mark.parametrize("fmt", FMTS)
def test_qkv_and_glu(oracle, fmt):
    cols = B.BLOCK_WEIGHTS[fmt] * 4
    shapes = [(896, cols), (128, cols), (130, cols)]
    mats = [B.synth_matrix(fmt, r, c, seed=60 + i) for i, (r, c) in enumerate(shapes)]
    ws = [D.upload_gmat(m, fmt, r, c) for m, (r, c) in zip(mats, shapes)]
    x = np.random.default_rng(4).standard_normal(cols).astype(np.float32) * 0.05
    act = dev_act(fmt, x)
    ah = act_to_host(act)
    outs = [torch.zeros(r, dtype=torch.float32, device="cuda") for r, _ in shapes]
    biases = [np.random.default_rng(i).standard_normal(r).astype(np.float32) for i, (r, _) in enumerate(shapes)]
    D.qkv_mul(ws[0], ws[1], ws[2], act, outs[0], outs[1], outs[2], to_dev(biases[0]), None, to_dev(biases[2]))
    for i, (r, c) in enumerate(shapes):
        want = oracle.matvec(fmt, mats[i], r, c, ah, bias=None if i == 1 else biases[i])[0]
        a, _ = rel_errors(outs[i].cpu().numpy(), want)
        assert a < 1e-5, (B.NAMES[fmt], i, a)
    # GLU: silu(G x) * (U x) with silu(g) = g / (1 + exp(-g))
    rows = 515
    g = B.synth_matrix(fmt, rows, cols, seed=70)
    u = B.synth_matrix(fmt, rows, cols, seed=71)
    fa = torch.zeros(rows, dtype=torch.float32, device="cuda")
    D.glu_mul(D.upload_gmat(g, fmt, rows, cols), D.upload_gmat(u, fmt, rows, cols), act, fa)
    gv = oracle.matvec(fmt, g, rows, cols, ah)[0].astype(np.float64)
    uv = oracle.matvec(fmt, u, rows, cols, ah)[0].astype(np.float64)
    want = gv / (1 + np.exp(-gv)) * uv
    a, _ = rel_errors(fa.cpu().numpy(), want)
    assert a < 1e-5, (B.NAMES[fmt], a)


def test_errors_are_reported_not_raised_as_faults():
    from illatio_b200 import _lib
    w = D.upload_gmat(B.synth_matrix(B.Q4_K, 4, 256, seed=1), B.Q4_K, 4, 256)
    act = dev_act(B.Q4_K, np.ones(256, np.float32))
    y = torch.zeros(4, device="cuda")
    with pytest.raises(_lib.IllatioError):
        _lib.call("ill_mv", B.Q4_K, w.qs.data_ptr(), 4, 256, act.xq.data_ptr() + 1, act.xs.data_ptr(),
                  act.xsum.data_ptr(), y.data_ptr(), 0, 0, 1, None)
    with pytest.raises(ValueError):
        D.upload_gmat(np.zeros(100, np.uint8), B.Q4_K, 4, 250)
