"""Dense products for a chunk of tokens (CMAT-MUL-N with more than 16 tokens: src/cuda-dense.lisp:220-255) --
the tensor cores' int8 kernel against the one-token product, token by token (the one-token product is what the
other tests hold against the CPU oracle, bit for bit in its integer sums), and against the oracle directly."""
import numpy as np
import pytest
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu(cuda_lib):
    assert torch.cuda.is_available()
    yield
    assert D.device_status() == 0


def _case(fmt, rows, cols, n, seed=0):
    w = D.CMat("w", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=seed))
    x = torch.randn(n * cols, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed + 1))
    act = D.quant_q8(x, D.make_qact(n * cols, D.matrix_act_kind(w)))
    return w, x, act


@pytest.mark.parametrize("fmt,rows,cols,n", [
    (B.Q4_K, 300, 512, 17), (B.Q4_K, 1000, 2560, 33), (B.Q4_K, 2560, 9728, 100), (B.Q4_K, 9728, 2560, 512),
    (B.Q6_K, 300, 768, 20), (B.Q6_K, 2560, 5120, 64), (B.Q6_K, 1031, 17408, 130), (B.Q6_K, 5120, 5120, 512),
    (B.Q8_0, 300, 896, 17), (B.Q8_0, 4864, 896, 96), (B.Q8_0, 896, 4864, 200), (B.Q8_0, 151936, 896, 40),
    # a few tokens of rows too long to keep their activations beside the weights: the columns dealt to a CTA's warps
    (B.Q6_K, 300, 17408, 4), (B.Q6_K, 1031, 17408, 16), (B.Q4_K, 250, 19456, 9), (B.Q8_0, 300, 17408, 16), (B.Q8_0, 40, 17280, 3),
])
def test_chunk_product_equals_token_by_token(fmt, rows, cols, n):
    w, x, act = _case(fmt, rows, cols, n)
    y = torch.full((n * rows,), -3.0, device="cuda")
    D.cmat_mul(w, act, y, n)
    want = torch.empty(n * rows, device="cuda")
    for t in range(n):   # one token at a time through the matvec kernel
        a1 = D.quant_q8(x[t * cols:(t + 1) * cols], D.make_qact(cols, D.matrix_act_kind(w)))
        D.cmat_mul(w, a1, want[t * rows:(t + 1) * rows], 1)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    # the integer sums are the same; the blocks' float terms are added in a different order (a row whole here,
    # lanes' partial sums in the one-token kernel)
    err = ((y - want).abs().max() / want.abs().max()).item()
    assert err < 2e-6, err


@pytest.mark.parametrize("fmt", [B.Q8_0, B.Q4_K, B.Q6_K])
def test_chunk_product_against_the_oracle(oracle, fmt):
    rows, cols, n = 200, 1024, 70
    wb = B.synth_matrix(fmt, rows, cols, seed=4)
    w = D.upload_gmat(wb, fmt, rows, cols)
    rng = np.random.default_rng(6)
    xh = rng.standard_normal((n, cols)).astype(np.float32)
    act = D.quant_q8(to_dev(xh.reshape(-1)), D.make_qact(n * cols, D.matrix_act_kind(w)))
    bias = to_dev(rng.standard_normal(rows).astype(np.float32))
    y = torch.zeros(n * rows, device="cuda")
    D.cmat_mul(w, act, y, n, bias=bias)
    torch.cuda.synchronize()
    got = y.cpu().numpy().reshape(n, rows)
    for t in (0, 1, 37, n - 1):
        want = oracle.matvec(fmt, wb, rows, cols, oracle.quantize_act(fmt, xh[t]), bias=bias.cpu().numpy())[0]
        assert np.abs(got[t] - want).max() / np.abs(want).max() < 2e-6
    # added into Y when ACC
    y2 = y.clone()
    D.cmat_mul(w, act, y2, n, acc=True)
    torch.cuda.synchronize()
    assert ((y2 - 2 * y + bias.repeat(n)).abs().max() / y.abs().max()).item() < 1e-5


def test_ffn_head_chunk_against_the_oracle(oracle):
    """DK-FFN-HEAD-CHUNK: RMSNorm, the router's logits and the shared expert over a chunk, token by token against
    the CPU routines (RMSNORM!, F32MV! on the widened router, D4-SHARED!)."""
    from illatio_b200 import cuda_ds4f_prefill as P
    n, d, ff, ne, clamp, eps = 70, 1024, 512, 64, 10.0, 1e-6
    rng = np.random.default_rng(11)
    mats = [B.synth_matrix(B.Q8_0, r, c, seed=20 + i) for i, (r, c) in enumerate(((ff, d), (ff, d), (d, ff)))]
    ws = [D.upload_gmat(m, B.Q8_0, r, c) for m, (r, c) in zip(mats, ((ff, d), (ff, d), (d, ff)))]
    router = torch.as_tensor(rng.standard_normal((ne, d)).astype(np.float32) * 0.05).to(torch.float16)
    cur = rng.standard_normal((n, d)).astype(np.float32)
    nw = (rng.random(d) + 0.5).astype(np.float32)
    hs = P.HeadScratch(n + 3, d, ff, ne)
    norm2, logits, sout = P.dk_ffn_head_chunk(to_dev(cur), to_dev(nw), eps, router.cuda(), ws[0], ws[1], ws[2], clamp, hs)
    torch.cuda.synchronize()
    norm2, logits, sout = norm2.cpu().numpy(), logits.cpu().numpy(), sout.cpu().numpy()
    rf = router.to(torch.float32).numpy()
    for t in (0, 16, 33, n - 1):
        want_n = oracle.rmsnorm(cur[t], nw, eps)
        assert np.abs(norm2[t] - want_n).max() <= 1e-6 * np.abs(want_n).max()
        want_l = oracle.f32mv(rf, norm2[t])
        terms = np.abs(rf.astype(np.float64) * norm2[t].astype(np.float64)).sum(1)
        assert (np.abs(logits[t] - want_l) <= 1e-6 * terms + 1e-30).all()
        want_s = oracle.moe_shared(d, ff, mats[0], mats[1], mats[2], norm2[t], clamp, threads=2)
        assert np.abs(sout[t] - want_s).max() / np.abs(want_s).max() < 2e-3


@pytest.mark.parametrize("fmt,rows,cols,n", [(B.Q4_K, 300, 512, 40), (B.Q4_K, 1000, 2560, 130), (B.Q4_K, 9728, 2560, 512),
                                             (B.Q4_K, 2560, 9728, 200), (B.Q6_K, 300, 768, 40), (B.Q6_K, 1031 - 3, 2560, 130),
                                             (B.Q6_K, 2560, 9728, 512), (B.Q6_K, 5120, 5120, 200)])
def test_chunk_on_tcgen05_equals_token_by_token(fmt, rows, cols, n):
    """The same chunk product through the tcgen05 kernel (the expert product with the matrix as its one expert):
    integer operands exact in fp16 (Q6_K's products as an even and an odd part), fp32 accumulation in tensor memory,
    the blocks scaled as they are drained."""
    w, x, act = _case(fmt, rows, cols, n, seed=3)
    cf = D.ChunkF16(n, cols).fill(act)
    y = torch.full((n * rows,), -3.0, device="cuda")
    D.cmat_mul_tc(w, cf, y)
    want = torch.empty(n * rows, device="cuda")
    one = D.make_qact(cols, "q8k")
    for t in range(n):   # one token at a time through the matvec kernel
        D.cmat_mul(w, D.quant_q8(x[t * cols:(t + 1) * cols], one), want[t * rows:(t + 1) * rows], 1)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    err = ((y - want).abs().max() / want.abs().max()).item()
    assert err < 2e-6, err
    # added into Y when asked; and cmat_mul takes this path by itself for chunks of large matrices
    y2 = y.clone()
    D.cmat_mul_tc(w, cf, y2, acc=True)
    y3 = torch.empty_like(y)
    D.cmat_mul(w, act, y3, n)
    torch.cuda.synchronize()
    assert torch.equal(y2, y + y)
    if rows >= D.TC_MIN_ROWS and n >= D.TC_MIN_TOKENS:
        assert torch.equal(y3, y)


@pytest.mark.parametrize("fmt", [B.Q4_K, B.Q6_K])
def test_chunk_on_tcgen05_against_the_oracle(oracle, fmt):
    rows, cols, n = 200, 1024, 70
    wb = B.synth_matrix(fmt, rows, cols, seed=4)
    w = D.upload_gmat(wb, fmt, rows, cols)
    rng = np.random.default_rng(6)
    xh = rng.standard_normal((n, cols)).astype(np.float32)
    act = D.quant_q8(to_dev(xh.reshape(-1)), D.make_qact(n * cols, "q8k"))
    y = torch.zeros(n * rows, device="cuda")
    D.cmat_mul_tc(w, D.ChunkF16(n, cols).fill(act), y)
    torch.cuda.synchronize()
    got = y.cpu().numpy().reshape(n, rows)
    for t in (0, 1, 37, n - 1):
        want = oracle.matvec(fmt, wb, rows, cols, oracle.quantize_act(fmt, xh[t]))[0]
        assert np.abs(got[t] - want).max() / np.abs(want).max() < 2e-6


def test_fused_swiglu_into_the_down_product():
    """SwiGLU, Q8_K and the fp16 form in one launch (swiglu_chunk_f16) feed the tcgen05 down product with the same
    bits as the three steps apart."""
    n, ff, rows = 130, 2560, 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    ga, ub = torch.randn(n * ff, device="cuda", generator=g), torch.randn(n * ff, device="cuda", generator=g)
    w = D.CMat("down", B.Q6_K, rows, ff, B.synth_matrix_torch(B.Q6_K, rows, ff, seed=2))
    assert D.tc_takes(w, n)
    y1 = torch.zeros(n * rows, device="cuda")
    D.cmat_mul_tc(w, D.swiglu_chunk_f16(ga, ub, D.ChunkF16(n, ff)), y1)
    mid = torch.empty_like(ga)
    D.swiglu(ga, ub, mid, ff)
    y2 = torch.zeros(n * rows, device="cuda")
    D.cmat_mul(w, D.quant_q8(mid, D.make_qact(n * ff, "q8k")), y2, n)
    torch.cuda.synchronize()
    assert torch.isfinite(y1).all() and torch.equal(y1, y2)


def test_vanishing_block_is_quantized_to_zeros(oracle):
    """A Q8_K block whose largest magnitude is below 3.8e-37 (-127 / max overflows: the reference's arithmetic is not
    defined there) is taken as zeros by the device quantizers and by the oracle alike -- and the fused SwiGLU step,
    where such blocks arise (silu of a very negative gate), hands the tcgen05 product finite operands."""
    x = np.zeros(768, np.float32)
    x[256:512] = np.float32(1e-40) * np.arange(1, 257, dtype=np.float32)   # denormals
    x[512:] = np.linspace(-1, 1, 256, dtype=np.float32)
    act = D.quant_q8(to_dev(x), D.make_qact(768, "q8k"))
    torch.cuda.synchronize()
    q, d, bs = oracle.quantize_q8k(x)
    assert np.array_equal(act.xq.cpu().numpy(), q) and np.array_equal(act.xs.cpu().numpy(), d)
    assert np.array_equal(act.xsum.cpu().numpy().astype(np.int32), bs)
    assert d[0] == 0 and d[1] == 0 and d[2] != 0 and not q[:512].any() and q[512:].any()
    # gates of -95 (e^-95 is a denormal) against ups of one: every middle value is a denormal
    n, ff = 64, 512
    g = torch.full((n * ff,), -95.0, device="cuda")
    u = torch.ones(n * ff, device="cuda")
    cf = D.swiglu_chunk_f16(g, u, D.ChunkF16(n, ff))
    torch.cuda.synchronize()
    assert torch.isfinite(cf.xh.float()).all() and (cf.xh == 0).all() and (cf.xd == 0).all()


@pytest.mark.parametrize("fmt", [B.Q4_K, B.Q6_K])
def test_gate_and_up_in_one_launch(fmt):
    """ill_mm_chunk2: two matrices against the same chunk in one launch give what two launches give, bit for bit."""
    rows, cols, n = 2048 + 128, 1024, 200
    wg, x, act = _case(fmt, rows, cols, n, seed=7)
    wu = D.CMat("u", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=8))
    fa, fb = torch.empty(n * rows, device="cuda"), torch.empty(n * rows, device="cuda")
    D.glu_mul_tc(wg, wu, act, n, fa, fb)
    ya, yb = torch.empty_like(fa), torch.empty_like(fb)
    D.cmat_mul(wg, act, ya, n)
    D.cmat_mul(wu, act, yb, n)
    torch.cuda.synchronize()
    assert torch.equal(fa, ya) and torch.equal(fb, yb) and torch.isfinite(fa).all()


def test_quantizers_that_also_leave_the_fp16_forms():
    """Once an activation buffer's fp16 form is in use (a chunk went to the tcgen05 kernel), quant_q8 and rmsnorm_q8
    renew it in their own launch: the same bytes, the same halves as ill_act_f16 makes."""
    n, cols = 96, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    w = D.CMat("w", B.Q4_K, 2048, cols, B.synth_matrix_torch(B.Q4_K, 2048, cols, seed=1))
    nw = torch.rand(cols, device="cuda", generator=g) + 0.5
    for norm in (False, True):
        act, ref = D.make_qact(n * cols, "q8k"), D.make_qact(n * cols, "q8k")
        y = torch.empty(n * 2048, device="cuda")
        outs = []
        for it in range(2):   # first pass: the fp16 form is made by ill_act_f16; second: by the quantizer itself
            x = torch.randn(n * cols, device="cuda", generator=g)
            if norm:
                D.rmsnorm_q8(x, nw, act, cols, 1e-6, n=n)
                D.rmsnorm_q8(x, nw, ref, cols, 1e-6, n=n)
            else:
                D.quant_q8(x, act)
                D.quant_q8(x, ref)
            assert bool(getattr(act, "_cf_fresh", False)) == (it == 1)
            D.cmat_mul(w, act, y, n)
            fresh = D.ChunkF16(n, cols).fill(ref)     # ref never goes to the tensor-core path: plain quantizer + ill_act_f16
            torch.cuda.synchronize()
            assert torch.equal(act.xq, ref.xq) and torch.equal(act.xs, ref.xs) and torch.equal(act.xsum, ref.xsum)
            assert torch.equal(act._cf.xh, fresh.xh) and torch.equal(act._cf.xe, fresh.xe)
            outs.append(y.clone())
        assert torch.isfinite(outs[1]).all()
