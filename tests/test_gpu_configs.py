"""Parity at the sizes the benchmark times: the kernels take other planner branches there
(wider rows, more lanes a row, more stages, many tiles per CTA) than at the small shapes of
the other GPU tests.

Matrices too large to multiply whole on the CPU are drawn on the device; the rows (or the
experts) a check needs are copied back and given to the oracle.
"""
import numpy as np
import pytest
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from illatio_b200 import cuda_ds4f_prefill as P
from illatio_b200 import microbench_moe as MB
from gpu_util import act_to_host, dev_act, rel_errors, sum_terms, to_dev

pytestmark = pytest.mark.gpu
TOL_SPEC = 2e-3      # max relative error the path is specified to (against max|ref|)
TOL_TERMS = 2e-6     # per row against sum|terms|: fp32 reassociation only
VOCAB = 151936


@pytest.fixture(autouse=True)
def _need_gpu(cuda_lib):
    assert torch.cuda.is_available()
    yield
    assert D.device_status() == 0


@pytest.mark.parametrize("fmt,cols", [(B.Q8_0, 896), (B.Q4_K, 2560), (B.Q6_K, 2560), (B.Q6_K, 5120), (B.Q2_K, 5120),
                                      (B.IQ2_XXS, 4096)])
def test_head_sized_matrix_sampled_rows(oracle, fmt, cols):
    """A 151936-row matrix per format (the output heads of the configurations): 512 sampled rows against
    the oracle, and the whole output finite."""
    wd = B.synth_matrix_torch(fmt, VOCAB, cols, seed=40 + fmt)
    w = D.CMat("head", fmt, VOCAB, cols, wd)
    x = np.random.default_rng(fmt).standard_normal(cols).astype(np.float32)
    act = dev_act(fmt, x)
    y = torch.full((VOCAB + 8,), 7.0, dtype=torch.float32, device="cuda")
    D.cmat_mul(w, act, y, 1)
    got = y.cpu().numpy()
    assert (got[VOCAB:] == 7.0).all() and np.isfinite(got).all()
    rng = np.random.default_rng(1)
    rows = np.unique(np.concatenate([[0, 1, VOCAB - 1, VOCAB - 2], rng.integers(0, VOCAB, 508)]))
    rb = B.row_bytes(fmt, cols)
    sub = wd.view(VOCAB, rb)[torch.as_tensor(rows).cuda()].cpu().numpy().reshape(-1)
    ah = act_to_host(act)
    want = oracle.matvec(fmt, sub, len(rows), cols, ah, threads=4)[0]
    a, b = rel_errors(got[rows], want, sum_terms(oracle, fmt, sub, len(rows), cols, ah)[0])
    assert a < TOL_SPEC and a < 1e-5, (B.NAMES[fmt], a)
    assert b < TOL_TERMS, (B.NAMES[fmt], b)


@pytest.mark.parametrize("n", [1, 4, 16])
def test_q6k_17408x5120_batches(oracle, n):
    """The 27B-scale FFN matrix of the Q6_K sweep, whole, at batch 1, 4 and 16."""
    rows, cols = 17408, 5120
    wb = B.synth_matrix(B.Q6_K, rows, cols, seed=17)
    w = D.upload_gmat(wb, B.Q6_K, rows, cols)
    x = np.random.default_rng(n).standard_normal(n * cols).astype(np.float32)
    act = dev_act(B.Q6_K, x)
    y = torch.zeros(n * rows, dtype=torch.float32, device="cuda")
    D.cmat_mul(w, act, y, n)
    want = oracle.matvec(B.Q6_K, wb, rows, cols, act_to_host(act), n=n, threads=8)
    a, _ = rel_errors(y.cpu().numpy().reshape(n, rows), want)
    assert a < TOL_SPEC and a < 1e-5, a


def test_q6k_5120x17408_long_rows(oracle):
    """Rows of 17408 columns (the down projection of the sweep): 68 blocks a row."""
    rows, cols = 5120, 17408
    wb = B.synth_matrix(B.Q6_K, rows, cols, seed=18)
    w = D.upload_gmat(wb, B.Q6_K, rows, cols)
    act = dev_act(B.Q6_K, np.random.default_rng(2).standard_normal(cols).astype(np.float32))
    y = torch.zeros(rows, dtype=torch.float32, device="cuda")
    D.cmat_mul(w, act, y, 1)
    want = oracle.matvec(B.Q6_K, wb, rows, cols, act_to_host(act), threads=8)[0]
    a, _ = rel_errors(y.cpu().numpy(), want)
    assert a < TOL_SPEC and a < 1e-5, a


def test_gated_q4k_9728x2560(oracle):
    """The 4B model's gate / up product (the kernel the benchmark's roofline entry names), whole."""
    rows, cols = 9728, 2560
    g, u = (B.synth_matrix(B.Q4_K, rows, cols, seed=s) for s in (31, 32))
    act = dev_act(B.Q4_K, np.random.default_rng(3).standard_normal(cols).astype(np.float32) * 0.05)
    fa = torch.zeros(rows, dtype=torch.float32, device="cuda")
    D.glu_mul(D.upload_gmat(g, B.Q4_K, rows, cols), D.upload_gmat(u, B.Q4_K, rows, cols), act, fa)
    ah = act_to_host(act)
    gv = oracle.matvec(B.Q4_K, g, rows, cols, ah, threads=8)[0].astype(np.float64)
    uv = oracle.matvec(B.Q4_K, u, rows, cols, ah, threads=8)[0].astype(np.float64)
    with np.errstate(over="ignore"):
        want = gv / (1 + np.exp(-gv)) * uv
    a, _ = rel_errors(fa.cpu().numpy(), want)
    assert a < TOL_SPEC and a < 1e-5, a


def _check_chunk(oracle, cfg, n_tok, n_check, clamp, seed, driver=None):
    """One chunk of N_TOK tokens through every expert of CFG; N_CHECK sampled tokens against the oracle's
    routed-expert layer, which is given only those tokens' experts (copied back from the device)."""
    pool = MB.make_pool(cfg, seed=seed)
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    norms = torch.randn(n_tok, cfg["d"], device="cuda", generator=g)
    logits = MB.router_logits(cfg, n_tok, seed=seed + 2)
    sc = P.make_chunk_scratch(pool, n_tok, cfg["nu"])
    moe = (driver or P.dk_ffn_routed_chunk)(pool, norms, logits, cfg["nu"], clamp, sc)
    torch.cuda.synchronize()
    counts = sc.counts.cpu().numpy()
    sel_d = sc.sel.cpu().numpy()
    osel, ow = oracle.route(logits.cpu().numpy(), cfg["nu"], mode=2)
    assert (sel_d == osel).mean() > 0.995   # expf's last place can swap two near-equal experts
    # sampled tokens: the first and last, some that use the fullest expert, the rest at random
    rng = np.random.default_rng(seed)
    busiest = int(counts.argmax())
    users = np.nonzero((osel == busiest).any(1))[0]
    toks = np.unique(np.concatenate([[0, n_tok - 1], users[:6], rng.integers(0, n_tok, n_check)]))[:n_check]
    toks = np.array([t for t in toks if np.array_equal(sel_d[t], osel[t])])
    d, ff, nu = cfg["d"], cfg["ff"], cfg["nu"]
    gb, db = pool.gate_bytes, pool.down_bytes
    slots = pool.pool.view(pool.n_expert, pool.slot_bytes)
    got = moe[torch.as_tensor(toks).cuda()].cpu().numpy()
    norms_h = norms[torch.as_tensor(toks).cuda()].cpu().numpy()
    worst = 0.0
    for i, t in enumerate(toks):
        mine = slots[torch.as_tensor(osel[t].astype(np.int64)).cuda()].cpu().numpy()   # [nu, slot]: this token's experts only
        gate = np.ascontiguousarray(mine[:, :gb]).reshape(-1)
        up = np.ascontiguousarray(mine[:, gb:2 * gb]).reshape(-1)
        down = np.ascontiguousarray(mine[:, 2 * gb:2 * gb + db]).reshape(-1)
        want = oracle.moe_routed(d, ff, cfg["gate_fmt"], B.Q2_K, gate, up, down, norms_h[i], np.arange(nu, dtype=np.int32),
                                 ow[t], clamp, threads=8)
        worst = max(worst, float(np.abs(got[i] - want).max() / np.abs(want).max()))
    return worst, counts, len(toks)


def test_c4_chunk_4096_tokens(oracle):
    """DeepSeek-V4-Flash-shaped layer as the benchmark runs it: hidden 4096, 256 experts of FFN 2048, top-6,
    IQ2_XXS gate / up, Q2_K down, one 4096-token chunk (8192 tiles a launch, 16 blocks of K)."""
    worst, counts, checked = _check_chunk(oracle, MB.CONFIGS["c4"], 4096, 32, 10.0, seed=5)
    assert counts.sum() == 4096 * 6 and checked >= 24
    assert worst < TOL_SPEC, worst
    print("c4 chunk: worst relative error %.3g over %d tokens, rows per expert max %d" % (worst, checked, counts.max()))


def test_c5_chunk_zipf_2048_tokens(oracle):
    """GLM-style layer: hidden 5120, 288 experts of FFN 1536, top-8, Q2_K throughout, Zipf(1.1) popularity --
    the popular experts get several tiles of rows, the rare ones none."""
    worst, counts, checked = _check_chunk(oracle, MB.CONFIGS["c5"], 2048, 32, 10.0, seed=6)
    assert counts.sum() == 2048 * 8 and counts.max() > 128 and checked >= 24
    assert worst < TOL_SPEC, worst
    print("c5 chunk: worst relative error %.3g over %d tokens, rows per expert max %d" % (worst, checked, counts.max()))


def test_c5_small_batch_64_sequences(oracle):
    """DK-FFN-SMALL at configs[4]'s decode shape: 64 sequences' tokens x top-8 of 288 experts (Zipf), rows grouped by
    expert; twelve tokens against the oracle, and four against the one-token driver (DK-FFN-TAIL)."""
    cfg = MB.CONFIGS["c5"]
    worst, counts, checked = _check_chunk(oracle, cfg, 64, 12, 10.0, seed=8, driver=P.dk_ffn_small)
    assert counts.sum() == 64 * 8 and checked >= 8
    assert worst < TOL_SPEC, worst
    from illatio_b200 import cuda_ds4f as M
    pool = MB.make_pool(cfg, seed=8)
    g = torch.Generator(device="cuda").manual_seed(9)
    norms = torch.randn(64, cfg["d"], device="cuda", generator=g)
    logits = MB.router_logits(cfg, 64, seed=10)
    sc = P.make_chunk_scratch(pool, 64, cfg["nu"])
    moe = P.dk_ffn_small(pool, norms, logits, cfg["nu"], 10.0, sc).clone()
    sel, w = M.route(logits, cfg["nu"], mode=2)
    for t in (0, 17, 42, 63):
        one, _ = M.dk_ffn_tail(pool, norms[t], sel[t], w[t], 10.0)
        assert ((moe[t] - one).abs().max() / one.abs().max()).item() < TOL_SPEC
    print("c5 small batch: worst relative error %.3g over %d tokens" % (worst, checked))


def test_c5_small_batch_matvec_path(oracle):
    """DK-FFN-SMALL on the one-token kernels (ill_moe_row_ptrs: an expert's rows next to each other): the same 64 x
    top-8 batch against the oracle, and token by token the very bits of the one-token driver (DK-FFN-TAIL), whose
    kernels and order of sums it shares."""
    cfg = MB.CONFIGS["c5"]
    worst, counts, checked = _check_chunk(oracle, cfg, 64, 12, 10.0, seed=8, driver=P.dk_ffn_small_mv)
    assert counts.sum() == 64 * 8 and checked >= 8
    assert worst < TOL_SPEC, worst
    from illatio_b200 import cuda_ds4f as M
    pool = MB.make_pool(cfg, seed=8)
    g = torch.Generator(device="cuda").manual_seed(9)
    norms = torch.randn(64, cfg["d"], device="cuda", generator=g)
    logits = MB.router_logits(cfg, 64, seed=10)
    sc = P.make_chunk_scratch(pool, 64, cfg["nu"])
    moe = P.dk_ffn_small_mv(pool, norms, logits, cfg["nu"], 10.0, sc).clone()
    sel, w = M.route(logits, cfg["nu"], mode=2)
    for t in (0, 17, 42, 63):
        one, _ = M.dk_ffn_tail(pool, norms[t], sel[t], w[t], 10.0)
        assert torch.equal(moe[t], one), (t, (moe[t] - one).abs().max().item())
    assert D.device_status() == 0
    print("c5 small batch, matvec path: worst relative error %.3g over %d tokens" % (worst, checked))
