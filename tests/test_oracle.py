"""The CPU oracle against its pins: gguf-py's dequantized floats (the fixtures
in tests/golden/), fp16 conversion against numpy, and the reference's own
row-dot criterion (inspect/iquant-test.lisp:45-53,61: |dot - exact| / sum|terms|
< 1e-6 against the float64 dot of the dequantized weights with the dequantized
activations)."""
import os

import numpy as np
import pytest

from illatio_b200 import blocks as B

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FMTS = list(range(5))


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_matches_golden(oracle, fmt):
    z = np.load(os.path.join(GOLD, "dequant_%s.npz" % B.NAMES[fmt]))
    blk, want = z["blocks"], z["floats"]
    bw = B.BLOCK_WEIGHTS[fmt]
    got = oracle.dequant(fmt, blk.reshape(-1), 1, blk.shape[0] * bw).reshape(-1, bw)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_matches_gguf_py_live(oracle, fmt):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    T = gguf.GGMLQuantizationType
    gg = {B.Q8_0: T.Q8_0, B.Q4_K: T.Q4_K, B.Q6_K: T.Q6_K, B.Q2_K: T.Q2_K, B.IQ2_XXS: T.IQ2_XXS}[fmt]
    nb = 20000
    blk = B.synth_blocks(fmt, nb, seed=77 + fmt)
    bw = B.BLOCK_WEIGHTS[fmt]
    got = oracle.dequant(fmt, blk.reshape(-1), 1, nb * bw).reshape(nb, bw)
    want = quants.dequantize(blk, gg).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_iq2xxs_tables_match_gguf_py(oracle):
    """The grid and sign tables (taken from the reference) against gguf-py's."""
    pytest.importorskip("gguf")
    from gguf import quants
    q = quants.IQ2_XXS
    q.init_grid()
    grid = np.asarray(q.grid).reshape(256, 8)
    # dequantize one block per grid index with d = 1, LS = 0, no signs: 0.125 * grid
    blk = np.zeros((256, 66), np.uint8)
    blk[:, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    blk[:, 2] = np.arange(256)
    got = oracle.dequant(B.IQ2_XXS, blk.reshape(-1), 256, 256)[:, :8]
    assert np.array_equal(got, grid.astype(np.float32) * 0.125)


def test_half_conversions(oracle):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.half_to_single(int(v)) for v in h[::7]], np.float32)
    w = want[::7]
    fin = np.isfinite(w)
    assert np.array_equal(got[fin].view(np.uint32), w[fin].view(np.uint32))
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 300.0, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.99e-8], np.float32)])
    with np.errstate(over="ignore"):
        want16 = xs.astype(np.float16).view(np.uint16)
    got16 = np.array([oracle.single_to_half(float(v)) for v in xs], np.uint16)
    assert np.array_equal(got16, want16)


def test_rmsnorm(oracle):
    """RMSNORM! (src/model.lisp:205-216): float squares summed in double, float scale, x scaled then weighted."""
    rng = np.random.default_rng(8)
    x = rng.standard_normal(2560).astype(np.float32) * 7
    w = rng.standard_normal(2560).astype(np.float32)
    eps = np.float32(1e-6)
    scale = np.float32(1) / np.sqrt(np.float32((x * x).astype(np.float64).sum() / 2560 + np.float64(eps)))
    assert np.array_equal(oracle.rmsnorm(x, w, eps), (x * scale) * w)
    assert np.allclose(oracle.rmsnorm(x, w, eps), x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6) * w,
                       rtol=1e-6, atol=1e-6)


def test_quantize_q8_0(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(32 * 64).astype(np.float32)
    x[32:64] = 0.0
    q, s = oracle.quantize_q8_0(x, f16_scale=False)
    amax = np.abs(x.reshape(-1, 32)).max(1)
    assert np.array_equal(s, (amax / np.float32(127.0)).astype(np.float32))
    assert (q[32:64] == 0).all() and s[1] == 0.0
    assert np.abs(q.reshape(-1, 32)).max(1)[0] == 127
    q2, s2 = oracle.quantize_q8_0(x, f16_scale=True)
    assert np.array_equal(q, q2)
    assert np.array_equal(s2, s.astype(np.float16).astype(np.float32))
    # round half to even: x/d exactly k + 0.5
    x = np.zeros(32, np.float32)
    x[0] = 127.0
    x[1:5] = [0.5, 1.5, 2.5, -2.5]
    q, _ = oracle.quantize_q8_0(x, f16_scale=False)
    assert list(q[:5]) == [127, 0, 2, 2, -2]


def test_quantize_q8_0_pinned_by_gguf_py(oracle):
    """QUANTIZE-Q8! with the fp16-rounded scale against gguf-py's Q8_0 `quantize` (the same ggml routine the
    reference's quantizer restates, src/tensor.lisp:245-262): identical fp16 scales, and identical quants
    except on exact .5 ties, which ggml rounds away from zero and the reference to even."""
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(32 * 4000) * rng.uniform(1e-3, 50.0, 32 * 4000)).astype(np.float32)
    x[:32] = 0.0
    x[32:64] = np.arange(32, dtype=np.float32) * 0.5 - 8.0  # a block full of exact ties (amax 8 -> id 15.875)
    blk = gguf.quants.quantize(x.reshape(-1, 32), gguf.GGMLQuantizationType.Q8_0).reshape(-1, 34)
    q, s = oracle.quantize_q8_0(x, f16_scale=True)
    want_d = blk[:, :2].copy().view(np.float16).astype(np.float32).reshape(-1)
    assert np.array_equal(s.view(np.uint32), want_d.view(np.uint32))
    want_q = blk[:, 2:].copy().view(np.int8).reshape(-1)
    d = np.abs(x.reshape(-1, 32)).max(1, keepdims=True) / np.float32(127)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1) / d).astype(np.float32)
    scaled = (x.reshape(-1, 32) * inv).reshape(-1)
    tie = np.abs(scaled - np.trunc(scaled)) == 0.5
    assert np.array_equal(q[~tie], want_q[~tie])
    assert tie.sum() < 64 and (np.abs(q[tie].astype(np.int32) - want_q[tie]) <= 1).all()
    assert (q[tie] % 2 == 0).all()  # the reference's ties go to even


def test_quantize_q8k(oracle):
    rng = np.random.default_rng(6)
    x = rng.standard_normal(256 * 8).astype(np.float32)
    x[256:512] = 0.0
    x[512] = 3.0
    x[513] = -3.0  # equal magnitudes: the first one sets the sign
    x[514:768] *= 0.1
    q, d, bs = oracle.quantize_q8k(x)
    assert d[1] == 0.0 and (q[256:512] == 0).all() and (bs[16:32] == 0).all()
    assert q[512] == -127 and q[513] == 127 and d[2] < 0
    assert np.array_equal(bs, q.reshape(-1, 16).astype(np.int32).sum(1))
    # the block's largest magnitude maps to -127 and d is the inverse of -127/max
    for b in (0, 3, 4):
        xb = x[256 * b:256 * (b + 1)]
        mx = xb[np.argmax(np.abs(xb))]
        isc = np.float32(-127.0) / np.float32(mx)
        assert d[b] == np.float32(1.0) / isc
        assert q[256 * b + np.argmax(np.abs(xb))] == -127


def _exact_dot(oracle, fmt, w, rows, cols, act):
    xq, xs, _ = act
    per = 32 if fmt == B.Q8_0 else 256
    xf = xq.astype(np.float64) * np.repeat(xs.astype(np.float64), per)
    wf = oracle.dequant(fmt, w, rows, cols).astype(np.float64)
    return wf @ xf, np.abs(wf) @ np.abs(xf)


@pytest.mark.parametrize("fmt", FMTS)
def test_row_dot_criterion(oracle, fmt):
    rows, cols = 64, 2048
    w = B.synth_matrix(fmt, rows, cols, seed=11 + fmt)
    rng = np.random.default_rng(7)  # U(-1,1), seed 7: inspect/iquant-test.lisp:37-38
    x = rng.uniform(-1, 1, cols).astype(np.float32)
    act = oracle.quantize_act(fmt, x)
    got = oracle.matvec(fmt, w, rows, cols, act)[0]
    exact, terms = _exact_dot(oracle, fmt, w, rows, cols, act)
    assert (np.abs(got - exact) / terms).max() < 1e-6


@pytest.mark.parametrize("fmt", [B.Q2_K, B.IQ2_XXS])
def test_x86_order_close_to_portable(oracle, fmt):
    rows, cols = 32, 4096
    w = B.synth_matrix(fmt, rows, cols, seed=21 + fmt)
    x = np.random.default_rng(8).standard_normal(cols).astype(np.float32)
    act = oracle.quantize_act(fmt, x)
    port = oracle.matvec(fmt, w, rows, cols, act)[0]
    rb = B.row_bytes(fmt, cols)
    x86 = np.array([oracle.row_dot_x86(fmt, w[r * rb:(r + 1) * rb], cols, act) for r in range(rows)], np.float32)
    _, terms = _exact_dot(oracle, fmt, w, rows, cols, act)
    assert (np.abs(port - x86) / terms).max() < 1e-6


@pytest.mark.parametrize("fmt", [B.Q8_0, B.Q4_K, B.Q6_K, B.Q2_K, B.IQ2_XXS])
def test_avx2_row_dots_are_the_scalar_bits(oracle, fmt):
    """The timed CPU baseline's AVX2 dots: the portable loop's bits for Q8_0 / Q4_K / Q6_K (same float steps, exact
    integer sums), the x86-order restatement's bits for IQ2_XXS / Q2_K (IQ2XXS-DOT-AVX2 / Q2K-DOT-AVX2,
    src/avx2.lisp:77-150)."""
    if not oracle.simd_available():
        pytest.skip("no AVX2 on this CPU")
    rows, cols = 64, B.BLOCK_WEIGHTS[fmt] * 8 if fmt != B.Q8_0 else 32 * 19
    w = B.synth_matrix(fmt, rows, cols, seed=31 + fmt)
    x = np.random.default_rng(fmt).standard_normal(cols).astype(np.float32)
    x[:32] = 127.0          # saturated quants
    act = oracle.quantize_act(fmt, x)
    rb = B.row_bytes(fmt, cols)
    want = (oracle.matvec(fmt, w, rows, cols, act)[0] if fmt in (B.Q8_0, B.Q4_K, B.Q6_K)
            else np.array([oracle.row_dot_x86(fmt, w[r * rb:(r + 1) * rb], cols, act) for r in range(rows)], np.float32))
    got = np.array([oracle.row_dot_simd(fmt, w[r * rb:(r + 1) * rb], cols, act) for r in range(rows)], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the pool of pinned threads gives what created threads give
    prev = oracle.set_fast(True)
    try:
        fast = oracle.matvec(fmt, w, rows, cols, act, threads=4)[0]
        again = oracle.matvec(fmt, w, rows, cols, act, threads=3)[0]
    finally:
        oracle.set_fast(prev)
    assert np.array_equal(fast.view(np.uint32), got.view(np.uint32)) and np.array_equal(again, fast)


def test_matvec_threads_and_bias(oracle):
    rows, cols = 37, 512
    w = B.synth_matrix(B.Q4_K, rows, cols, seed=31)
    x = np.random.default_rng(9).standard_normal(2 * cols).astype(np.float32)
    act = oracle.quantize_act(B.Q4_K, x)
    bias = np.arange(rows, dtype=np.float32)
    a = oracle.matvec(B.Q4_K, w, rows, cols, act, n=2, bias=bias, threads=1)
    b = oracle.matvec(B.Q4_K, w, rows, cols, act, n=2, bias=bias, threads=5)
    assert np.array_equal(a, b)  # 1 thread = many (inspect/consistency-test.lisp:48-51)
    c = oracle.matvec(B.Q4_K, w, rows, cols, act, n=2)
    assert np.array_equal(a, c + bias)


def test_route(oracle):
    rng = np.random.default_rng(10)
    logits = rng.standard_normal((5, 64)).astype(np.float32)
    logits[0, 7] = logits[0, 3] = 4.0  # a tie: the earlier expert first
    for mode in (0, 2):
        sel, w = oracle.route(logits, 6, mode=mode, scale=1.5)
        assert list(sel[0][:2]) == [3, 7]
        p = 1 / (1 + np.exp(-logits.astype(np.float64))) if mode == 2 else np.sqrt(np.log1p(np.exp(logits.astype(np.float64))))
        for t in range(5):
            order = np.argsort(-p[t], kind="stable")[:6]
            assert list(sel[t]) == list(order)
            np.testing.assert_allclose(w[t], p[t][order] / p[t][order].sum() * 1.5, rtol=1e-5)
    bias = np.zeros(64, np.float32)
    bias[60] = 10.0
    sel, w = oracle.route(logits, 6, mode=2, bias=bias)
    assert (sel[:, 0] == 60).all()  # biased scores pick, unbiased probabilities weigh
    assert abs(w.sum(1) - 1).max() < 1e-5


def test_moe_routed_composition(oracle):
    """orc_moe_routed against the same steps taken one at a time."""
    d, ff, ne, nu = 512, 256, 8, 3
    gate = B.synth_matrix(B.IQ2_XXS, ne * ff, d, seed=41)
    up = B.synth_matrix(B.IQ2_XXS, ne * ff, d, seed=42)
    down = B.synth_matrix(B.Q2_K, ne * d, ff, seed=43)
    x = np.random.default_rng(11).standard_normal(d).astype(np.float32)
    sel = np.array([5, 0, 6], np.int32)
    wts = np.array([0.5, 0.3, 0.2], np.float32)
    clamp = 0.05
    moe, mid = oracle.moe_routed(d, ff, B.IQ2_XXS, B.Q2_K, gate, up, down, x, sel, wts, clamp, threads=3, want_mid=True)
    act = oracle.quantize_q8k(x)
    grb, drb = B.row_bytes(B.IQ2_XXS, d), B.row_bytes(B.Q2_K, ff)
    want = np.zeros(d, np.float32)
    for i, e in enumerate(sel):
        g = oracle.matvec(B.IQ2_XXS, gate[e * ff * grb:(e + 1) * ff * grb], ff, d, act)[0]
        u = oracle.matvec(B.IQ2_XXS, up[e * ff * grb:(e + 1) * ff * grb], ff, d, act)[0]
        g = np.minimum(g, np.float32(clamp))
        u = np.clip(u, -np.float32(clamp), np.float32(clamp))
        silu = np.array([oracle.lib().orc_silu(float(v)) for v in g], np.float32)
        m = ((silu * u).astype(np.float32) * wts[i]).astype(np.float32)
        assert np.array_equal(m, mid[i * ff:(i + 1) * ff])
        dn = oracle.matvec(B.Q2_K, down[e * d * drb:(e + 1) * d * drb], d, ff, oracle.quantize_q8k(m))[0]
        want = (want + dn).astype(np.float32)
    assert np.array_equal(moe, want)


def test_f32mv(oracle):
    """F32MV!'s plain loop: a float accumulator, columns in order."""
    rng = np.random.default_rng(12)
    w = rng.standard_normal((7, 300)).astype(np.float32)
    x = rng.standard_normal(300).astype(np.float32)
    got = oracle.f32mv(w, x)
    want = np.empty(7, np.float32)
    for r in range(7):
        acc = np.float32(0)
        for j in range(300):
            acc = np.float32(acc + np.float32(w[r, j] * x[j]))
        want[r] = acc
    assert np.array_equal(got, want)
