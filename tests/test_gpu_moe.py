"""The routed experts on a B200 against the CPU oracle: routing, the stable
grouping by expert, and one decoded token through DK-FFN-TAIL (IQ2_XXS gate/up,
Q2_K down) plus the Q8_0 shared expert."""
import numpy as np
import pytest
import torch

from illatio_b200 import _lib
from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from illatio_b200 import cuda_ds4f as M
from gpu_util import rel_errors, to_dev

pytestmark = pytest.mark.gpu
TOL_SPEC = 2e-3


@pytest.fixture(autouse=True)
def _need_gpu(cuda_lib):
    assert torch.cuda.is_available()
    yield
    assert D.device_status() == 0


@pytest.mark.parametrize("ne,nu,mode", [(256, 6, 2), (288, 8, 2), (256, 6, 0), (64, 1, 2), (33, 32, 0)])
def test_route_matches_oracle(oracle, ne, nu, mode):
    rng = np.random.default_rng(ne + nu)
    n = 777
    logits = rng.standard_normal((n, ne)).astype(np.float32)
    logits[0, 7 % ne] = logits[0, 3 % ne] = 4.0      # equal scores: the earlier expert first
    logits[1, :] = 0.25                               # all equal
    logits[2, :] = -30.0                              # tiny probabilities (the floor on the sum)
    bias = (rng.standard_normal(ne) * 0.1).astype(np.float32) if mode == 2 else None
    sel, w = M.route(to_dev(logits), nu, mode=mode, bias=None if bias is None else to_dev(bias), scale=1.5)
    osel, ow = oracle.route(logits, nu, mode=mode, bias=bias, scale=1.5)
    gs, gw = sel.cpu().numpy(), w.cpu().numpy()
    same = (gs == osel).all(axis=1)
    # expf / logf differ from libm by an ulp: a pick may only differ where two scores are within rounding
    assert same.mean() > 0.995 and same[:3].all()
    np.testing.assert_allclose(gw[same], ow[same], rtol=2e-6, atol=1e-9)


@pytest.mark.parametrize("n,ne,nu", [(1, 256, 6), (4096, 256, 6), (1000, 288, 8), (3, 8, 2)])
def test_group_is_a_stable_sort(n, ne, nu):
    rng = np.random.default_rng(n)
    p = 1.0 / np.arange(1, ne + 1) ** 1.1  # skewed popularity
    p /= p.sum()
    sel = np.stack([rng.choice(ne, size=nu, replace=False, p=p) for _ in range(n)]).astype(np.int32)
    w = rng.random((n, nu)).astype(np.float32)
    rows = n * nu
    dsel, dw = to_dev(sel), to_dev(w)
    scratch = torch.empty(_lib.lib().ill_moe_group_scratch_bytes(rows, ne), dtype=torch.uint8, device="cuda")
    counts = torch.empty(ne, dtype=torch.int32, device="cuda")
    bases = torch.empty(ne, dtype=torch.int32, device="cuda")
    rmap = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    smap = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    wrow = torch.zeros(rows, dtype=torch.float32, device="cuda")
    _lib.call("ill_moe_group", rows, ne, nu, dsel.data_ptr(), dw.data_ptr(), scratch.data_ptr(), counts.data_ptr(),
              bases.data_ptr(), rmap.data_ptr(), smap.data_ptr(), wrow.data_ptr(), None)
    flat = sel.reshape(-1)
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(counts.cpu().numpy(), np.bincount(flat, minlength=ne))
    assert np.array_equal(bases.cpu().numpy(), np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=ne))[:-1]]))
    assert np.array_equal(rmap.cpu().numpy(), order // nu)
    inv = np.empty(rows, np.int64)
    inv[order] = np.arange(rows)
    assert np.array_equal(smap.cpu().numpy(), inv)
    assert np.array_equal(wrow.cpu().numpy(), w.reshape(-1)[order])


def _experts(d, ff, ne, gate_fmt=B.IQ2_XXS, down_fmt=B.Q2_K, seed=0):
    gate = B.synth_matrix(gate_fmt, ne * ff, d, seed=seed + 1)
    up = B.synth_matrix(gate_fmt, ne * ff, d, seed=seed + 2)
    down = B.synth_matrix(down_fmt, ne * d, ff, seed=seed + 3)
    return gate, up, down


@pytest.mark.parametrize("d,ff,ne,nu,gate_fmt,clamp", [
    (4096, 2048, 12, 6, B.IQ2_XXS, 10.0),   # the DeepSeek-V4-Flash-shaped layer's sizes, fewer experts
    (5120, 1536, 10, 8, B.Q2_K, 0.0),       # the GLM-style layer: Q2_K throughout
    (512, 256, 4, 1, B.IQ2_XXS, 0.05),      # one expert, a clamp that bites
])
def test_decode_token_matches_oracle(oracle, d, ff, ne, nu, gate_fmt, clamp):
    gate, up, down = _experts(d, ff, ne, gate_fmt=gate_fmt, seed=d)
    pool = M.make_expert_pool(gate, up, down, d, ff, ne, gate_fmt=gate_fmt)
    rng = np.random.default_rng(5)
    x = rng.standard_normal(d).astype(np.float32)
    logits = rng.standard_normal((1, ne)).astype(np.float32)
    sel, w = M.route(to_dev(logits), nu, mode=2)
    osel, ow = oracle.route(logits, nu, mode=2)
    assert np.array_equal(sel.cpu().numpy(), osel)
    moe, mid = M.dk_ffn_tail(pool, to_dev(x), sel[0], w[0], clamp)
    want, wmid = oracle.moe_routed(d, ff, gate_fmt, B.Q2_K, gate, up, down, x, osel[0], ow[0], clamp, threads=4,
                                   want_mid=True)
    a, _ = rel_errors(mid.cpu().numpy(), wmid)
    assert a < 1e-4, ("mid", a)
    a, _ = rel_errors(moe.cpu().numpy(), want)
    assert a < TOL_SPEC, ("moe", a)


def test_shared_expert_matches_oracle(oracle):
    d, ff, clamp = 4096, 2048, 10.0
    mats = [B.synth_matrix(B.Q8_0, r, c, seed=s) for s, (r, c) in enumerate([(ff, d), (ff, d), (d, ff)])]
    ws = [D.upload_gmat(m, B.Q8_0, r, c) for m, (r, c) in zip(mats, [(ff, d), (ff, d), (d, ff)])]
    x = np.random.default_rng(6).standard_normal(d).astype(np.float32) * 0.3
    out = torch.empty(d, device="cuda")
    M.dk_shared(ws[0], ws[1], ws[2], to_dev(x), clamp, out)
    want = oracle.moe_shared(d, ff, mats[0], mats[1], mats[2], x, clamp, threads=4)
    a, _ = rel_errors(out.cpu().numpy(), want)
    assert a < TOL_SPEC, a


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,n", [(256, 4096, 1), (37, 1000, 3), (5, 250, 16), (37, 1000, 40), (256, 2048, 130)])
def test_mv_dense_matches_f32mv(oracle, dtype, rows, cols, n):
    """The router's matvec and its kin: unquantized weights, float activations, the CPU's float dot as the check."""
    rng = np.random.default_rng(rows + cols)
    w = torch.as_tensor(rng.standard_normal((rows, cols)).astype(np.float32)).to(dtype)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    y = torch.full((n, rows + 3), 5.0, device="cuda")
    wd, xd = w.cuda(), to_dev(x)
    _lib.call("ill_mv_dense", M._DENSE_TYPES[dtype], wd.data_ptr(), rows, cols, xd.data_ptr(), y.data_ptr(), n, rows + 3, None)
    got = y.cpu().numpy()
    assert (got[:, rows:] == 5.0).all()
    wf = w.to(torch.float32).numpy()  # the CPU path's widened copy
    for t in range(n):
        want = oracle.f32mv(wf, x[t])
        terms = np.abs(wf.astype(np.float64) * x[t].astype(np.float64)).sum(1)
        assert (np.abs(got[t, :rows] - want) <= 1e-6 * terms + 1e-30).all()
    y1 = torch.empty(rows, device="cuda")
    M.dk_mv16(wd, xd[:1], y1)
    assert torch.equal(y1, y[0, :rows])
