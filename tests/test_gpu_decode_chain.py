"""A token's chain of products in one launch (ill_decode_plan / ill_decode_run) against the same chain issued
product by product (ill_rmsnorm_q8, ill_quant_q8_k / ill_quant_q8_0, ill_mv, ill_mv_glu): the same bits, since a
row's arithmetic and the quantizers are shared; and the per-product path is what the other tests hold against
the CPU oracle.  One chain is also checked against the oracle directly.
"""
import numpy as np
import pytest
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from gpu_util import to_dev

pytestmark = pytest.mark.gpu
EPS = 1e-6


@pytest.fixture(autouse=True)
def _need_gpu(cuda_lib):
    assert torch.cuda.is_available()
    yield
    assert D.device_status() == 0


def _mat(fmt, rows, cols, seed):
    return D.CMat("m", fmt, rows, cols, B.synth_matrix_torch(fmt, rows, cols, seed=seed))


class Model:
    """A transformer's in-scope products, the attention itself stood in for by its query vector: per layer
    q / k / v <- rmsnorm(h); h += o(q); fa <- glu(rmsnorm(h)); h += down(fa); then the head on rmsnorm(h)."""

    def __init__(self, hidden, qdim, kvdim, ffn, vocab, layers, fmt_main, fmt_alt, seed=0):
        self.dims = (hidden, qdim, kvdim, ffn, vocab)
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.layers = []
        for li in range(layers):
            s = 100 * li + seed
            self.layers.append(dict(
                q=_mat(fmt_main, qdim, hidden, s + 1), k=_mat(fmt_main, kvdim, hidden, s + 2), v=_mat(fmt_alt, kvdim, hidden, s + 3),
                o=_mat(fmt_main, hidden, qdim, s + 4), gate=_mat(fmt_main, ffn, hidden, s + 5), up=_mat(fmt_main, ffn, hidden, s + 6),
                down=_mat(fmt_alt, hidden, ffn, s + 7),
                nw1=torch.rand(hidden, device="cuda", generator=g) + 0.5, nw2=torch.rand(hidden, device="cuda", generator=g) + 0.5))
        self.head = _mat(fmt_alt, vocab, hidden, seed + 99)
        self.nwf = torch.rand(hidden, device="cuda", generator=g) + 0.5
        f = dict(dtype=torch.float32, device="cuda")
        self.h = torch.empty(hidden, **f)
        self.q, self.k, self.v = torch.empty(qdim, **f), torch.empty(kvdim, **f), torch.empty(kvdim, **f)
        self.fa, self.logits = torch.empty(ffn, **f), torch.empty(vocab, **f)
        self.bias = torch.randn(kvdim, **f)

    def ops(self):
        out = []
        for L in self.layers:
            out += [D.decode_op(L["q"], self.h, self.q, norm_w=L["nw1"], eps=EPS, after=True),
                    D.decode_op(L["k"], self.h, self.k, norm_w=L["nw1"], eps=EPS, after=False, bias=self.bias),
                    D.decode_op(L["v"], self.h, self.v, norm_w=L["nw1"], eps=EPS, after=False),
                    D.decode_op(L["o"], self.q, self.h, acc=True, after=True),
                    D.decode_op(L["gate"], self.h, self.fa, w2=L["up"], norm_w=L["nw2"], eps=EPS, after=True),
                    D.decode_op(L["down"], self.fa, self.h, acc=True, after=True)]
        out.append(D.decode_op(self.head, self.h, self.logits, norm_w=self.nwf, eps=EPS, after=True))
        return out

    def per_product(self):
        """The same chain, a launch per product and per quantization."""
        hidden, qdim, kvdim, ffn, vocab = self.dims

        def act_of(w, n):
            return D.make_qact(n, D.matrix_act_kind(w), want_xsum=False)
        for L in self.layers:
            a = D.rmsnorm_q8(self.h, L["nw1"], act_of(L["q"], hidden), hidden, EPS)
            D.cmat_mul(L["q"], a, self.q, 1)
            D.cmat_mul(L["k"], a, self.k, 1, bias=self.bias)
            a2 = a if D.matrix_act_kind(L["v"]) == a.kind else D.rmsnorm_q8(self.h, L["nw1"], act_of(L["v"], hidden), hidden, EPS)
            D.cmat_mul(L["v"], a2, self.v, 1)
            D.cmat_mul(L["o"], D.quant_q8(self.q, act_of(L["o"], qdim)), self.h, 1, acc=True)
            a = D.rmsnorm_q8(self.h, L["nw2"], act_of(L["gate"], hidden), hidden, EPS)
            D.glu_mul(L["gate"], L["up"], a, self.fa)
            D.cmat_mul(L["down"], D.quant_q8(self.fa, act_of(L["down"], ffn)), self.h, 1, acc=True)
        a = D.rmsnorm_q8(self.h, self.nwf, act_of(self.head, hidden), hidden, EPS)
        D.cmat_mul(self.head, a, self.logits, 1)

    def state(self):
        return [t.clone() for t in (self.h, self.q, self.k, self.v, self.fa, self.logits)]


@pytest.mark.parametrize("dims,layers,fmt_main,fmt_alt", [
    ((512, 1024, 256, 1536, 3000), 3, B.Q4_K, B.Q6_K),       # a small Q4_K_M-style model
    ((896, 896, 128, 4864, 5000), 2, B.Q8_0, B.Q8_0),        # the 0.5B model's shapes, Q8_0 activations
    ((2560, 4096, 1024, 9728, 151936), 2, B.Q4_K, B.Q6_K),   # the 4B model's shapes and its whole head
    ((1024, 2048, 512, 2048, 2000), 2, B.IQ2_XXS, B.Q2_K),   # the 2-bit formats
])
def test_chain_equals_per_product_path(dims, layers, fmt_main, fmt_alt):
    m = Model(*dims, layers, fmt_main, fmt_alt, seed=3)
    x0 = torch.randn(dims[0], device="cuda", generator=torch.Generator(device="cuda").manual_seed(9))
    m.h.copy_(x0)
    m.per_product()
    want = m.state()
    plan = D.DecodePlan(m.ops())
    for _ in range(2):   # the plan and its barrier serve any number of tokens
        for t in (m.q, m.k, m.v, m.fa, m.logits):
            t.fill_(-3.0)
        m.h.copy_(x0)
        plan.run()
        torch.cuda.synchronize()
        for name, a, b in zip("h q k v fa logits".split(), m.state(), want):
            assert torch.isfinite(a).all(), name
            assert torch.equal(a, b), "%s differs: %g" % (name, (a - b).abs().max().item())


def test_chain_against_the_oracle(oracle):
    """rmsnorm -> gated Q4_K product -> Q6_K product added into h, each step against the CPU routines."""
    hidden, ffn = 768, 1280
    rng = np.random.default_rng(5)
    g, u = (B.synth_matrix(B.Q4_K, ffn, hidden, seed=s) for s in (1, 2))
    dn = B.synth_matrix(B.Q6_K, hidden, ffn, seed=3)
    h0 = rng.standard_normal(hidden).astype(np.float32)
    nw = (rng.random(hidden) + 0.5).astype(np.float32)
    h, fa = to_dev(h0), torch.empty(ffn, device="cuda")
    G, U, DN = (D.upload_gmat(m, f, r, c) for m, f, r, c in ((g, B.Q4_K, ffn, hidden), (u, B.Q4_K, ffn, hidden), (dn, B.Q6_K, hidden, ffn)))
    nwd = to_dev(nw)   # the plan keeps addresses only: every buffer it names must outlive it
    plan = D.DecodePlan([D.decode_op(G, h, fa, w2=U, norm_w=nwd, eps=EPS, after=False),
                         D.decode_op(DN, fa, h, acc=True, after=True)])
    plan.run()
    torch.cuda.synchronize()
    act = oracle.quantize_q8k(oracle.rmsnorm(h0, nw, EPS))
    gv = oracle.matvec(B.Q4_K, g, ffn, hidden, act)[0].astype(np.float64)
    uv = oracle.matvec(B.Q4_K, u, ffn, hidden, act)[0].astype(np.float64)
    want_fa = gv / (1 + np.exp(-gv)) * uv
    got_fa = fa.cpu().numpy()
    assert np.abs(got_fa - want_fa).max() / np.abs(want_fa).max() < 1e-5
    want_h = h0 + oracle.matvec(B.Q6_K, dn, hidden, ffn, oracle.quantize_q8k(got_fa))[0]
    assert np.abs(h.cpu().numpy() - want_h).max() / np.abs(want_h).max() < 1e-5


def test_long_rows_are_taken_in_runs_of_columns():
    """Rows too long to fit a tile whole (and for ill_mv to keep in registers): 17408 columns, Q6_K and Q8_0.
    The chain takes such a row in runs of columns and carries its sum; against ill_mv, whose order of additions
    differs for such rows, to fp32 reassociation."""
    for fmt in (B.Q6_K, B.Q8_0, B.Q4_K):
        w = _mat(fmt, 300, 17408, 1)
        x = torch.randn(17408, device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
        y, want = torch.zeros(300, device="cuda"), torch.zeros(300, device="cuda")
        D.DecodePlan([D.decode_op(w, x, y, after=False)]).run()
        D.cmat_mul(w, D.quant_q8(x, D.make_qact(17408, D.matrix_act_kind(w))), want, 1)
        torch.cuda.synchronize()
        assert ((y - want).abs().max() / want.abs().max()).item() < 1e-5


def test_plan_refuses_what_it_cannot_run():
    from illatio_b200 import _lib
    w = _mat(B.Q4_K, 64, 512, 1)
    op = D.decode_op(w, torch.zeros(516, device="cuda")[1:513], torch.zeros(64, device="cuda"))   # X not 16-byte aligned
    with pytest.raises(_lib.IllatioError) as e:
        D.DecodePlan([op])
    assert e.value.code == 2
    op = D.decode_op(w, torch.zeros(512, device="cuda"), torch.zeros(64, device="cuda"))
    op.cols = 500                                                                                # not whole blocks
    with pytest.raises(_lib.IllatioError) as e:
        D.DecodePlan([op])
    assert e.value.code == 1
