"""GGUF file -> device (UPLOAD-GMAT, src/cuda-dense.lisp:75-100): a matrix uploaded from a file multiplies like the
same blocks uploaded directly, and an unquantized tensor arrives with its values."""
import numpy as np
import pytest
import torch

from illatio_b200 import blocks as B
from illatio_b200 import cuda_dense as D
from illatio_b200 import gguf as G
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def test_upload_gmat_from_a_file(cuda_lib, tmp_path):
    rows, cols = 300, 1024
    fmts = (("q8_0", B.Q8_0), ("q4_k", B.Q4_K), ("q6_k", B.Q6_K), ("q2_k", B.Q2_K), ("iq2_xxs", B.IQ2_XXS))
    mats = {name: B.synth_matrix(f, rows, cols, seed=10 + f) for name, f in fmts}
    router = np.random.default_rng(3).standard_normal((16, cols)).astype("<f4")
    tensors = [("blk.0.%s.weight" % name, (cols, rows), name, np.asarray(m).tobytes()) for name, m in mats.items()]
    tensors.append(("blk.0.ffn_gate_inp.weight", (cols, 16), "f32", router.tobytes()))
    p = tmp_path / "m.gguf"
    G.write_gguf(p, {"general.architecture": "test"}, tensors)
    g = G.read_gguf(p)
    x = torch.randn(cols, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    for name, f in fmts:
        w = G.upload_gmat(g, "blk.0.%s.weight" % name)
        assert (w.type, w.rows, w.cols) == (f, rows, cols)
        direct = D.upload_gmat(mats[name], f, rows, cols)
        act = D.quant_q8(x, D.make_qact(cols, D.matrix_act_kind(w)))
        y, want = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
        D.cmat_mul(w, act, y, 1)
        D.cmat_mul(direct, act, want, 1)
        torch.cuda.synchronize()
        assert torch.equal(y, want) and torch.isfinite(y).all()
    r = G.upload_gmat(g, "blk.0.ffn_gate_inp.weight")
    assert r.dtype == torch.float32 and tuple(r.shape) == (16, cols) and np.array_equal(r.cpu().numpy(), router)
    # small chunks: the staging buffers alternate
    raw = G.upload_tensor(g, "blk.0.q6_k.weight", chunk=4096)
    assert raw.cpu().numpy().tobytes() == np.asarray(mats["q6_k"]).tobytes()
    with pytest.raises(G.GgufError):
        G.upload_gmat(g, "absent")
    assert D.device_status() == 0
