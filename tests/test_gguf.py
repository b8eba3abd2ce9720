"""The GGUF reader (src/gguf.lisp:105-157) on files written here: header, every metadata value type, the tensor
directory and its alignment, the raw bytes; and what is refused."""
import struct

import numpy as np
import pytest

from illatio_b200 import blocks as B
from illatio_b200 import gguf as G


def _file(tmp_path, version=3, alignment=32):
    rng = np.random.default_rng(1)
    q4 = B.synth_matrix(B.Q4_K, 6, 512, seed=1)
    q8 = B.synth_matrix(B.Q8_0, 5, 96, seed=2)
    f32 = rng.standard_normal((3, 7)).astype("<f4")
    meta = {"general.architecture": "qwen3", "qwen3.block_count": 36, "qwen3.rope.freq_base": 1000000.0, "flag": True,
            "neg": -5, "big": 1 << 40, "tokenizer.ggml.tokens": ["a", "bc", ""], "ints": [1, 2, 3], "floats": [0.5, 1.5]}
    tensors = [("blk.0.ffn_gate.weight", (512, 6), "q4_k", np.asarray(q4).tobytes()),
               ("output_norm.weight", (7, 3), "f32", f32.tobytes()),
               ("token_embd.weight", (96, 5), "q8_0", np.asarray(q8).tobytes())]
    p = tmp_path / "m.gguf"
    G.write_gguf(p, meta, tensors, version=version, alignment=alignment)
    return p, meta, tensors


@pytest.mark.parametrize("version,alignment", [(3, 32), (2, 32), (3, 64)])
def test_read_back(tmp_path, version, alignment):
    p, meta, tensors = _file(tmp_path, version, alignment)
    g = G.read_gguf(p)
    assert g.version == version and g.alignment == alignment and g.data_offset % alignment == 0
    for k, v in meta.items():
        got = g.meta(k)
        if isinstance(v, float):
            assert got == pytest.approx(v)
        elif isinstance(v, list) and v and isinstance(v[0], float):
            assert got == pytest.approx(v)
        else:
            assert got == v, k
    assert g.meta("absent", 7) == 7
    assert g.tensor_order == [t[0] for t in tensors]
    for name, dims, tname, data in tensors:
        ti = g.tensor(name)
        assert ti.dims == dims and ti.type == tname and ti.offset % alignment == 0
        assert G.tensor_bytes(ti) == len(data)
        assert G.tensor_view(g, ti).tobytes() == data
        parts = []
        G.call_with_tensor_bytes(g, ti, lambda buf, pos: parts.append((pos, bytes(buf))), chunk=100)
        assert b"".join(b for _, b in parts) == data and [q for q, _ in parts] == list(range(0, len(data), 100))
    assert G.tensor_elements(g.tensor("blk.0.ffn_gate.weight")) == 6 * 512
    assert g.tensor("nope", errorp=False) is None
    with pytest.raises(G.GgufError):
        g.tensor("nope")


def test_refusals(tmp_path):
    p, _, _ = _file(tmp_path)
    raw = bytearray(p.read_bytes())
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + raw[4:])
    with pytest.raises(G.GgufError, match="not a GGUF file"):
        G.read_gguf(bad)
    bad.write_bytes(raw[:4] + struct.pack("<I", 1) + raw[8:])
    with pytest.raises(G.GgufError, match="version 1"):
        G.read_gguf(bad)
    bad.write_bytes(raw[:40])
    with pytest.raises(G.GgufError, match="ends inside"):
        G.read_gguf(bad)
    g = G.read_gguf(p)
    bad.write_bytes(raw[:len(raw) - 64])   # the directory is whole, the last tensor is not
    gb = G.read_gguf(bad)
    with pytest.raises(G.GgufError, match="truncated"):
        G.tensor_view(gb, gb.tensor(g.tensor_order[-1]))
    # a tensor that is not a whole number of blocks
    odd = tmp_path / "odd.gguf"
    G.write_gguf(odd, {}, [("w", (100, 2), "q4_k", b"\0" * 144)])
    go = G.read_gguf(odd)
    with pytest.raises(G.GgufError, match="whole number"):
        G.tensor_bytes(go.tensor("w"))


def test_file_written_by_gguf_py():
    """tests/golden/tiny.gguf comes from gguf-py's GGUFWriter (tests/golden/gen_gguf_fixture.py): the container as its
    reference implementation writes it."""
    import os
    g = G.read_gguf(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny.gguf"))
    assert g.version == 3 and g.alignment == 32 and g.data_offset % 32 == 0
    assert g.meta("general.architecture") == "qwen3" and g.meta("qwen3.block_count") == 2
    assert g.meta("qwen3.context_length") == 4096 and g.meta("qwen3.attention.layer_norm_rms_epsilon") == pytest.approx(1e-6)
    assert g.meta("test.flag") is True and g.meta("test.negative") == -7 and g.meta("test.big") == 1 << 40
    assert g.meta("test.name") == "tiny fixture" and g.meta("test.ints") == [3, 1, 4, 1, 5]
    assert g.meta("test.words") == ["alpha", "beta", ""]
    assert g.tensor_order == ["token_embd.weight", "output_norm.weight", "blk.0.attn_q.bias", "blk.0.ffn_gate.weight"]
    # the values the generating script drew
    rng = np.random.default_rng(20240501)
    emb = rng.standard_normal((5, 64)).astype(np.float32)
    norm = rng.standard_normal(7).astype(np.float32)
    half = rng.standard_normal((3, 8)).astype(np.float16)
    q4 = np.asarray(B.synth_matrix(B.Q4_K, 4, 256, seed=9), dtype=np.uint8)
    t = g.tensor("token_embd.weight")
    assert (t.dims, t.type) == ((64, 5), "q8_0") and G.tensor_bytes(t) == 5 * 2 * 34
    blocks = G.tensor_view(g, t).reshape(10, 34)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)          # a block: its scale, then 32 int8
    deq = (blocks[:, 2:].copy().view(np.int8).astype(np.float32) * d).reshape(5, 64)
    assert np.abs(deq - emb).max() <= 0.51 * d.max()
    assert np.array_equal(G.tensor_view(g, g.tensor("output_norm.weight")).view(np.float32), norm)
    assert g.tensor("blk.0.attn_q.bias").dims == (8, 3)
    assert np.array_equal(G.tensor_view(g, g.tensor("blk.0.attn_q.bias")).view(np.float16).reshape(3, 8), half)
    assert np.array_equal(G.tensor_view(g, g.tensor("blk.0.ffn_gate.weight")), q4.reshape(-1))
