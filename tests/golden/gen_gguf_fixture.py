"""Writes tests/golden/tiny.gguf with gguf-py's own GGUFWriter (the container's reference writer), so that the
reader in illatio_b200/gguf.py is checked against a file it did not write itself.

    python tests/golden/gen_gguf_fixture.py

Contents: metadata of several value types, a Q8_0 matrix quantized by gguf-py, an F32 and an F16 tensor, and a
Q4_K tensor of seeded raw blocks.  The values are fixed by the seeds below; tests/test_gguf.py re-derives them.
"""
import os
import sys

import numpy as np
import gguf
from gguf import GGMLQuantizationType as T

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from illatio_b200 import blocks as B  # noqa: E402


def contents():
    rng = np.random.default_rng(20240501)
    emb = rng.standard_normal((5, 64)).astype(np.float32)
    norm = rng.standard_normal(7).astype(np.float32)
    half = rng.standard_normal((3, 8)).astype(np.float16)
    q4 = np.asarray(B.synth_matrix(B.Q4_K, 4, 256, seed=9), dtype=np.uint8)
    return emb, norm, half, q4


def main():
    emb, norm, half, q4 = contents()
    w = gguf.GGUFWriter(os.path.join(HERE, "tiny.gguf"), "qwen3")
    w.add_block_count(2)
    w.add_context_length(4096)
    w.add_layer_norm_rms_eps(1e-6)
    w.add_bool("test.flag", True)
    w.add_int32("test.negative", -7)
    w.add_uint64("test.big", 1 << 40)
    w.add_string("test.name", "tiny fixture")
    w.add_array("test.ints", [3, 1, 4, 1, 5])
    w.add_array("test.words", ["alpha", "beta", ""])
    w.add_tensor("token_embd.weight", gguf.quants.quantize(emb, T.Q8_0), raw_dtype=T.Q8_0)
    w.add_tensor("output_norm.weight", norm)
    w.add_tensor("blk.0.attn_q.bias", half)
    w.add_tensor("blk.0.ffn_gate.weight", q4.reshape(4, 144), raw_dtype=T.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


if __name__ == "__main__":
    main()
