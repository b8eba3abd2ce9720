"""Generates the dequantization fixtures in this directory.

    python tests/golden/gen_golden.py

For each of the five block formats: 48 raw blocks (seeded random bytes with the
scale distributions of illatio_b200.blocks, then edge cases: zero scales, fp16
subnormal and negative scales, IQ2_XXS sub-block scales 0 and 15, saturated
quants) and their floats from gguf-py's `gguf.quants.dequantize` (gguf 0.19.0)
-- the dequantizer the reference's own inspect/iquant-test.lisp compares
against and requires identical floats from.  The fixture pins the CPU oracle
(tests/test_oracle.py) and, through it, the CUDA kernels.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from gguf import GGMLQuantizationType as T  # noqa: E402
from gguf import quants  # noqa: E402

from illatio_b200 import blocks as B  # noqa: E402

GG = {B.Q8_0: T.Q8_0, B.Q4_K: T.Q4_K, B.Q6_K: T.Q6_K, B.Q2_K: T.Q2_K, B.IQ2_XXS: T.IQ2_XXS}


def f16_bytes(v):
    return np.array([v], np.float16).view(np.uint8)


def edge_cases(fmt, blk):
    """Overwrite the last blocks of BLK with edge cases."""
    offs = B.SCALE_OFFSETS[fmt]
    specials = [0.0, -0.0, 5.96e-8, 6.0e-5, -0.0123, 65504.0, 1.0, -1.0]
    for i, v in enumerate(specials):
        b = blk[-1 - i]
        for off in offs:
            b[off:off + 2] = f16_bytes(v)
    if fmt == B.IQ2_XXS:
        blk[-9, 2:] = 0x00          # grid index 0, sign pattern 0, LS 0
        blk[-10, 2:] = 0xFF         # grid index 255, sign pattern 127, LS 15
    if fmt == B.Q8_0:
        blk[-9, 2:] = 0x81          # -127
        blk[-10, 2:] = 0x80         # -128 (never produced by a quantizer, still defined)
    if fmt in (B.Q4_K, B.Q2_K, B.Q6_K):
        lo = {B.Q4_K: 4, B.Q2_K: 0, B.Q6_K: 0}[fmt]
        hi = {B.Q4_K: 144, B.Q2_K: 80, B.Q6_K: 208}[fmt]
        blk[-9, lo:hi] = 0xFF
        blk[-10, lo:hi] = 0x00
    return blk


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    for fmt in range(5):
        blk = edge_cases(fmt, B.synth_blocks(fmt, 48, seed=1000 + fmt))
        floats = quants.dequantize(blk, GG[fmt]).astype(np.float32)
        assert floats.shape == (48, B.BLOCK_WEIGHTS[fmt])
        assert np.isfinite(floats).all()
        np.savez_compressed(os.path.join(here, "dequant_%s.npz" % B.NAMES[fmt]), blocks=blk, floats=floats)
        print(B.NAMES[fmt], blk.shape, floats.shape, float(np.abs(floats).max()))


if __name__ == "__main__":
    main()
