"""GGUF block formats of the quantized-product path, and seeded synthetic blocks.

Block geometry follows the reference's type table (src/gguf.lisp:31-40) and the
layouts its CPU kernels read (src/tensor.lisp:213-225, src/kquant.lisp:6-11,
src/iquant.lisp:11-18).  Real model files are not available, so matrices are
drawn from seeded distributions: fp16 scales |N(0,1)| * sigma, every other byte
uniform (int8 quants of Q8_0 uniform in [-127, 127]).
"""
import numpy as np

Q8_0, Q4_K, Q6_K, Q2_K, IQ2_XXS = range(5)
NAMES = {Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k", Q2_K: "q2_k", IQ2_XXS: "iq2_xxs"}
BY_NAME = {v: k for k, v in NAMES.items()}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210, Q2_K: 84, IQ2_XXS: 66}
BLOCK_WEIGHTS = {Q8_0: 32, Q4_K: 256, Q6_K: 256, Q2_K: 256, IQ2_XXS: 256}
# byte offsets of the fp16 scale fields inside a block
SCALE_OFFSETS = {Q8_0: (0,), Q4_K: (0, 2), Q6_K: (208,), Q2_K: (80, 82), IQ2_XXS: (0,)}
SCALE_SIGMA = {Q8_0: 0.02, Q4_K: 0.01, Q6_K: 0.01, Q2_K: 0.01, IQ2_XXS: 0.01}


def row_bytes(fmt, cols):
    if cols % BLOCK_WEIGHTS[fmt]:
        raise ValueError("%d columns is not a whole number of %s blocks" % (cols, NAMES[fmt]))
    return cols // BLOCK_WEIGHTS[fmt] * BLOCK_BYTES[fmt]


def matrix_bytes(fmt, rows, cols):
    return rows * row_bytes(fmt, cols)


def synth_blocks(fmt, nblocks, seed):
    """NBLOCKS raw blocks as a uint8 array [nblocks, block_bytes]."""
    rng = np.random.default_rng(seed)
    bb = BLOCK_BYTES[fmt]
    blk = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    if fmt == Q8_0:
        q = rng.integers(-127, 128, size=(nblocks, 32), dtype=np.int8)
        blk[:, 2:34] = q.view(np.uint8)
    for off in SCALE_OFFSETS[fmt]:
        d = (np.abs(rng.standard_normal(nblocks)) * SCALE_SIGMA[fmt]).astype(np.float16)
        blk[:, off:off + 2] = d.view(np.uint8).reshape(nblocks, 2)
    return blk


def synth_matrix(fmt, rows, cols, seed):
    """A rows x cols matrix as a flat uint8 array of raw row-major blocks."""
    nb = rows * (cols // BLOCK_WEIGHTS[fmt])
    return synth_blocks(fmt, nb, seed).reshape(-1)


def synth_matrix_torch(fmt, rows, cols, seed, device="cuda"):
    """synth_matrix drawn on the device with torch's generator (same
    distributions, different stream of numbers): for matrices too large to be
    worth drawing on the host."""
    import torch
    nb = rows * (cols // BLOCK_WEIGHTS[fmt])
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    blk = torch.randint(0, 256, (nb, BLOCK_BYTES[fmt]), dtype=torch.uint8, device=device, generator=g)
    if fmt == Q8_0:
        q = torch.randint(-127, 128, (nb, 32), dtype=torch.int8, device=device, generator=g)
        blk[:, 2:34] = q.view(torch.uint8)
    for off in SCALE_OFFSETS[fmt]:
        d = (torch.randn(nb, device=device, generator=g).abs() * SCALE_SIGMA[fmt]).to(torch.float16)
        blk[:, off:off + 2] = d.view(torch.uint8).reshape(nb, 2)
    return blk.reshape(-1)
