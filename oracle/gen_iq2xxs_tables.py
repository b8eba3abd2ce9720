"""Generate iq2xxs_tables.h from the reference's own copy of the IQ2_XXS tables.

The 256-entry grid and the 128-entry sign table are data from ggml (MIT,
Copyright (c) 2023-2026 The ggml authors); the reference keeps its copy in
src/iquant.lisp (+IQ2XXS-GRID+ and +KSIGNS-IQ2XS+).  This script parses the two
`:initial-contents` lists out of that file and writes them as C arrays, so the
numbers are taken from the reference and not retyped.

    python oracle/gen_iq2xxs_tables.py /path/to/reference/src/iquant.lisp

writes oracle/iq2xxs_tables.h and illatio_b200/csrc/iq2xxs_tables.cuh (the same
numbers; the second is the copy the CUDA kernels include).
"""
import os
import re
import sys

NOTICE = """\
/* IQ2_XXS codebook and sign patterns.  Data from ggml (MIT License,
 * Copyright (c) 2023-2026 The ggml authors), taken from the reference's copy
 * in src/iquant.lisp (+IQ2XXS-GRID+, +KSIGNS-IQ2XS+) by
 * oracle/gen_iq2xxs_tables.py.  Generated file: do not edit.
 *
 * Grid entry g holds eight magnitudes (8, 25 or 43), one per byte, little
 * endian.  Sign pattern s (7 bits) expands to 8 sign bits; bit 7 is the parity
 * of the low seven. */
"""


def parse(path):
    text = open(path).read()
    m = re.search(r"\+iq2xxs-grid\+.*?:initial-contents\s*'\((.*?)\)\)\)", text, re.S)
    grid = [int(t[2:], 16) for t in m.group(1).split()]
    m = re.search(r"\+ksigns-iq2xs\+.*?:initial-contents\s*'\((.*?)\)\)\)", text, re.S)
    signs = [int(t) for t in m.group(1).split()]
    assert len(grid) == 256 and len(signs) == 128
    for g in grid:
        assert all(((g >> (8 * j)) & 0xFF) in (8, 25, 43) for j in range(8))
    for s, v in enumerate(signs):
        assert v & 127 == s and (v >> 7) == bin(s).count("1") % 2
    return grid, signs


def emit(grid, signs, qual_grid, qual_signs, guard):
    out = [NOTICE, "#ifndef %s\n#define %s\n#include <stdint.h>\n" % (guard, guard)]
    out.append("%s uint64_t ill_iq2xxs_grid[256] = {" % qual_grid)
    for i in range(0, 256, 4):
        out.append("  " + " ".join("0x%016xULL," % g for g in grid[i:i + 4]))
    out.append("};\n")
    out.append("%s uint8_t ill_ksigns_iq2xs[128] = {" % qual_signs)
    for i in range(0, 128, 16):
        out.append("  " + " ".join("%3d," % s for s in signs[i:i + 16]))
    out.append("};\n\n#endif\n")
    return "\n".join(out)


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: gen_iq2xxs_tables.py <the reference's src/iquant.lisp>")
    src = sys.argv[1]
    grid, signs = parse(src)
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "iq2xxs_tables.h"), "w") as f:
        f.write(emit(grid, signs, "static const", "static const", "ILL_ORACLE_IQ2XXS_TABLES_H"))
    cu = os.path.join(here, "..", "illatio_b200", "csrc", "iq2xxs_tables.cuh")
    with open(cu, "w") as f:
        f.write(emit(grid, signs, "static __device__ const", "static __device__ const",
                     "ILL_B200_IQ2XXS_TABLES_CUH"))


if __name__ == "__main__":
    main()
