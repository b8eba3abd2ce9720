"""The C ABI without a GPU: the library loads and exports every entry point
include/illatio_b200.h declares, and the argument checks that need no device."""
import ctypes
import os
import re

from illatio_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "illatio_b200.h")).read()
    return re.findall(r"ILL_API\s+[\w\s\*]+?\b(ill_\w+)\s*\(", text)


def test_library_builds_and_exports_every_declared_symbol():
    build.build()
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(L, n), "libillatio_b200.so does not export %s" % n
        assert n in _lib.SIGNATURES, "no ctypes signature for %s" % n


def test_block_geometry_and_error_text():
    L = _lib.lib()
    assert L.ill_b200_version() >= 100
    assert [L.ill_block_bytes(f) for f in range(6)] == [34, 144, 210, 84, 66, 0]
    assert [L.ill_block_weights(f) for f in range(6)] == [32, 256, 256, 256, 256, 0]
    assert L.ill_error_string(0) == b"ok"
    for code in range(1, 7):
        assert len(L.ill_error_string(code)) > 4


def test_argument_checks_need_no_device():
    # bad format, bad sizes, null and misaligned pointers are rejected before any CUDA call
    s = _lib.status
    assert s("ill_mv", 9, 16, 4, 256, 16, 16, 16, 16, 0, 0, 1, None) == 1
    assert s("ill_mv", 1, 16, 4, 100, 16, 16, 16, 16, 0, 0, 1, None) == 1   # cols not a multiple of 256
    assert s("ill_mv", 1, 16, 4, 256, 16, 16, 0, 16, 0, 0, 1, None) == 1    # Q4_K needs the sums
    assert s("ill_mv", 1, 16, 4, 256, 17, 16, 16, 16, 0, 0, 1, None) == 2   # xq not 16-byte aligned
    assert s("ill_mv", 0, 16, 4, 256, 16, 16, 0, 16, 0, 0, 0, None) == 1    # no tokens
    assert s("ill_quant_q8_k", 8, 16, 16, 16, 1, None) == 2
    assert s("ill_dequant_rows", 4, 16, 100, 0, 0, 1, 16, None) == 1


def test_argument_checks_of_the_chunk_and_peer_entry_points():
    s = _lib.status
    # ill_mm_chunk: Q8_0 has no tcgen05 form; null pointers; a misaligned Q4_K matrix
    assert s("ill_mm_chunk", 0, 16, 4, 256, 16, 16, 16, 8, 16, 0, None) == 3
    assert s("ill_mm_chunk", 1, 0, 4, 256, 16, 16, 16, 8, 16, 0, None) == 1
    assert s("ill_mm_chunk", 1, 24, 4, 256, 16, 16, 16, 8, 16, 0, None) == 2
    assert s("ill_mm_chunk", 1, 16, 4, 256, 16, 0, 16, 8, 16, 0, None) == 1      # Q4_K needs the sums' tile
    assert s("ill_mm_chunk2", 3, 16, 32, 4, 256, 16, 16, 16, 8, 16, 32, None) == 3
    assert s("ill_mm_chunk2", 1, 16, 24, 4, 256, 16, 16, 16, 8, 16, 32, None) == 2  # the second matrix 8 bytes off
    # the peer-storing product and the all-gather by peer stores
    assert s("ill_mv_peers", 2, 16, 4, 256, 16, 16, 16, 0, 0, 0, 16, 16, 2, 0, 2, 1, 0, None) == 1      # no table of buffers
    assert s("ill_mv_peers", 2, 16, 4, 256, 16, 16, 16, 16, 0, 0, 16, 16, 2, 2, 2, 1, 0, None) == 1     # rank >= world
    assert s("ill_peer_put", 16, 64, 16, 0, 16, 16, 65, 0, 2, 1, 0, None) == 1                          # more ranks than flags
    assert s("ill_peer_put", 18, 64, 16, 0, 16, 16, 2, 0, 2, 1, 0, None) == 2                           # SRC not a multiple of 4
    assert s("ill_ep_dispatch", 4, 33, 256, 16, 16, 16, 16, 16, 1, 2, 8, 0, 16, 16, 16, 16, 1, None) == 1   # more than 32 slots
    assert s("ill_quant_q8_k_f16", 16, 16, 16, 16, 0, 16, 1, None) == 1
    # the table of a pointer a row for the one-token kernels: no experts, a misaligned table
    assert s("ill_moe_row_ptrs", 0, 16, 16, 16, 8, 16, None) == 1
    assert s("ill_moe_row_ptrs", 4, 16, 16, 16, 8, 20, None) == 1
    assert s("ill_moe_row_ptrs", 4, 16, 16, 16, 0, 16, None) == 0   # no rows: nothing to do
