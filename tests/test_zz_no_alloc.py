"""ill_moe_group_static: the grouping of (token, slot) rows by expert for hosts
that cannot allocate device memory -- its scratch lives in the library's own
device image instead of a caller's buffer.

It must give exactly what ill_moe_group gives (the outputs are integers and
copied floats, so the comparison is exact), on two calls in a row with
different inputs: the second call runs over whatever the first left in the
shared array.  The file sorts last so that a run that stops at the first
failure has already run everything else.
"""
import numpy as np
import pytest
import torch

from illatio_b200 import _lib
from illatio_b200 import cuda_dense as D

pytestmark = pytest.mark.gpu


def _group(entry, sel, w, ne, nu, scratch=None):
    rows = sel.numel()
    i32 = dict(dtype=torch.int32, device="cuda")
    counts, bases = torch.empty(ne, **i32), torch.empty(ne, **i32)
    rmap, smap = torch.full((rows,), -1, **i32), torch.full((rows,), -1, **i32)
    wrow = torch.zeros(rows, dtype=torch.float32, device="cuda")
    args = [rows, ne, nu, sel.data_ptr(), w.data_ptr()]
    if scratch is not None:
        args.append(scratch.data_ptr())
    args += [counts.data_ptr(), bases.data_ptr(), rmap.data_ptr(), smap.data_ptr(), wrow.data_ptr(), None]
    _lib.call(entry, *args)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (counts, bases, rmap, smap, wrow)]


def test_static_grouping_matches_on_two_calls_in_a_row(cuda_lib):
    assert torch.cuda.is_available()
    L = _lib.lib()
    for call, (n, ne, nu, seed) in enumerate([(4096, 256, 6, 1), (1500, 288, 8, 2)]):
        rng = np.random.default_rng(seed)
        sel_h = np.stack([rng.choice(ne, size=nu, replace=False) for _ in range(n)]).astype(np.int32)
        sel = torch.as_tensor(sel_h).cuda()
        w = torch.as_tensor(rng.random((n, nu)).astype(np.float32)).cuda()
        scratch = torch.empty(L.ill_moe_group_scratch_bytes(n * nu, ne), dtype=torch.uint8, device="cuda")
        want = _group("ill_moe_group", sel, w, ne, nu, scratch)
        got = _group("ill_moe_group_static", sel, w, ne, nu)
        for a, b in zip(got, want):
            assert np.array_equal(a, b), "call %d differs from ill_moe_group" % call
    assert D.device_status() == 0


def test_static_grouping_leaves_device_memory_as_it_found_it(cuda_lib):
    """The property in the entry point's name: the device's free memory is the same after the calls as
    before them.  One call comes first, so that the driver's lazy loading of the kernels (which is not
    an allocation of the entry point's) is over before the figure is taken; the inputs and outputs are
    allocated before it too."""
    assert torch.cuda.is_available()
    n, ne, nu = 3000, 256, 6
    rng = np.random.default_rng(3)
    sel = torch.as_tensor(np.stack([rng.choice(ne, size=nu, replace=False) for _ in range(n)]).astype(np.int32)).cuda()
    w = torch.rand(n, nu, device="cuda")
    rows = n * nu
    i32 = dict(dtype=torch.int32, device="cuda")
    counts, bases, rmap, smap = (torch.empty(k, **i32) for k in (ne, ne, rows, rows))
    wrow = torch.empty(rows, device="cuda")
    args = (rows, ne, nu, sel.data_ptr(), w.data_ptr(), counts.data_ptr(), bases.data_ptr(), rmap.data_ptr(), smap.data_ptr(),
            wrow.data_ptr(), None)
    _lib.call("ill_moe_group_static", *args)
    torch.cuda.synchronize()
    free0, total0 = torch.cuda.mem_get_info()
    for _ in range(2):
        _lib.call("ill_moe_group_static", *args)
    torch.cuda.synchronize()
    free1, total1 = torch.cuda.mem_get_info()
    assert (free1, total1) == (free0, total0)
    assert counts.sum().item() == rows


def test_static_grouping_rejects_sizes_beyond_its_array(cuda_lib):
    assert torch.cuda.is_available()
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = z.data_ptr()
    assert _lib.status("ill_moe_group_static", 65537, 8, 1, p, p, p, p, p, p, 0, None) == 6
    assert _lib.status("ill_moe_group_static", 8, 513, 1, p, p, p, p, p, p, 0, None) == 6
    assert b"maximum" in _lib.lib().ill_error_string(6)
