"""aclsparseB200SpMVNoAlloc: the SpMV entry point for callers that cannot allocate.

Some callers have no way to hand the library an external buffer at the moment they need a product -
their device memory was fixed at start-up, or an outer framework owns the allocator - so this entry
point keeps the plan and the carries in a device array built into the library.  The test calls it
through the C ABI, twice in a row on different matrices (the second call meets the first call's
leftovers in the shared scratch), and checks each result against aclsparseSpMV with an external
buffer, with the tolerance of the other SpMV tests, and against the fp64 truth.  The file sorts
last so that a run that stops at the first failure has already run every other test.
"""
from ctypes import c_void_p

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import workloads  # noqa: E402
from tests.gpu_util import SpmvCase, dev  # noqa: E402

RTOL, ATOL = 1e-5, 1e-6


def _call(cfg, arrays, alpha, beta, base):
    d_rp, d_ci, d_va, d_x, d_y = arrays
    st = L.lib().aclsparseB200SpMVNoAlloc(
        c_void_p(torch.cuda.current_stream().cuda_stream or 0x1), cfg["rows"], cfg["cols"], cfg["nnz"],
        c_void_p(d_rp.data_ptr()), c_void_p(d_ci.data_ptr()), c_void_p(d_va.data_ptr()), base,
        c_void_p(d_x.data_ptr()), c_void_p(d_y.data_ptr()), alpha, beta)
    assert st == L.SUCCESS, L.STATUS_NAMES.get(st, st)
    torch.cuda.synchronize()


def _no_alloc(cfg, alpha, beta, base=0):
    """One product through the entry point.  The first call on a device may load the library's device code and
    look up the scratch (that can take device memory once); after a warm-up call the free device memory the
    driver reports (cudaMemGetInfo, which sees every allocation, not only PyTorch's) must not move."""
    arrays = (dev(cfg["row_ptr"] + base), dev(cfg["col_ind"] + base), dev(cfg["values"]), dev(cfg["x"]), dev(cfg["y"]))
    _call(cfg, arrays, alpha, beta, base)                       # warm-up: result discarded below
    arrays[4].copy_(torch.from_numpy(cfg["y"]))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    _call(cfg, arrays, alpha, beta, base)
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_reserved() == reserved_before     # PyTorch itself took nothing in between
    assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes during the call"
    return arrays[4].cpu().numpy()


def test_matches_the_buffered_entry_point_twice_in_a_row():
    cases = [(workloads.make("c3", rows=1 << 15), 1.5, 0.5, 0), (workloads.make("c2", rows=30 ** 3), 1.0, 0.0, 1),
             (workloads.make("c1"), -0.5, 2.0, 0)]
    for cfg, alpha, beta, base in cases:
        got = _no_alloc(cfg, alpha, beta, base)
        ref = SpmvCase(cfg["row_ptr"] + base, cfg["col_ind"] + base, cfg["values"], cfg["x"], cfg["y"],
                       base=base).run(alpha, beta)
        np.testing.assert_allclose(got, ref, rtol=RTOL, atol=ATOL)
        truth = O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], alpha, beta)
        bad, max_abs, _ = O.check_tolerance(got, truth, RTOL, ATOL)
        assert bad == 0, (cfg["name"], bad, max_abs)


def test_refuses_what_does_not_fit():
    lib = L.lib()
    fake = c_void_p(0x10000)
    stream = c_void_p(0x1)
    # 4 M rows need 16 MB of row offsets alone: more than the built-in scratch
    st = lib.aclsparseB200SpMVNoAlloc(stream, 4 << 20, 4 << 20, 1 << 20, fake, fake, fake, 0, fake, fake, 1.0, 0.0)
    assert st == L.INSUFFICIENT_RESOURCES
    assert lib.aclsparseB200SpMVNoAlloc(stream, -1, 4, 0, fake, fake, fake, 0, fake, fake, 1.0, 0.0) == L.INVALID_VALUE
    assert lib.aclsparseB200SpMVNoAlloc(stream, 4, 4, 2, None, fake, fake, 0, fake, fake, 1.0, 0.0) == L.INVALID_VALUE
    assert lib.aclsparseB200SpMVNoAlloc(stream, 0, 4, 0, None, None, None, 0, fake, None, 1.0, 0.0) == L.SUCCESS
