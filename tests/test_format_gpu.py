"""aclsparseXcoo2csr and aclsparseXcsrsort on the GPU, bit for bit against their CPU twins, and the chain a
caller with unsorted COO data follows into SpMV: sort by row on the host side of the test, coo2csr, csrsort,
gather the values through P, multiply."""
import ctypes
from ctypes import byref, c_size_t, c_void_p

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import api  # noqa: E402
from tests.gpu_util import SpmvCase, dev  # noqa: E402


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("m,nnz", [(1, 0), (5, 3), (1000, 0), (4097, 50000), (3, 100000), (200000, 150000)])
def test_coo2csr_equals_twin(m, nnz, base):
    rng = np.random.default_rng(m + nnz)
    rows = np.sort(rng.integers(0, m, nnz)).astype(np.int32) + base
    d_rows = dev(rows) if nnz else None
    d_ptr = torch.full((m + 1,), -7, dtype=torch.int32, device="cuda:0")
    h = api.Handle()
    st = L.lib().aclsparseXcoo2csr(h.raw, c_void_p(d_rows.data_ptr()) if nnz else None, nnz, m,
                                   c_void_p(d_ptr.data_ptr()), base)
    assert st == L.SUCCESS
    torch.cuda.synchronize()
    assert np.array_equal(d_ptr.cpu().numpy(), O.coo2csr_twin(rows, m, base))


def test_coo2csr_argument_checks():
    lib = L.lib()
    h = api.Handle()
    fake = c_void_p(0x1000)
    assert lib.aclsparseXcoo2csr(None, fake, 1, 1, fake, 0) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseXcoo2csr(h.raw, fake, -1, 1, fake, 0) == L.INVALID_VALUE
    assert lib.aclsparseXcoo2csr(h.raw, fake, 1, 0, fake, 0) == L.INVALID_VALUE
    assert lib.aclsparseXcoo2csr(h.raw, fake, 1, 1, fake, 2) == L.INVALID_VALUE
    assert lib.aclsparseXcoo2csr(h.raw, None, 1, 1, fake, 0) == L.INVALID_VALUE
    assert lib.aclsparseXcoo2csr(h.raw, fake, 1, 1, None, 0) == L.INVALID_VALUE


def _mat_descr(base):
    lib = L.lib()
    d = c_void_p(None)
    assert lib.aclsparseCreateMatDescr(byref(d)) == L.SUCCESS
    lib.aclsparseSetMatIndexBase(d, base)
    assert lib.aclsparseGetMatIndexBase(d) == base
    return d


@pytest.mark.parametrize("base", [0, 1])
def test_csrsort_equals_twin(base):
    """Short rows, rows beyond a warp, rows beyond shared memory, empty rows, repeated columns (stability)."""
    lib = L.lib()
    rng = np.random.default_rng(70 + base)
    n = 5000
    lengths = np.concatenate([rng.integers(0, 33, 3000), [33, 64, 100, 2048, 2049, 7000], np.zeros(50, int),
                              rng.integers(0, 200, 300)])
    m = lengths.size
    rp = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    nnz = int(rp[-1])
    col = rng.integers(0, n, nnz).astype(np.int32)
    col[rng.integers(0, nnz, nnz // 10)] = 17       # many repeated columns: equal keys must keep their order
    perm = np.arange(nnz, dtype=np.int32)
    d_rp, d_col, d_p = dev(rp + base), dev(col + base), dev(perm)
    h = api.Handle()
    size = c_size_t(0)
    assert lib.aclsparseXcsrsort_bufferSizeExt(h.raw, m, n, nnz, c_void_p(d_rp.data_ptr()), c_void_p(d_col.data_ptr()),
                                               byref(size)) == L.SUCCESS
    assert size.value == 8 * nnz
    buf = torch.empty(size.value, dtype=torch.uint8, device="cuda:0")
    descr = _mat_descr(base)
    assert lib.aclsparseXcsrsort(h.raw, m, n, nnz, descr, c_void_p(d_rp.data_ptr()), c_void_p(d_col.data_ptr()),
                                 c_void_p(d_p.data_ptr()), c_void_p(buf.data_ptr())) == L.SUCCESS
    torch.cuda.synchronize()
    want_col, want_p = O.csrsort_twin(rp + base, col + base, perm, base)
    assert np.array_equal(d_col.cpu().numpy(), want_col)
    assert np.array_equal(d_p.cpu().numpy(), want_p)
    # argument checks
    assert lib.aclsparseXcsrsort(None, m, n, nnz, descr, None, None, None, None) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseXcsrsort(h.raw, -1, n, nnz, descr, None, None, None, None) == L.INVALID_VALUE
    assert lib.aclsparseXcsrsort(h.raw, m, n, nnz, None, c_void_p(d_rp.data_ptr()), c_void_p(d_col.data_ptr()),
                                 c_void_p(d_p.data_ptr()), c_void_p(buf.data_ptr())) == L.INVALID_VALUE
    assert lib.aclsparseXcsrsort(h.raw, m, n, nnz, descr, c_void_p(d_rp.data_ptr()), c_void_p(d_col.data_ptr()),
                                 None, c_void_p(buf.data_ptr())) == L.INVALID_VALUE
    assert lib.aclsparseXcsrsort(h.raw, m, n, 0, descr, c_void_p(d_rp.data_ptr()), None, None, None) == L.SUCCESS
    assert lib.aclsparseDestroyMatDescr(descr) == L.SUCCESS and lib.aclsparseDestroyMatDescr(None) == L.SUCCESS


def test_coo_to_spmv_chain():
    """COO sorted by row only -> coo2csr -> csrsort -> values gathered through P -> SpMV == the oracle."""
    lib = L.lib()
    rng = np.random.default_rng(77)
    m, n, nnz = 3000, 2500, 40000
    rows = np.sort(rng.integers(0, m, nnz)).astype(np.int32)
    cols = rng.integers(0, n, nnz).astype(np.int32)           # unsorted inside a row, repeats allowed
    vals = rng.standard_normal(nnz).astype(np.float32)
    x = rng.standard_normal(n).astype(np.float32)
    h = api.Handle()
    d_rows, d_cols = dev(rows), dev(cols)
    d_ptr = torch.empty(m + 1, dtype=torch.int32, device="cuda:0")
    assert lib.aclsparseXcoo2csr(h.raw, c_void_p(d_rows.data_ptr()), nnz, m, c_void_p(d_ptr.data_ptr()), 0) == L.SUCCESS
    d_p = torch.arange(nnz, dtype=torch.int32, device="cuda:0")
    buf = torch.empty(8 * nnz, dtype=torch.uint8, device="cuda:0")
    descr = _mat_descr(0)
    assert lib.aclsparseXcsrsort(h.raw, m, n, nnz, descr, c_void_p(d_ptr.data_ptr()), c_void_p(d_cols.data_ptr()),
                                 c_void_p(d_p.data_ptr()), c_void_p(buf.data_ptr())) == L.SUCCESS
    torch.cuda.synchronize()
    rp = d_ptr.cpu().numpy()
    sorted_cols = d_cols.cpu().numpy()
    sorted_vals = vals[d_p.cpu().numpy()]
    got = SpmvCase(rp, sorted_cols, sorted_vals, x, np.zeros(m, np.float32)).run(1.0, 0.0)
    truth = O.spmv_f64(O.coo2csr_twin(rows, m), cols, vals, x, np.zeros(m, np.float32))   # order inside a row is free
    bad, max_abs, _ = O.check_tolerance(got, truth)
    assert bad == 0, (bad, max_abs)
