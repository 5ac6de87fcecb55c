"""Host logic of the C API without a GPU: every status below is decided before anything is launched.

The cases replay the reference's parameter-validation tests
(test/spmv/arch35/spmv_test.cpp:235-314,474-568; test/spmm/arch35/spmm_test.cpp:783-784 and the
status lists in sparse/spmv/README.md, sparse/spmm/README.md).  Device pointers are fake
addresses: a correct implementation never dereferences them on the host.
"""
import ctypes
import os
import re
from ctypes import byref, c_float, c_int, c_int64, c_size_t, c_void_p

import pytest

from ops_sparse_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE = [c_void_p(0x10000 + 0x1000 * i) for i in range(16)]  # distinct, 64-byte aligned fake device addresses
STREAM = c_void_p(0x5000)


def f32(v):
    return ctypes.cast(byref(c_float(v)), c_void_p)


@pytest.fixture()
def handle(lib):
    h = c_void_p(None)
    assert lib.aclsparseCreate(byref(h)) == L.SUCCESS
    assert lib.aclsparseSetStream(h, STREAM) == L.SUCCESS
    yield h
    # the fake stream must not be synchronised on destroy
    lib.aclsparseSetStream(h, None)
    assert lib.aclsparseDestroy(h) == L.SUCCESS


def make_csr(lib, rows=2, cols=3, nnz=3, ptrs=FAKE[0], idx=FAKE[1], val=FAKE[2], ptype=L.INDEX_32I,
             itype=L.INDEX_32I, base=L.BASE_ZERO, dtype=L.ACL_FLOAT, expect=L.SUCCESS):
    d = c_void_p(None)
    assert lib.aclsparseCreateCsr(byref(d), rows, cols, nnz, ptrs, idx, val, ptype, itype, base, dtype) == expect
    return d


def make_vec(lib, size, values=FAKE[3], dtype=L.ACL_FLOAT):
    d = c_void_p(None)
    assert lib.aclsparseCreateDnVec(byref(d), size, values, dtype) == L.SUCCESS
    return d


def make_mat(lib, rows, cols, ld, values=FAKE[5], order=L.ORDER_ROW, dtype=L.ACL_FLOAT, expect=L.SUCCESS):
    d = c_void_p(None)
    assert lib.aclsparseCreateDnMat(byref(d), rows, cols, ld, values, dtype, order) == expect
    return d


# ------------------------------------------------------------------ ABI --

def declared_functions():
    names = set()
    for header in ("cann_ops_sparse.h", "aclsparse_b200_ext.h", "aclsparse_b200_kernels.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(aclsparse[A-Za-z0-9_]+|spm[vm]_b200_[a-z_]+|aclsp_b200_[a-z_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 55
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"
    assert set(L.SIGNATURES) == set(names)


# --------------------------------------------------------------- handle --

def test_handle_lifecycle(lib):
    assert lib.aclsparseCreate(None) == L.HANDLE_IS_NULLPTR
    h = c_void_p(None)
    assert lib.aclsparseCreate(byref(h)) == L.SUCCESS
    assert lib.aclsparseCreate(byref(h)) == L.INVALID_VALUE  # *handle must be NULL on entry
    ver = c_int(0)
    assert lib.aclsparseGetVersion(None, byref(ver)) == L.SUCCESS and ver.value == 10000
    assert lib.aclsparseGetVersion(h, None) == L.INVALID_VALUE
    mode = c_int(-1)
    assert lib.aclsparseGetPointerMode(h, byref(mode)) == L.SUCCESS and mode.value == L.POINTER_MODE_HOST
    assert lib.aclsparseSetPointerMode(h, 7) == L.INVALID_VALUE
    assert lib.aclsparseSetPointerMode(h, L.POINTER_MODE_DEVICE) == L.SUCCESS
    assert lib.aclsparseGetPointerMode(None, byref(mode)) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseGetPointerMode(h, None) == L.INVALID_VALUE
    s = c_void_p(1)
    assert lib.aclsparseGetStream(h, byref(s)) == L.SUCCESS and s.value is None
    assert lib.aclsparseGetStream(h, None) == L.INVALID_VALUE
    assert lib.aclsparseSetStream(None, STREAM) == L.HANDLE_IS_NULLPTR
    # user workspace: grow-only, NULL switches back
    ws, size = c_void_p(None), c_size_t(0)
    assert lib.aclsparseSetWorkspace(h, FAKE[0], 0) == L.INVALID_VALUE
    assert lib.aclsparseSetWorkspace(h, FAKE[0], 1024) == L.SUCCESS
    assert lib.aclsparseSetWorkspace(h, FAKE[1], 512) == L.SUCCESS
    assert lib.aclsparseGetWorkspace(h, byref(ws), byref(size)) == L.SUCCESS
    assert (ws.value, size.value) == (FAKE[0].value, 1024)
    assert lib.aclsparseSetWorkspace(h, FAKE[1], 4096) == L.SUCCESS
    assert lib.aclsparseGetWorkspace(h, byref(ws), byref(size)) == L.SUCCESS
    assert (ws.value, size.value) == (FAKE[1].value, 4096)
    assert lib.aclsparseGetWorkspace(h, None, byref(size)) == L.INVALID_VALUE
    # a foreign pointer is rejected by its signature
    junk = (ctypes.c_uint32 * 64)()
    assert lib.aclsparseSetStream(ctypes.cast(junk, c_void_p), STREAM) == L.INVALID_VALUE
    assert lib.aclsparseDestroy(None) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseDestroy(h) == L.SUCCESS


# ---------------------------------------------------------- descriptors --

def test_dnvec_descriptor(lib):
    d = c_void_p(None)
    assert lib.aclsparseCreateDnVec(None, 3, FAKE[0], L.ACL_FLOAT) == L.INVALID_VALUE
    assert lib.aclsparseCreateDnVec(byref(d), -1, FAKE[0], L.ACL_FLOAT) == L.INVALID_VALUE
    assert lib.aclsparseCreateDnVec(byref(d), 3, FAKE[0], 12345) == L.INVALID_VALUE
    assert lib.aclsparseCreateDnVec(byref(d), 3, None, L.ACL_FLOAT) == L.SUCCESS  # storage may be bound later
    size, vals, dt = c_int64(0), c_void_p(1), c_int(-1)
    assert lib.aclsparseDnVecGet(d, byref(size), byref(vals), byref(dt)) == L.SUCCESS
    assert (size.value, vals.value, dt.value) == (3, None, L.ACL_FLOAT)
    assert lib.aclsparseDnVecGet(d, None, None, None) == L.SUCCESS  # every OUT pointer is optional
    assert lib.aclsparseDnVecSetValues(d, FAKE[4]) == L.SUCCESS
    assert lib.aclsparseDnVecGetValues(d, byref(vals)) == L.SUCCESS and vals.value == FAKE[4].value
    assert lib.aclsparseDnVecGetValues(d, None) == L.INVALID_VALUE
    stride = c_int64(0)
    assert lib.aclsparseDnVecSetStride(d, 0) == L.INVALID_VALUE
    assert lib.aclsparseDnVecSetStride(d, 5) == L.SUCCESS
    assert lib.aclsparseDnVecGetStride(d, byref(stride)) == L.SUCCESS and stride.value == 5
    # wrong descriptor kind
    m = make_csr(lib)
    assert lib.aclsparseDnVecGet(m, None, None, None) == L.INVALID_VALUE
    assert lib.aclsparseDestroyDnVec(m) == L.INVALID_VALUE
    assert lib.aclsparseDestroySpMat(m) == L.SUCCESS
    assert lib.aclsparseDestroyDnVec(None) == L.SUCCESS
    assert lib.aclsparseDestroyDnVec(d) == L.SUCCESS


def test_csr_descriptor(lib):
    d = c_void_p(None)
    args = (FAKE[0], FAKE[1], FAKE[2], L.INDEX_32I, L.INDEX_32I, L.BASE_ZERO, L.ACL_FLOAT)
    assert lib.aclsparseCreateCsr(None, 2, 3, 3, *args) == L.INVALID_VALUE
    assert lib.aclsparseCreateCsr(byref(d), -2, 3, 3, *args) == L.INVALID_VALUE
    assert lib.aclsparseCreateCsr(byref(d), 2, 3, -1, *args) == L.INVALID_VALUE
    make_csr(lib, ptype=5, expect=L.NOT_SUPPORTED)
    make_csr(lib, base=2, expect=L.INVALID_VALUE)
    make_csr(lib, dtype=999, expect=L.INVALID_VALUE)
    d = make_csr(lib, ptrs=None, idx=None, val=None)  # delayed binding
    rows, cols, nnz = c_int64(0), c_int64(0), c_int64(0)
    assert lib.aclsparseSpMatGetSize(d, byref(rows), byref(cols), byref(nnz)) == L.SUCCESS
    assert (rows.value, cols.value, nnz.value) == (2, 3, 3)
    fmt, base = c_int(-1), c_int(-1)
    assert lib.aclsparseSpMatGetFormat(d, byref(fmt)) == L.SUCCESS and fmt.value == L.FORMAT_CSR
    assert lib.aclsparseSpMatGetIndexBase(d, byref(base)) == L.SUCCESS and base.value == L.BASE_ZERO
    assert lib.aclsparseCsrSetPointers(d, None, FAKE[1], FAKE[2]) == L.INVALID_VALUE
    assert lib.aclsparseCsrSetPointers(d, FAKE[0], None, FAKE[2]) == L.INVALID_VALUE
    assert lib.aclsparseCsrSetPointers(d, FAKE[0], FAKE[1], FAKE[2]) == L.SUCCESS
    p0, p1, p2 = c_void_p(None), c_void_p(None), c_void_p(None)
    t0, t1, vt = c_int(-1), c_int(-1), c_int(-1)
    assert lib.aclsparseCsrGet(d, byref(rows), None, None, byref(p0), byref(p1), byref(p2), byref(t0), byref(t1),
                               byref(base), byref(vt)) == L.SUCCESS
    assert (p0.value, p1.value, p2.value) == (FAKE[0].value, FAKE[1].value, FAKE[2].value)
    assert lib.aclsparseSpMatSetValues(d, FAKE[7]) == L.SUCCESS
    assert lib.aclsparseSpMatGetValues(d, byref(p2)) == L.SUCCESS and p2.value == FAKE[7].value
    s0, s1, s2 = c_int64(0), c_int64(0), c_int64(0)
    assert lib.aclsparseCsrSetStrides(d, 2, 0, 1) == L.INVALID_VALUE
    assert lib.aclsparseCsrSetStrides(d, 2, 3, 4) == L.SUCCESS
    assert lib.aclsparseCsrGetStrides(d, byref(s0), byref(s1), byref(s2)) == L.SUCCESS
    assert (s0.value, s1.value, s2.value) == (2, 3, 4)
    assert lib.aclsparseCsrGetStrides(d, None, byref(s1), byref(s2)) == L.INVALID_VALUE
    assert lib.aclsparseDestroySpMat(None) == L.SUCCESS
    assert lib.aclsparseDestroySpMat(d) == L.SUCCESS


def test_dnmat_descriptor(lib):
    make_mat(lib, -1, 2, 2, expect=L.INVALID_VALUE)
    make_mat(lib, 2 ** 31, 2, 2, expect=L.INVALID_VALUE)
    make_mat(lib, 3, 2, 1, expect=L.INVALID_VALUE)                      # row-major needs ld >= cols
    make_mat(lib, 3, 2, 2, order=L.ORDER_COL, expect=L.INVALID_VALUE)   # column-major needs ld >= rows
    make_mat(lib, 3, 2, 2, values=None, expect=L.INVALID_VALUE)
    make_mat(lib, 3, 2, 2, order=9, expect=L.INVALID_VALUE)
    lib.aclsparseDestroyDnMat(make_mat(lib, 0, 2, 2, values=None))      # empty matrices need no storage
    d = make_mat(lib, 3, 2, 4)
    rows, cols, ld, vals, dt, order = c_int64(0), c_int64(0), c_int64(0), c_void_p(None), c_int(-1), c_int(-1)
    assert lib.aclsparseDnMatGet(d, byref(rows), byref(cols), byref(ld), byref(vals), byref(dt),
                                 byref(order)) == L.SUCCESS
    assert (rows.value, cols.value, ld.value, vals.value, order.value) == (3, 2, 4, FAKE[5].value, L.ORDER_ROW)
    cnt, bstride = c_int(0), c_int64(-1)
    assert lib.aclsparseDnMatGetStridedBatch(d, byref(cnt), byref(bstride)) == L.SUCCESS
    assert (cnt.value, bstride.value) == (1, 0)
    assert lib.aclsparseDnMatSetStridedBatch(d, 0, 0) == L.INVALID_VALUE
    assert lib.aclsparseDnMatSetStridedBatch(d, 4, 5) == L.INVALID_VALUE   # stride shorter than one matrix
    assert lib.aclsparseDnMatSetStridedBatch(d, 4, 12) == L.SUCCESS
    assert lib.aclsparseDnMatSetValues(d, FAKE[6]) == L.SUCCESS
    assert lib.aclsparseDestroyDnMat(d) == L.SUCCESS
    assert lib.aclsparseDestroyDnMat(None) == L.SUCCESS


# ----------------------------------------------------------------- SpMV --

def spmv_args(handle, mat, x, y, alpha=None, beta=None, op=L.OP_N, ctype=L.ACL_FLOAT, alg=L.SPMV_ALG_DEFAULT):
    return (handle, op, alpha if alpha is not None else f32(1.0), mat, x, beta if beta is not None else f32(0.0), y,
            ctype, alg)


def test_spmv_buffer_size_and_status_precedence(lib, handle):
    mat, x, y = make_csr(lib), make_vec(lib, 3), make_vec(lib, 2, FAKE[4])
    size = c_size_t(7)
    # bufferSize == NULL is checked first and *bufferSize is zeroed before anything else
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(None, mat, x, y), None) == L.INVALID_VALUE
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(None, mat, x, y), byref(size)) == L.HANDLE_IS_NULLPTR
    assert size.value == 0
    junk = ctypes.cast((ctypes.c_uint32 * 64)(), c_void_p)
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(junk, mat, x, y), byref(size)) == L.INVALID_VALUE
    h2 = c_void_p(None)
    lib.aclsparseCreate(byref(h2))  # no stream set
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(h2, mat, x, y), byref(size)) == L.INVALID_VALUE
    lib.aclsparseDestroy(h2)
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, None, x, y), byref(size)) == L.INVALID_VALUE
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, x, x, y), byref(size)) == L.INVALID_VALUE
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y, op=5), byref(size)) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y, ctype=L.ACL_DOUBLE),
                                          byref(size)) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y, alg=L.SPMV_COO_ALG1),
                                          byref(size)) == L.NOT_SUPPORTED
    # NULL and misaligned scalars
    args = list(spmv_args(handle, mat, x, y))
    args[2] = None
    assert lib.aclsparseSpMVGetBufferSize(*args, byref(size)) == L.INVALID_VALUE
    buf = (ctypes.c_char * 16)()
    args[2] = c_void_p(ctypes.addressof(buf) + 1)
    assert lib.aclsparseSpMVGetBufferSize(*args, byref(size)) == L.INVALID_VALUE
    # vector sizes must match exactly
    x_bad = make_vec(lib, 4)
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x_bad, y), byref(size)) == L.INVALID_VALUE
    # int64 indices, other dtypes, transposed A
    m64 = make_csr(lib, ptype=L.INDEX_64I, itype=L.INDEX_64I)
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, m64, x, y), byref(size)) == L.NOT_SUPPORTED
    mh = make_csr(lib, dtype=L.ACL_FLOAT16)
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mh, x, y), byref(size)) == L.NOT_SUPPORTED
    # op(A) = T / H: x has one entry per row of A and y one per column; the buffer also holds the transpose
    xt, yt = make_vec(lib, 2), make_vec(lib, 3, FAKE[4])
    from oracle import oracle as O
    for op in (L.OP_T, L.OP_H):
        assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, xt, yt, op=op), byref(size)) == L.SUCCESS
        assert size.value == O.transpose_plan_layout(3, 3, O.spmv_plan_layout(3, 3)["total_bytes"])["total_bytes"]
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y, op=L.OP_T), byref(size)) == L.INVALID_VALUE
    # the three accepted algorithms, and unbound storage is fine for a size query
    unbound = make_csr(lib, ptrs=None, idx=None, val=None)
    xu, yu = make_vec(lib, 3, None), make_vec(lib, 2, None)
    for alg in (L.SPMV_ALG_DEFAULT, L.SPMV_CSR_ALG1, L.SPMV_CSR_ALG2):
        assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, unbound, xu, yu, alg=alg), byref(size)) == L.SUCCESS
        assert size.value >= 64 and size.value % 64 == 0
    # nnz > 0 with a zero dimension
    z = make_csr(lib, rows=0, cols=2, nnz=1, ptrs=None, idx=None, val=None)
    x2, y0 = make_vec(lib, 2, None), make_vec(lib, 0, None)
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, z, x2, y0), byref(size)) == L.INVALID_VALUE
    # strides are part of the descriptor and accepted (reference: spmv_test.cpp:269-272)
    assert lib.aclsparseCsrSetStrides(mat, 2, 1, 1) == L.SUCCESS
    assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y), byref(size)) == L.SUCCESS


def test_spmv_buffer_size_formula(lib, handle):
    from oracle import oracle as O
    for rows, nnz in ((2, 3), (1, 0), (4096, 100000), (100000, 7)):
        mat = make_csr(lib, rows=rows, cols=rows + 1, nnz=nnz)
        x, y = make_vec(lib, rows + 1), make_vec(lib, rows, FAKE[4])
        size = c_size_t(0)
        assert lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y), byref(size)) == L.SUCCESS
        lay = O.spmv_plan_layout(rows, nnz)
        assert size.value == lay["total_bytes"]
        # the reference's own buffer (header + row offsets) is a prefix of ours
        assert lay["tile_row_off"] == O.ref_spmv_workspace_bytes(rows)


def test_spmv_execute_validation(lib, handle):
    mat, x, y = make_csr(lib), make_vec(lib, 3), make_vec(lib, 2, FAKE[4])
    ws = FAKE[8]
    a = spmv_args(handle, mat, x, y)
    assert lib.aclsparseSpMV(*a, None) == L.INSUFFICIENT_RESOURCES
    assert lib.aclsparseSpMV(*a, c_void_p(ws.value + 1)) == L.INVALID_VALUE
    assert lib.aclsparseSpMVPreprocess(*a, None) == L.INSUFFICIENT_RESOURCES
    assert lib.aclsparseSpMVPreprocess(*a, c_void_p(ws.value + 8)) == L.INVALID_VALUE
    # unbound storage
    unbound = make_csr(lib, ptrs=None, idx=None, val=None)
    assert lib.aclsparseSpMVPreprocess(*spmv_args(handle, unbound, x, y), ws) == L.INVALID_VALUE
    novals = make_csr(lib, val=None)
    assert lib.aclsparseSpMV(*spmv_args(handle, novals, x, y), ws) == L.INVALID_VALUE
    xu = make_vec(lib, 3, None)
    assert lib.aclsparseSpMV(*spmv_args(handle, mat, xu, y), ws) == L.INVALID_VALUE
    # exact aliases among the CSR arrays, x and y
    y_alias = make_vec(lib, 2, FAKE[3])
    assert lib.aclsparseSpMV(*spmv_args(handle, mat, x, y_alias), ws) == L.INVALID_VALUE
    m_alias = make_csr(lib, idx=FAKE[0])
    assert lib.aclsparseSpMV(*spmv_args(handle, m_alias, x, y), ws) == L.INVALID_VALUE
    # nothing to write: silent success without a launch
    empty = make_csr(lib, rows=0, cols=3, nnz=0, ptrs=None, idx=None, val=None)
    y0 = make_vec(lib, 0, None)
    assert lib.aclsparseSpMV(*spmv_args(handle, empty, x, y0), ws) == L.SUCCESS


# ----------------------------------------------------------------- SpMM --

def spmm_args(handle, mat, b, c, alpha=None, beta=None, op_a=L.OP_N, op_b=L.OP_N, ctype=L.ACL_FLOAT,
              alg=L.SPMM_ALG_DEFAULT):
    return (handle, op_a, op_b, alpha if alpha is not None else f32(1.0), mat, b,
            beta if beta is not None else f32(0.0), c, ctype, alg)


def test_spmm_status_precedence(lib, handle):
    mat = make_csr(lib, rows=4, cols=3, nnz=5)
    b, c = make_mat(lib, 3, 2, 2), make_mat(lib, 4, 2, 2, values=FAKE[6])
    size = c_size_t(0)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(None, mat, b, c), byref(size)) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c), None) == L.INVALID_VALUE
    args = list(spmm_args(handle, mat, b, c))
    args[3] = None
    assert lib.aclsparseSpMMGetBufferSize(*args, byref(size)) == L.INVALID_VALUE
    # a NULL descriptor is reported as a NULL handle by SpMM (reference: spmm_host.cpp:479-482)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, None, b, c), byref(size)) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c, alg=9), byref(size)) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c, op_b=7), byref(size)) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c, op_a=L.OP_T, alg=L.SPMM_CSR_ALG3),
                                          byref(size)) == L.NOT_SUPPORTED
    m64 = make_csr(lib, rows=4, cols=3, nnz=5, ptype=L.INDEX_64I)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, m64, b, c), byref(size)) == L.NOT_SUPPORTED
    mh = make_csr(lib, rows=4, cols=3, nnz=5, dtype=L.ACL_FLOAT16)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mh, b, c), byref(size)) == L.NOT_SUPPORTED
    b_bad = make_mat(lib, 5, 2, 2)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b_bad, c), byref(size)) == L.INVALID_VALUE
    unbound = make_csr(lib, rows=4, cols=3, nnz=5, val=None)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, unbound, b, c), byref(size)) == L.INVALID_VALUE
    # op(B) = T takes B as n x k
    bt = make_mat(lib, 2, 3, 3)
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, bt, c, op_b=L.OP_T), byref(size)) == L.SUCCESS
    assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c, op_a=L.OP_T), byref(size)) != L.SUCCESS
    for alg in (L.SPMM_ALG_DEFAULT, L.SPMM_CSR_ALG1, L.SPMM_CSR_ALG2, L.SPMM_CSR_ALG3,
                L.SPMM_CSR_FP32_HIGH_PRECISION_ALG):
        assert lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c, alg=alg), byref(size)) == L.SUCCESS
    from oracle import oracle as O
    assert size.value == O.spmm_plan_layout(4, 5, 2)["total_bytes"]
    assert lib.aclsparseSpMM(*spmm_args(handle, mat, b, c), None) == L.INSUFFICIENT_RESOURCES
    assert lib.aclsparseSpMMPreprocess(*spmm_args(handle, mat, b, c), None) == L.INSUFFICIENT_RESOURCES
    assert lib.aclsparseSpMM(*spmm_args(handle, mat, b, c), c_void_p(FAKE[8].value + 4)) == L.INVALID_VALUE


def test_row_block_bounds_validation(lib, handle):
    mat = make_csr(lib)
    assert lib.aclsparseB200RowBlockBounds(None, mat, 2, FAKE[9]) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseB200RowBlockBounds(handle, None, 2, FAKE[9]) == L.INVALID_VALUE
    assert lib.aclsparseB200RowBlockBounds(handle, mat, 0, FAKE[9]) == L.INVALID_VALUE
    assert lib.aclsparseB200RowBlockBounds(handle, mat, 2, None) == L.INVALID_VALUE


def test_mirror_list_validation(lib):
    """aclsparseB200Dn{Vec,Mat}Set[Multicast]Mirror[s]: at most 7 non-null mirrors, right descriptor kind."""
    import ctypes
    vec, mat, csr = make_vec(lib, 8), make_mat(lib, 4, 4, 4), make_csr(lib)
    seven = (c_void_p * 7)(*[FAKE[i].value for i in range(7)])
    eight = (c_void_p * 8)(*[FAKE[i % 7].value for i in range(8)])
    holed = (c_void_p * 2)(FAKE[0].value, None)
    for setter, multi, good, other in ((lib.aclsparseB200DnVecSetMirrors, lib.aclsparseB200DnVecSetMulticastMirror, vec, mat),
                                       (lib.aclsparseB200DnMatSetMirrors, lib.aclsparseB200DnMatSetMulticastMirror, mat, vec)):
        assert setter(good, 7, seven) == L.SUCCESS
        assert setter(good, 8, eight) == L.INVALID_VALUE
        assert setter(good, -1, seven) == L.INVALID_VALUE
        assert setter(good, 2, holed) == L.INVALID_VALUE
        assert setter(good, 1, None) == L.INVALID_VALUE
        assert setter(good, 0, None) == L.SUCCESS  # clears the list
        assert setter(None, 0, None) == L.INVALID_VALUE
        assert setter(other, 0, None) == L.INVALID_VALUE  # wrong descriptor kind
        assert setter(csr, 0, None) == L.INVALID_VALUE
        assert multi(good, FAKE[1]) == L.SUCCESS
        assert multi(good, None) == L.INVALID_VALUE
        assert multi(other, FAKE[1]) == L.INVALID_VALUE
        assert setter(good, 0, None) == L.SUCCESS
    assert lib.aclsparseDestroyDnVec(vec) == L.SUCCESS
    assert lib.aclsparseDestroyDnMat(mat) == L.SUCCESS
    assert lib.aclsparseDestroySpMat(csr) == L.SUCCESS


def test_dtype_tables(lib, handle):
    """The supported element-type combinations are the reference's tables without the complex rows
    (sparse/spmv/arch35/spmv_host.cpp:44-66, sparse/spmm/arch35/host/spmm_host.cpp:379-387); everything else is
    NOT_SUPPORTED at the buffer-size query already."""
    F, H, B, I8, I32, C = L.ACL_FLOAT, L.ACL_FLOAT16, L.ACL_BF16, L.ACL_INT8, L.ACL_INT32, L.ACL_COMPLEX64
    size = c_size_t(0)
    spmv_ok = {(F, F, F, F), (H, H, H, F), (H, H, F, F), (B, B, B, F), (B, B, F, F), (I8, I8, F, F), (I8, I8, I32, I32)}
    spmm_ok = {(F, F, F, F), (H, H, H, F), (H, H, F, F), (B, B, B, F), (B, B, F, F), (I8, I8, I32, I32)}
    types = (F, H, B, I8, I32, C)
    for a in types:
        for xb in types:
            for yc in types:
                for ct in (F, I32, C):
                    mat = make_csr(lib, rows=4, cols=3, nnz=5, dtype=a)
                    x, y = make_vec(lib, 3, dtype=xb), make_vec(lib, 4, FAKE[4], dtype=yc)
                    want = L.SUCCESS if (a, xb, yc, ct) in spmv_ok else L.NOT_SUPPORTED
                    got = lib.aclsparseSpMVGetBufferSize(*spmv_args(handle, mat, x, y, ctype=ct), byref(size))
                    assert got == want, ("spmv", a, xb, yc, ct, got)
                    b, c = make_mat(lib, 3, 2, 2, dtype=xb), make_mat(lib, 4, 2, 2, values=FAKE[6], dtype=yc)
                    want = L.SUCCESS if (a, xb, yc, ct) in spmm_ok else L.NOT_SUPPORTED
                    got = lib.aclsparseSpMMGetBufferSize(*spmm_args(handle, mat, b, c, ctype=ct), byref(size))
                    assert got == want, ("spmm", a, xb, yc, ct, got)
                    for d, destroy in ((mat, lib.aclsparseDestroySpMat), (x, lib.aclsparseDestroyDnVec),
                                       (y, lib.aclsparseDestroyDnVec), (b, lib.aclsparseDestroyDnMat),
                                       (c, lib.aclsparseDestroyDnMat)):
                        assert destroy(d) == L.SUCCESS


def test_closing_barrier_validation(lib):
    """aclsparseB200Dn{Vec,Mat}SetClosingBarrier: argument checks; world <= 1 or a NULL state clears it."""
    vec, mat = make_vec(lib, 8), make_mat(lib, 4, 4, 4)
    peers = (c_void_p * 4)(*[FAKE[i].value for i in range(4)])
    holed = (c_void_p * 4)(FAKE[0].value, None, FAKE[2].value, FAKE[3].value)
    for setter, good, other in ((lib.aclsparseB200DnVecSetClosingBarrier, vec, mat),
                                (lib.aclsparseB200DnMatSetClosingBarrier, mat, vec)):
        assert setter(good, FAKE[8], peers, 4, 1, 0) == L.SUCCESS
        assert setter(good, FAKE[8], holed, 4, 1, 0) == L.SUCCESS        # the rank's own entry is not used
        assert setter(good, FAKE[8], holed, 4, 0, 0) == L.INVALID_VALUE  # a peer's entry is
        assert setter(good, FAKE[8], None, 4, 1, 0) == L.INVALID_VALUE
        assert setter(good, FAKE[8], peers, 17, 1, 0) == L.INVALID_VALUE
        assert setter(good, FAKE[8], peers, 4, 4, 0) == L.INVALID_VALUE
        assert setter(good, FAKE[8], peers, 4, -1, 0) == L.INVALID_VALUE
        assert setter(good, None, None, 0, 0, 0) == L.SUCCESS            # cleared
        assert setter(good, FAKE[8], peers, 1, 0, 0) == L.SUCCESS        # one rank: nothing to wait for
        assert setter(None, FAKE[8], peers, 4, 1, 0) == L.INVALID_VALUE
        assert setter(other, FAKE[8], peers, 4, 1, 0) == L.INVALID_VALUE  # wrong descriptor kind
    assert lib.aclsparseDestroyDnVec(vec) == L.SUCCESS
    assert lib.aclsparseDestroyDnMat(mat) == L.SUCCESS


def test_wait_failure_counter_validation(lib):
    count = ctypes.c_uint32(7)
    assert lib.aclsparseB200SpMVWaitFailures(STREAM, None, byref(count)) == L.INVALID_VALUE
    assert lib.aclsparseB200SpMVWaitFailures(STREAM, FAKE[0], None) == L.INVALID_VALUE


def test_create_destroy_loop(lib):
    """Descriptor churn does not accumulate state (the reference's leak loop, spmv_test.cpp:1710-1738)."""
    for _ in range(2000):
        m, x = make_csr(lib), make_vec(lib, 3)
        assert lib.aclsparseDestroySpMat(m) == L.SUCCESS
        assert lib.aclsparseDestroyDnVec(x) == L.SUCCESS


def test_public_headers_are_plain_c(tmp_path):
    """The boundary is a C ABI: the three public headers compile as C99 with no C++ and no CUDA in sight, and the
    parameter blocks have the sizes the ctypes mirrors in ops_sparse_b200/_lib.py assume."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    src = tmp_path / "abi.c"
    src.write_text(
        '#include <stdio.h>\n#include "cann_ops_sparse.h"\n#include "aclsparse_b200_ext.h"\n'
        '#include "aclsparse_b200_kernels.h"\n'
        'int main(void) { printf("%zu %zu %zu %zu\\n", sizeof(AclspSpmvParams), sizeof(AclspSpmmParams), '
        'sizeof(AclspBarrierLink), sizeof(AclspNodeBarrierState)); return 0; }\n')
    exe = tmp_path / "abi"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe)], check=True)
    sizes = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert sizes == [ctypes.sizeof(L.SpmvParams), ctypes.sizeof(L.SpmmParams), ctypes.sizeof(L.BarrierLink), 80]


def test_library_exports_only_its_c_api():
    """Hidden visibility: the dynamic symbol table holds the C entry points and nothing else of this library."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", L.LIB_PATH], capture_output=True, text=True, check=True).stdout
    names = [line.split()[-1] for line in out.splitlines() if line.strip()]
    assert names, "no dynamic symbols found"
    stray = [n for n in names if not (n.startswith("aclsparse") or n.startswith("aclsp_") or "_b200_" in n)]
    assert not stray, f"internal symbols exported: {stray[:10]}"
