"""The plan API (aclsparseSpMVOp_*, aclsparseSpMMOp_*) on the GPU, through the C ABI, against the oracle.

Shapes follow the reference's CSV cases for SpMVOp (test/spmv_op/arch35/spmv_op_test.csv: square and
rectangular matrices from 1 x 1 to tens of thousands of rows, densities from empty to dense rows, every
algorithm value, alpha / beta in {0, 1, other}) and its SpMMOp cases (test/spmm_op/): the golden is the
fp64 truth, the tolerance |got - truth| <= 1e-6 + 1e-5 |truth| on every element, and reruns are bit-equal.
"""
import ctypes
from ctypes import byref, c_float, c_size_t, c_void_p

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import api  # noqa: E402
from tests.gpu_util import dev, random_csr  # noqa: E402

SPMVOP_ALGS = (0, 1, 2)      # DEFAULT, ALG1, ALG2
SPMMOP_ALGS = (0, 1, 2, 3)   # DEFAULT, ALG1, ALG2, ALG1_HIGH_PRECISION


def assert_close(got, truth, what=""):
    bad, max_abs, max_rel = O.check_tolerance(got, truth, 1e-5, 1e-6)
    assert bad == 0, f"{what}: {bad} of {got.size} outside tolerance (max abs {max_abs:.3e}, max rel {max_rel:.3e})"


def fptr(v):
    c = c_float(v)
    return c, ctypes.cast(byref(c), c_void_p)


class SpMVOp:
    """bufferSize -> createDescr -> createPlan, then execute as often as wanted."""

    def __init__(self, handle, mat, x, y, z, alg):
        lib = L.lib()
        self.lib, self.handle = lib, handle
        size = c_size_t(0)
        api.check("bufferSize", lib.aclsparseSpMVOp_bufferSize(handle.raw, L.OP_N, mat.raw, x.raw, y.raw, z.raw,
                                                               L.ACL_FLOAT, alg, byref(size)))
        self.buffer = torch.empty(max(size.value, 64), dtype=torch.uint8, device="cuda:0")
        self.descr, self.plan = c_void_p(None), c_void_p(None)
        api.check("createDescr", lib.aclsparseSpMVOp_createDescr(handle.raw, byref(self.descr), L.OP_N, mat.raw, x.raw,
                                                                 y.raw, z.raw, L.ACL_FLOAT, alg,
                                                                 c_void_p(self.buffer.data_ptr())))
        api.check("createPlan", lib.aclsparseSpMVOp_createPlan(handle.raw, self.descr, byref(self.plan), None, 0))
        api.check("setGlobalUserData", lib.aclsparseSpMVOp_setGlobalUserData(handle.raw, self.plan, b"x", None, 0))

    def __call__(self, alpha, beta, x, y, z):
        ka, pa = fptr(alpha)
        kb, pb = fptr(beta)
        api.check("SpMVOp", self.lib.aclsparseSpMVOp(self.handle.raw, self.plan, pa, pb, x.raw, y.raw, z.raw))

    def close(self):
        assert self.lib.aclsparseSpMVOp_destroyPlan(self.plan) == L.SUCCESS
        assert self.lib.aclsparseSpMVOp_destroyDescr(self.descr) == L.SUCCESS


@pytest.mark.parametrize("alg", SPMVOP_ALGS)
@pytest.mark.parametrize("rows,cols,mean", [(1, 1, 1), (7, 5, 2), (100, 300, 0), (1000, 1000, 10), (4096, 2048, 40),
                                            (20000, 20000, 5), (300, 20000, 900)])
def test_spmvop_vs_oracle(rows, cols, mean, alg):
    rng = np.random.default_rng(rows * 7 + cols + alg)
    lengths = np.minimum(rng.poisson(mean, rows), cols)
    rp, ci = random_csr(rng, lengths, cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    y = rng.uniform(-1, 1, rows).astype(np.float32)
    d_rp, d_x, d_y = dev(rp, np.int32), dev(x), dev(y)
    d_ci = dev(ci, np.int32) if ci.size else None
    d_va = dev(va) if ci.size else None
    d_z = torch.full((rows,), 7.0, device="cuda:0")
    h = api.Handle()
    mat = api.CsrMatrix(rows, cols, d_rp, d_ci, d_va, nnz=ci.size)
    vx, vy, vz = api.DnVec(d_x), api.DnVec(d_y), api.DnVec(d_z)
    op = SpMVOp(h, mat, vx, vy, vz, alg)
    for alpha, beta in ((1.0, 0.0), (0.0, 1.0), (1.5, -0.5)):
        d_z.fill_(7.0)
        op(alpha, beta, vx, vy, vz)
        torch.cuda.synchronize()
        got = d_z.cpu().numpy()
        assert_close(got, O.spmv_f64(rp, ci, va, x, y, alpha, beta), f"{rows}x{cols} alg={alg} {alpha},{beta}")
        assert np.array_equal(d_y.cpu().numpy(), y)          # Y is an input only
        op(alpha, beta, vx, vy, vz)                           # bit-wise reproducible
        torch.cuda.synchronize()
        assert np.array_equal(d_z.cpu().numpy().view(np.uint32), got.view(np.uint32))
    # Z may be Y: then Y is updated in place
    op(2.0, 3.0, vx, vy, vy)
    torch.cuda.synchronize()
    assert_close(d_y.cpu().numpy(), O.spmv_f64(rp, ci, va, x, y, 2.0, 3.0), "Z is Y")
    op.close()


def test_spmvop_new_values_and_unbound_y():
    """Values written into the bound array after createDescr are used by the next execute; with beta == 0 the
    vector Y may have no storage."""
    rng = np.random.default_rng(3)
    rows = cols = 3000
    rp, ci = random_csr(rng, rng.integers(0, 20, rows), cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    d_rp, d_ci, d_va, d_x = dev(rp, np.int32), dev(ci, np.int32), dev(va), dev(x)
    d_z = torch.zeros(rows, device="cuda:0")
    h = api.Handle()
    mat = api.CsrMatrix(rows, cols, d_rp, d_ci, d_va, nnz=ci.size)
    vx, vz = api.DnVec(d_x), api.DnVec(d_z)
    vy = api.DnVec(None, size=rows)
    op = SpMVOp(h, mat, vx, vy, vz, 2)
    op(1.0, 0.0, vx, vy, vz)
    torch.cuda.synchronize()
    assert_close(d_z.cpu().numpy(), O.spmv_f64(rp, ci, va, x, np.zeros(rows, np.float32)), "unbound Y")
    d_va.mul_(-2.0)
    op(1.0, 0.0, vx, vy, vz)
    torch.cuda.synchronize()
    assert_close(d_z.cpu().numpy(), O.spmv_f64(rp, ci, -2.0 * va, x, np.zeros(rows, np.float32)), "new values")
    ka, pa = fptr(1.0)
    kb, pb = fptr(0.5)
    assert L.lib().aclsparseSpMVOp(h.raw, op.plan, pa, pb, vx.raw, vy.raw, vz.raw) == L.INVALID_VALUE  # beta != 0 needs Y
    op.close()


def test_spmvop_argument_checks():
    lib = L.lib()
    rng = np.random.default_rng(4)
    rp, ci = random_csr(rng, rng.integers(0, 5, 10), 10)
    d_rp, d_ci, d_va = dev(rp, np.int32), dev(ci, np.int32), dev(np.ones(ci.size, np.float32))
    d_x, d_y = dev(np.ones(10, np.float32)), dev(np.ones(10, np.float32))
    h = api.Handle()
    mat = api.CsrMatrix(10, 10, d_rp, d_ci, d_va, nnz=ci.size)
    vx, vy = api.DnVec(d_x), api.DnVec(d_y)
    size = c_size_t(0)
    args = (L.OP_N, mat.raw, vx.raw, vy.raw, vy.raw, L.ACL_FLOAT)
    assert lib.aclsparseSpMVOp_bufferSize(None, *args, 0, byref(size)) == L.HANDLE_IS_NULLPTR
    assert lib.aclsparseSpMVOp_bufferSize(h.raw, L.OP_T, *args[1:], 0, byref(size)) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMVOp_bufferSize(h.raw, *args, 9, byref(size)) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMVOp_bufferSize(h.raw, *args, 0, None) == L.INVALID_VALUE
    assert lib.aclsparseSpMVOp_bufferSize(h.raw, L.OP_N, None, *args[2:], 0, byref(size)) == L.INVALID_VALUE
    descr = c_void_p(None)
    assert lib.aclsparseSpMVOp_createDescr(h.raw, byref(descr), *args, 2, None) == L.INVALID_VALUE
    assert lib.aclsparseSpMVOp_createDescr(h.raw, None, *args, 2, None) == L.INVALID_VALUE
    assert lib.aclsparseSpMVOp_destroyDescr(None) == L.SUCCESS and lib.aclsparseSpMVOp_destroyPlan(None) == L.SUCCESS
    op = SpMVOp(h, mat, vx, vy, vy, 1)
    plan = c_void_p(None)
    assert lib.aclsparseSpMVOp_createPlan(h.raw, op.descr, byref(plan), c_void_p(8), 4) == L.NOT_SUPPORTED
    assert lib.aclsparseSpMVOp_createPlan(h.raw, None, byref(plan), None, 0) == L.INVALID_VALUE
    assert lib.aclsparseSpMVOp_setGlobalUserData(h.raw, op.plan, b"n", c_void_p(8), 0) == L.INVALID_VALUE
    ka, pa = fptr(1.0)
    short = api.DnVec(dev(np.ones(4, np.float32)))
    assert lib.aclsparseSpMVOp(h.raw, op.plan, pa, pa, short.raw, vy.raw, vy.raw) == L.INVALID_VALUE
    assert lib.aclsparseSpMVOp(h.raw, None, pa, pa, vx.raw, vy.raw, vy.raw) == L.INVALID_VALUE
    assert lib.aclsparseSpMVOp(h.raw, op.plan, None, pa, vx.raw, vy.raw, vy.raw) == L.INVALID_VALUE
    op.close()


@pytest.mark.parametrize("alg", SPMMOP_ALGS)
@pytest.mark.parametrize("op_b", [L.OP_N, L.OP_T])
def test_spmmop_vs_oracle(alg, op_b):
    """One descriptor, several (B, C) pairs of different widths, both layouts of op(B)."""
    lib = L.lib()
    rng = np.random.default_rng(60 + alg)
    m, k, nmax = 900, 700, 96
    rp, ci = random_csr(rng, np.concatenate([rng.integers(0, 30, m - 1), [600]]), k)
    va = rng.uniform(-1, 1, ci.size).astype(np.float32)
    d_rp, d_ci, d_va = dev(rp, np.int32), dev(ci, np.int32), dev(va)
    h = api.Handle()
    mat = api.CsrMatrix(m, k, d_rp, d_ci, d_va, nnz=ci.size)

    def dense(n):
        b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
        store = np.ascontiguousarray(b.T) if op_b == L.OP_T else b
        d_b, d_c = dev(store), dev(c0)
        mb = api.DnMat(*(store.shape), store.shape[1], d_b)
        mc = api.DnMat(m, n, n, d_c)
        return b, c0, d_b, d_c, mb, mc

    b, c0, d_b, d_c, mb, mc = dense(nmax)
    size = c_size_t(0)
    api.check("bufferSize", lib.aclsparseSpMMOp_bufferSize(h.raw, L.OP_N, op_b, mat.raw, mb.raw, mc.raw, L.ACL_FLOAT,
                                                           alg, byref(size)))
    buf = torch.empty(size.value, dtype=torch.uint8, device="cuda:0")
    descr, plan = c_void_p(None), c_void_p(None)
    api.check("createDescr", lib.aclsparseSpMMOp_createDescr(h.raw, byref(descr), L.OP_N, op_b, mat.raw, mb.raw, mc.raw,
                                                             L.ACL_FLOAT, alg, c_void_p(buf.data_ptr())))
    api.check("createPlan", lib.aclsparseSpMMOp_createPlan(h.raw, descr, byref(plan), None, 0))
    ka, pa = fptr(0.75)
    kb, pb = fptr(-0.5)
    for n in (nmax, 64, 5):
        if n != nmax:
            b, c0, d_b, d_c, mb, mc = dense(n)
        api.check("SpMMOp", lib.aclsparseSpMMOp(h.raw, plan, pa, pb, mb.raw, mc.raw))
        torch.cuda.synchronize()
        assert_close(d_c.cpu().numpy(), O.spmm_f64(rp, ci, va, b, n, c0, n, n, k, 0.75, -0.5), f"n={n} alg={alg}")
    wide = dense(nmax + 8)
    assert lib.aclsparseSpMMOp(h.raw, plan, pa, pb, wide[4].raw, wide[5].raw) == L.INVALID_VALUE
    assert lib.aclsparseSpMMOp(h.raw, None, pa, pb, mb.raw, mc.raw) == L.INVALID_VALUE
    assert lib.aclsparseSpMMOp_destroyPlan(plan) == L.SUCCESS and lib.aclsparseSpMMOp_destroyDescr(descr) == L.SUCCESS
    assert lib.aclsparseSpMMOp_destroyPlan(None) == L.SUCCESS and lib.aclsparseSpMMOp_destroyDescr(None) == L.SUCCESS
    assert lib.aclsparseSpMMOp_bufferSize(h.raw, L.OP_T, op_b, mat.raw, mb.raw, mc.raw, L.ACL_FLOAT, alg,
                                          byref(size)) == L.NOT_SUPPORTED
