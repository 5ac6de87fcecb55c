"""SpMM with fp16 / bf16 / int8 storage on the GPU, through the C ABI, against the oracle.

The supported combinations are the reference's table (sparse/spmm/arch35/host/spmm_host.cpp:379-387) without its
complex row: A and B of one type, C of that type or fp32, compute type fp32; int8 with an int32 C and the int32
compute type.  Floating results: the fp64 truth rounded once to C's type, up to the summation order.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import api  # noqa: E402
from tests.gpu_util import bits_of, dev, expected_bits, quantize, random_csr, to_device  # noqa: E402


class NarrowSpmm:
    """b and c are (rows x ld) row-major or (cols x ld) column-major storage arrays, as fp32 numbers that the
    storage type holds exactly."""

    def __init__(self, rp, ci, values, k, n, b, ldb, c, ldc, in_kind, out_kind, order_b=L.ORDER_ROW,
                 order_c=L.ORDER_ROW, op_a=L.OP_N, op_b=L.OP_N, base=0):
        rows = len(rp) - 1  # A is rows x k
        m = rows if op_a == L.OP_N else k
        inner = k if op_a == L.OP_N else rows
        self.d_rp, self.d_ci = dev(np.asarray(rp), np.int32), dev(np.asarray(ci), np.int32)
        self.d_va, self.d_b, self.d_c = to_device(values, in_kind), to_device(b, in_kind), to_device(c, out_kind)
        self.handle = api.Handle()
        self.mat = api.CsrMatrix(rows, k, self.d_rp, self.d_ci, self.d_va, base, nnz=len(ci))
        b_rows, b_cols = (inner, n) if op_b == L.OP_N else (n, inner)
        self.mb = api.DnMat(b_rows, b_cols, ldb, self.d_b, order_b)
        self.mc = api.DnMat(m, n, ldc, self.d_c, order_c)
        self.op = api.SpMM(self.handle, self.mat, self.mb, self.mc, op_a=op_a, op_b=op_b)

    def run(self, alpha, beta):
        self.op.preprocess(alpha, beta)
        self.op(alpha, beta)
        torch.cuda.synchronize()
        return bits_of(self.d_c)


def check(got, truth, out_kind, c_storage_mask=None):
    if out_kind == "f32":
        bad, max_abs, max_rel = O.check_tolerance(got, truth, 1e-6, 1e-7)
        assert bad == 0, (max_abs, max_rel)
        return
    want = expected_bits(truth, out_kind)
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3, (diff.max(), (diff != 0).mean())


@pytest.mark.parametrize("in_kind, out_kind", [("f16", "f16"), ("f16", "f32"), ("bf16", "bf16"), ("bf16", "f32")])
@pytest.mark.parametrize("n", [1, 7, 32, 50])
def test_random_matrices_against_truth(in_kind, out_kind, n):
    rng = np.random.default_rng(21 + n)
    m, k = 900, 1300
    lengths = rng.poisson(10, m)
    lengths[5], lengths[6] = 1250, 0
    rp, ci = random_csr(rng, lengths, k)
    va = quantize(rng.standard_normal(ci.size), in_kind)
    ldb, ldc = n + 3, n + 1
    b = quantize(rng.standard_normal((k, ldb)), in_kind)
    c = quantize(rng.uniform(-1, 1, (m, ldc)), out_kind)
    for alpha, beta in [(1.0, 0.0), (-0.75, 0.5)]:
        truth = O.spmm_f64(rp, ci, va, b, ldb, c, ldc, n, k, alpha, beta)
        got = NarrowSpmm(rp, ci, va, k, n, b, ldb, c, ldc, in_kind, out_kind).run(alpha, beta)
        got = got.reshape(m, ldc)
        check(got[:, :n], truth, out_kind)
        # the padding columns of C are not touched
        assert np.array_equal(got[:, n:], bits_of(to_device(c, out_kind)).reshape(m, ldc)[:, n:])


@pytest.mark.parametrize("order_b, order_c, op_b", [(L.ORDER_COL, L.ORDER_ROW, L.OP_N), (L.ORDER_ROW, L.ORDER_COL, L.OP_T),
                                                    (L.ORDER_COL, L.ORDER_COL, L.OP_T)])
def test_layouts_and_transposed_operands(order_b, order_c, op_b):
    rng = np.random.default_rng(4)
    m, k, n = 300, 420, 24
    rp, ci = random_csr(rng, rng.poisson(8, m), k)
    va = quantize(rng.standard_normal(ci.size), "f16")
    # op(B) is k x n; its storage is (rows x ld) for row-major and (cols x ld) for column-major
    b_rows, b_cols = (k, n) if op_b == L.OP_N else (n, k)
    ldb = (b_cols if order_b == L.ORDER_ROW else b_rows) + 2
    b = quantize(rng.standard_normal(((b_rows if order_b == L.ORDER_ROW else b_cols), ldb)), "f16")
    ldc = (n if order_c == L.ORDER_ROW else m) + 1
    c = quantize(rng.uniform(-1, 1, ((m if order_c == L.ORDER_ROW else n), ldc)), "f16")
    # (B's elements are row-major in memory exactly when storage order and op(B) agree)
    truth = O.spmm_f64(rp, ci, va, b, ldb, c, ldc, n, k, 1.25, 0.5,
                       b_row_major=(order_b == L.ORDER_ROW), op_b_transpose=(op_b != L.OP_N),
                       c_row_major=(order_c == L.ORDER_ROW))
    got = NarrowSpmm(rp, ci, va, k, n, b, ldb, c, ldc, "f16", "f16", order_b, order_c, op_b=op_b).run(1.25, 0.5)
    got = got.reshape(c.shape)
    got = got[:, :n] if order_c == L.ORDER_ROW else got[:, :m].T
    check(got, truth, "f16")


def test_transposed_sparse_operand():
    rng = np.random.default_rng(8)
    rows, cols, n = 350, 280, 16  # A is rows x cols; C = A^T B is cols x n, B is rows x n
    rp, ci = random_csr(rng, rng.poisson(7, rows), cols)
    va = quantize(rng.standard_normal(ci.size), "bf16")
    b = quantize(rng.standard_normal((rows, n)), "bf16")
    c = quantize(rng.uniform(-1, 1, (cols, n)), "f32")
    rp_t, ci_t, perm = O.transpose_twin(rp, ci, cols)
    truth = O.spmm_f64(rp_t, ci_t, va[perm], b, n, c, n, n, rows, 2.0, -1.0)
    got = NarrowSpmm(rp, ci, va, cols, n, b, n, c, n, "bf16", "f32", op_a=L.OP_T).run(2.0, -1.0).reshape(cols, n)
    check(got, truth, "f32")


def test_int8_to_int32_exact_and_saturating():
    rng = np.random.default_rng(9)
    m, k, n = 400, 500, 20
    lengths = rng.poisson(9, m)
    lengths[11] = 480
    rp, ci = random_csr(rng, lengths, k)
    va = rng.integers(-127, 128, ci.size).astype(np.int8)
    b = rng.integers(-127, 128, (k, n)).astype(np.int8)
    c = rng.integers(-10**6, 10**6, (m, n)).astype(np.int32)
    for alpha, beta in [(1, 0), (3, -2), (-500, 7)]:
        truth = O.spmm_f64(rp, ci, va.astype(np.float32), b.astype(np.float32), n, c.astype(np.float32), n, n, k,
                           float(alpha), float(beta))  # every term is an integer far below 2^53: exact
        want = np.clip(truth, -2.0**31, 2.0**31 - 1).astype(np.int64).astype(np.int32)
        got = NarrowSpmm(rp, ci, va, k, n, b, n, c, n, "i8", "i32").run(alpha, beta).reshape(m, n)
        assert np.array_equal(got, want), (alpha, beta)
    # saturation both ways, and a beta term that brings the value back into range
    rp2, ci2 = np.array([0, 1, 2, 3], np.int32), np.array([0, 0, 0], np.int32)
    va2, b2 = np.array([127, -127, 127], np.int8), np.array([[127, -127]], np.int8)
    c2 = np.array([[0, 0], [0, 0], [-2**31, 2**31 - 1]], np.int32)
    got = NarrowSpmm(rp2, ci2, va2, 1, 2, b2, 2, c2, 2, "i8", "i32").run(2**31 - 1, 16129).reshape(3, 2)
    exact = [[(2**31 - 1) * int(va2[r]) * int(b2[0, j]) + 16129 * int(c2[r, j]) for j in range(2)] for r in range(3)]
    want = np.clip(np.array(exact, dtype=object), -2**31, 2**31 - 1).astype(np.int64).astype(np.int32)
    assert np.array_equal(got, want), (got, want)


def test_unsupported_combinations_are_rejected():
    rp, ci = dev(np.array([0, 1], np.int32)), dev(np.array([0], np.int32))
    for a_kind, b_kind, c_kind in [("f16", "f32", "f32"), ("f16", "f16", "bf16"), ("f32", "f32", "f16"),
                                   ("i8", "i8", "f32")]:
        va, b, c = to_device([1], a_kind), to_device([[1]], b_kind), to_device([[0]], c_kind)
        h = api.Handle()
        op = api.SpMM(h, api.CsrMatrix(1, 1, rp, ci, va), api.DnMat(1, 1, 1, b), api.DnMat(1, 1, 1, c))
        with pytest.raises(api.AclsparseError) as err:
            op.buffer_size()
        assert err.value.status == L.NOT_SUPPORTED
