"""SpMV with fp16 / bf16 / int8 storage on the GPU, through the C ABI, against the oracle.

The supported combinations are the reference's table (sparse/spmv/arch35/spmv_host.cpp:44-66) without its
complex rows.  Floating results must be the fp64 truth rounded ONCE to the output type (to nearest even) up to
the summation order; integer results must be exact.  Known answers: test/spmv/arch35/spmv_test.cpp:617-697.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import api  # noqa: E402
from tests.gpu_util import bits_of, dev, expected_bits, quantize, random_csr, to_device  # noqa: E402


class NarrowCase:
    def __init__(self, rp, ci, values, x, y, in_kind, out_kind, cols=None, base=0, op=L.OP_N, strides=None):
        self.rows, self.cols = len(rp) - 1, (len(x) if cols is None else cols)
        self.d_rp, self.d_ci = dev(np.asarray(rp), np.int32), dev(np.asarray(ci), np.int32)
        self.d_va, self.d_x, self.d_y = to_device(values, in_kind), to_device(x, in_kind), to_device(y, out_kind)
        self.handle = api.Handle()
        self.mat = api.CsrMatrix(self.rows, self.cols, self.d_rp, self.d_ci, self.d_va, base, nnz=len(ci))
        self.vx, self.vy = api.DnVec(self.d_x), api.DnVec(self.d_y)
        self.op = api.SpMV(self.handle, self.mat, self.vx, self.vy, op=op)

    def run(self, alpha, beta, preprocess=True):
        if preprocess:
            self.op.preprocess(alpha, beta)
        self.op(alpha, beta)
        torch.cuda.synchronize()
        return bits_of(self.d_y)


def test_halfway_results_round_to_even():
    """test/spmv/arch35/spmv_test.cpp:665-697: 1 + 2^-11 and its negative in fp16 round to +-1."""
    vals = np.array([0x3C00, 0x1000, 0xBC00, 0x9000], np.uint16).view(np.float16)
    case = NarrowCase([0, 2, 4], [0, 1, 0, 1], vals, np.array([1, 1], np.float16), [0, 0], "f16", "f16")
    assert case.run(1.0, 0.0).tolist() == [0x3C00, 0xBC00]


@pytest.mark.parametrize("kind, tie, up", [("f16", 1 + 2.0**-11, 0x3C01), ("bf16", 1 + 2.0**-8, 0x3F81)])
def test_result_is_rounded_once(kind, tie, up):
    """alpha*sum + beta*y a hair above a tie of the output type: rounding the double to fp32 first would land on
    the tie and then on the even neighbour below; one rounding goes up."""
    case = NarrowCase([0, 1, 2], [0, 0], [1.0, 1.0], [1.0], [2.0**-24, 0.0], kind, kind)
    got = case.run(float(tie), 2.0**-6)
    assert got.tolist() == [up, up - 1]  # the second row is exactly the tie: down to the even neighbour


@pytest.mark.parametrize("op", [L.OP_N, L.OP_T, L.OP_H])
@pytest.mark.parametrize("rows", [2, 4096])
def test_int32_saturation(op, rows):
    """test/spmv/arch35/spmv_test.cpp:617-663: alpha = INT32_MAX times +-127*127 saturates both ways."""
    rp = np.full(rows + 1, 2, np.int32)
    rp[0], rp[1] = 0, 1
    transposed = op != L.OP_N
    x = np.full(rows if transposed else 2, 127, np.int8)
    y = np.zeros(2 if transposed else rows, np.int32)
    case = NarrowCase(rp, [0, 1], np.array([127, -127], np.int8), x, y, "i8", "i32", cols=2, op=op)
    got = case.run(2**31 - 1, 0)
    assert got[0] == 2**31 - 1 and got[1] == -2**31 and not got[2:].any()


def test_int32_exact_against_oracle():
    rng = np.random.default_rng(5)
    rows, cols = 3000, 2500
    lengths = rng.integers(0, 90, rows)
    lengths[7] = 2400
    rp, ci = random_csr(rng, lengths, cols)
    va = rng.integers(-127, 128, ci.size).astype(np.int8)
    x = rng.integers(-127, 128, cols).astype(np.int8)
    y = rng.integers(-2**31, 2**31 - 1, rows).astype(np.int32)
    for alpha, beta in [(1, 0), (3, -2), (-70000, 1), (2**31 - 1, 2**31 - 1), (0, 5), (-(2**31), -(2**31))]:
        case = NarrowCase(rp, ci, va, x, y, "i8", "i32")
        got = case.run(alpha, beta)
        want = O.spmv_i8_i32(rp, ci, va, x, y, alpha, beta)
        assert np.array_equal(got, want), (alpha, beta, np.nonzero(got != want)[0][:5])


@pytest.mark.parametrize("in_kind, out_kind", [("f16", "f16"), ("f16", "f32"), ("bf16", "bf16"), ("bf16", "f32"),
                                               ("i8", "f32")])
@pytest.mark.parametrize("shape", ["short", "ragged"])
def test_random_matrices_against_truth(in_kind, out_kind, shape):
    rng = np.random.default_rng(11)
    rows, cols = (5000, 4000) if shape == "short" else (1500, 9000)
    lengths = rng.poisson(12, rows) if shape == "short" else (rng.zipf(1.7, rows) % 400)
    if shape == "ragged":
        lengths[3], lengths[900] = 8000, 0
    rp, ci = random_csr(rng, lengths, cols)
    scale = 20.0 if in_kind == "i8" else 1.0
    va = quantize(rng.standard_normal(ci.size) * scale, in_kind)
    x = quantize(rng.standard_normal(cols) * scale, in_kind)
    y = quantize(rng.uniform(-1, 1, rows), out_kind)
    for alpha, beta in [(1.0, 0.0), (1.5, 0.5)]:
        truth = O.spmv_f64(rp, ci, va, x, y, alpha, beta)
        case = NarrowCase(rp, ci, va, x, y, in_kind, out_kind)
        got = case.run(alpha, beta)
        if out_kind == "f32":
            bad, max_abs, max_rel = O.check_tolerance(got, truth, 1e-6, 1e-7)
            assert bad == 0, (max_abs, max_rel)
        else:
            want = expected_bits(truth, out_kind)
            # The summation order differs from the oracle's, so a truth within 1e-15 of a tie may round the other
            # way: never more than one unit in the last place, and (measured) almost never at all.
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert diff.max() <= 1 and (diff != 0).mean() < 1e-3, (diff.max(), (diff != 0).mean())
        again = NarrowCase(rp, ci, va, x, y, in_kind, out_kind).run(alpha, beta)
        assert np.array_equal(got, again)  # bit-reproducible


@pytest.mark.parametrize("in_kind, out_kind", [("f16", "f32"), ("bf16", "bf16")])
def test_transposed_and_index_base_one(in_kind, out_kind):
    rng = np.random.default_rng(3)
    rows, cols = 700, 1100
    rp, ci = random_csr(rng, rng.poisson(9, rows), cols)
    va = quantize(rng.standard_normal(ci.size), in_kind)
    x = quantize(rng.standard_normal(rows), in_kind)
    y = quantize(rng.uniform(-1, 1, cols), out_kind)
    truth = O.spmv_transpose_f64(rp, ci, va, x, y, cols, 0.75, -0.5)
    case = NarrowCase(rp + 1, ci + 1, va, x, y, in_kind, out_kind, cols=cols, base=1, op=L.OP_T)
    got = case.run(0.75, -0.5)
    if out_kind == "f32":
        assert O.check_tolerance(got, truth, 1e-6, 1e-7)[0] == 0
    else:
        diff = np.abs(got.astype(np.int32) - expected_bits(truth, out_kind).astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 1e-2


def test_bf16_products_that_overflow_fp32():
    """3e38 * 3e38 is not an fp32 number; the row is summed again in fp64 and cancels as in the truth."""
    big = quantize([3.0e38], "bf16")[0]
    va = np.array([big, -big, 2.0, 1.0], np.float32)
    case = NarrowCase([0, 3, 4], [0, 1, 2, 0], va, quantize([big, big, 1.5], "bf16"), [0, 0], "bf16", "f32")
    got = case.run(1.0, 0.0)
    assert got[0] == 3.0 and got[1] == big


def test_unsupported_combinations_are_rejected():
    rp, ci = np.array([0, 1], np.int32), np.array([0], np.int32)
    for in_kind, x_kind, out_kind in [("f16", "f32", "f32"), ("f16", "f16", "bf16"), ("f32", "f32", "f16"),
                                      ("i8", "i8", "f16")]:
        d_rp, d_ci = dev(rp), dev(ci)
        va, x, y = to_device([1], in_kind), to_device([1], x_kind), to_device([0], out_kind)
        h = api.Handle()
        mat = api.CsrMatrix(1, 1, d_rp, d_ci, va)
        op = api.SpMV(h, mat, api.DnVec(x), api.DnVec(y))
        with pytest.raises(api.AclsparseError) as err:
            op.buffer_size()
        assert err.value.status == L.NOT_SUPPORTED
