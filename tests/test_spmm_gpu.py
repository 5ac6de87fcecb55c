"""SpMM parity on the GPU, through the C ABI, against the oracle and the reference's golden vectors.

Tolerance of every fp32 output against the fp64 truth: |got - truth| <= 1e-6 + 1e-5*|truth| on every
element, for EVERY algorithm value (the library computes all of them with fp64 row sums); the case matrix
follows the reference's kFp32Cases (test/spmm/arch35/spmm_test.cpp:1366-1424).  The forward error bound
below is only applied to the oracle's restatement of the reference's fp32 golden, which accumulates in fp32.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import workloads  # noqa: E402
from tests.gpu_util import SpmmCase, dev, random_csr  # noqa: E402

RTOL, ATOL = 1e-5, 1e-6


HP = L.SPMM_CSR_FP32_HIGH_PRECISION_ALG


def assert_close(got, truth, what=""):
    bad, max_abs, max_rel = O.check_tolerance(got, truth, RTOL, ATOL)
    assert bad == 0, f"{what}: {bad} of {got.size} outside tolerance (max abs {max_abs:.3e}, max rel {max_rel:.3e})"


def assert_fp32_forward_bound(got, truth, rp, ci, va, b, alpha, beta, c0, what=""):
    """Plain fp32 accumulation, in any order, obeys the classical forward bound of a dot product:
    |got - truth| <= (len + 4) * 2^-24 * (|alpha| * |A||B| + |beta| * |C|), element by element.  The
    reference's own fp32 golden is held to this (the library's kernels to the strict tolerance); the
    reference's relative bar (test/spmm/arch35/spmm_test.cpp:330-378) cannot be used on cancelling rows."""
    n = b.shape[1]
    mag = O.spmm_f64(rp, ci, np.abs(va), np.abs(b), n, np.abs(c0), n, n, b.shape[0], abs(alpha), abs(beta))
    lens = np.diff(rp)[:, None]
    bound = (lens + 4) * 2.0 ** -24 * mag + 1e-30
    err = np.abs(got.astype(np.float64) - truth)
    assert (err <= bound).all(), f"{what}: worst err/bound {np.max(err / bound):.3f}"


def test_reference_known_answers(kats):
    for k in kats["spmm"]:
        n = k["n"]
        case = SpmmCase(k["row_ptr"], k["col_ind"], k["values"], k["k"], n, np.array(k["b"], np.float32), n,
                        np.array(k["c"], np.float32), n, base=k["base"])
        got = case.run(k["alpha"], k["beta"]).reshape(k["m"], n)
        np.testing.assert_allclose(got, np.array(k["expect"], np.float32), rtol=0, atol=1e-5, err_msg=k["name"])


def test_reference_goldens(goldens):
    for name, g in goldens.items():
        n = g["n"]
        # every algorithm value meets the strict tolerance on any data, cancelling rows included
        for alg in (L.SPMM_ALG_DEFAULT, HP, L.SPMM_CSR_ALG2):
            case = SpmmCase(g["row_ptr"], g["col_ind"], g["values"], g["cols"], n, g["b"], n, g["c0"], n,
                            base=g["base"], alg=alg)
            got = case.run(g["alpha"], g["beta"]).reshape(g["rows"], n)
            assert_close(got, g["truth"], f"{name} alg={alg}")


def test_two_matrices_sharing_one_workspace():
    """A1, A2, A1 through one external buffer: every product uses its own matrix's plan."""
    rng = np.random.default_rng(32)
    m, k, n = 3000, 2500, 16
    lens1 = rng.integers(0, 30, m)
    lens2 = rng.permutation(lens1)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = np.zeros((m, n), np.float32)
    mats, cases = [], []
    from ops_sparse_b200 import api
    h = api.Handle()
    for lens in (lens1, lens2):
        rp, ci = random_csr(rng, lens, k)
        va = rng.uniform(0, 1, ci.size).astype(np.float32)
        mats.append(O.spmm_f64(rp, ci, va, b, n, c0, n, n, k))
        cases.append(SpmmCase(rp, ci, va, k, n, b, n, c0, n, alg=HP, handle=h))
    shared = cases[0].op.allocate()
    cases[1].op.buffer = shared
    for preprocess in (True, False):
        if preprocess:
            cases[0].op.preprocess()
            cases[1].op.preprocess()
        for which in (0, 1, 0, 0, 1):
            cases[which].d_c.zero_()
            got = cases[which].run(1.0, 0.0, preprocess=False).reshape(m, n)
            assert_close(got, mats[which], f"matrix {which}, preprocess={preprocess}")


def test_extreme_and_non_finite_values():
    """fp32 products that overflow while the fp64 sum is finite, and Inf / NaN in A and in B: every algorithm
    gives the fp64 golden rounded to fp32 (NaN where it is NaN, the same infinity where it is infinite)."""
    rng = np.random.default_rng(22)
    big = np.float32(3.0e38)
    n = 8
    rows_v = [[big, -big, 1.0], [big, 2.0], [np.inf, 1.0, 1.0], [-np.inf, 1.0], [np.inf, -np.inf], [np.nan, 1.0],
              [1.0, 2.0, 3.0], [0.0, 5.0], [1.0, 1.0]]
    rows_b = [[2.0, 2.0, 1.0], [2.0, 1.0], [1.0, 1.0, 1.0], [2.0, 1.0], [1.0, 1.0], [1.0, 1.0],
              [np.inf, 1.0, 1.0], [np.inf, 1.0], [np.nan, 1.0]]
    lv = rng.standard_normal(3000).astype(np.float32)
    lb = rng.standard_normal(3000).astype(np.float32)
    lv[0], lv[1], lb[0], lb[1] = big, -big, 2.0, 2.0  # a row over three tiles that overflows in fp32 only (the pair leads
    # the row: the golden adds in array order, and a 6e38 term met later would swallow what was summed before it)
    rows_v, rows_b = [list(lv)] + rows_v, [list(lb)] + rows_b
    lens = [len(r) for r in rows_v]
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    nnz = int(rp[-1])
    ci = np.arange(nnz, dtype=np.int32)           # every entry has its own row of B
    va = np.concatenate(rows_v).astype(np.float32)
    b = rng.uniform(0.5, 1.5, (nnz, n)).astype(np.float32)
    b[:, 0] = np.concatenate(rows_b)              # column 0 carries the special factors
    b[:, 3] = np.concatenate(rows_b)
    c0 = np.ones((len(lens), n), np.float32)
    for alg in (L.SPMM_ALG_DEFAULT, HP):
        for a, be in ((1.0, 0.0), (0.5, 2.0)):
            got = SpmmCase(rp, ci, va, nnz, n, b, n, c0, n, alg=alg).run(a, be).reshape(len(lens), n)
            truth = O.spmm_f64(rp, ci, va, b, n, c0, n, n, nnz, a, be)
            with np.errstate(over="ignore", invalid="ignore"):
                want = truth.astype(np.float32)
            assert np.array_equal(np.isnan(got), np.isnan(want)), (alg, a, be)
            inf = np.isinf(want)
            assert np.array_equal(got[inf], want[inf]), (alg, a, be)
            fin = np.isfinite(want)
            assert_close(got[fin], truth[fin], f"non-finite alg={alg} {a},{be}")


def layout(a, row_major, pad):
    """Storage array of matrix `a` in the given order with `pad` extra leading-dimension elements."""
    r, c = a.shape
    if row_major:
        out = np.full((r, c + pad), 55.0, np.float32); out[:, :c] = a
        return out.ravel(), c + pad
    out = np.full((c, r + pad), 55.0, np.float32); out[:, :r] = a.T
    return out.ravel(), r + pad


def unlayout(flat, r, c, ld, row_major):
    return flat.reshape(r, ld)[:, :c] if row_major else flat.reshape(c, ld)[:, :r].T


# name, m, k, n, nnz, alpha, beta, opB transposed, B row-major, C row-major, pad B, pad C, base, preprocess
CASES = [
    ("N_Brow_Crow", 37, 23, 11, 170, 1.0, 0.0, False, True, True, 0, 0, 0, True),
    ("N_Brow_Ccol", 37, 23, 11, 170, 1.0, 0.0, False, True, False, 0, 0, 0, True),
    ("N_Bcol_Crow", 37, 23, 11, 170, 1.0, 0.0, False, False, True, 0, 0, 0, True),
    ("N_Bcol_Ccol", 37, 23, 11, 170, 1.0, 0.0, False, False, False, 0, 0, 0, True),
    ("T_Brow_Crow", 37, 23, 11, 170, 1.0, 0.0, True, True, True, 0, 0, 0, True),
    ("T_Brow_Ccol", 37, 23, 11, 170, 1.0, 0.0, True, True, False, 0, 0, 0, True),
    ("T_Bcol_Crow", 37, 23, 11, 170, 1.0, 0.0, True, False, True, 0, 0, 0, True),
    ("T_Bcol_Ccol", 37, 23, 11, 170, 1.0, 0.0, True, False, False, 0, 0, 0, True),
    ("T_padded_ld_beta", 41, 29, 13, 205, -0.75, 0.5, True, False, True, 3, 5, 0, True),
    ("small_non_square", 7, 5, 3, 14, 1.0, 0.0, False, True, True, 0, 0, 0, True),
    ("baseline_256", 256, 256, 64, 2048, 1.0, 0.0, False, True, True, 0, 0, 0, True),
    ("beta_nonzero_256", 256, 256, 64, 2048, 1.0, 0.5, False, True, True, 0, 0, 0, True),
    ("wide_128", 200, 300, 128, 3000, 1.0, 0.5, False, True, True, 0, 0, 0, True),
    ("wide_256_padded", 90, 70, 256, 900, 2.5, 1.5, False, True, True, 4, 8, 0, True),
    ("odd_ld_forces_scalar", 64, 64, 64, 512, 1.0, 0.0, False, True, True, 1, 3, 0, True),
    ("without_preprocess", 19, 13, 7, 61, -1.25, 0.75, False, False, True, 2, 3, 0, False),
    ("one_based_csr", 17, 11, 5, 44, 0.5, -0.25, False, True, False, 0, 0, 1, True),
    ("alpha_zero_beta_one", 9, 7, 3, 18, 0.0, 1.0, False, False, False, 1, 2, 0, True),
    ("empty_csr_beta", 5, 6, 4, 0, 0.0, 0.5, False, False, True, 0, 0, 0, True),
    ("unit_shape", 1, 1, 1, 1, 1.0, 0.5, False, True, True, 0, 0, 0, True),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_layout_and_scalar_matrix(case):
    name, m, k, n, nnz, alpha, beta, op_t, b_row, c_row, pad_b, pad_c, base, pre = case
    rng = np.random.default_rng(sum(ord(ch) * (i + 1) for i, ch in enumerate(name)))  # stable across runs
    per = np.full(m, nnz // m) + (np.arange(m) < nnz % m)
    rp, ci = random_csr(rng, per, k)
    va = rng.uniform(-5, 5, ci.size).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    b_store, ldb = layout(b.T if op_t else b, b_row, pad_b)
    c_store, ldc = layout(c0, c_row, pad_c)
    sc = SpmmCase(rp + base, ci + base, va, k, n, b_store, ldb, c_store, ldc, base=base,
                  order_b=L.ORDER_ROW if b_row else L.ORDER_COL, order_c=L.ORDER_ROW if c_row else L.ORDER_COL,
                  op_b=L.OP_T if op_t else L.OP_N, alg=HP)
    got_store = sc.run(alpha, beta, preprocess=pre)
    truth = O.spmm_f64(rp, ci, va, b, n, c0, n, n, k, alpha, beta)
    assert_close(unlayout(got_store, m, n, ldc, c_row), truth, name)
    # padding of C is untouched
    mask = np.ones_like(c_store, bool)
    idx = np.arange(c_store.size).reshape(-1, ldc)
    mask[idx[:, :(n if c_row else m)].ravel()] = False
    assert (got_store[mask] == 55.0).all()
    # the oracle's fp32 golden of the same stored layout agrees too
    gold = O.spmm_f32(rp, ci, va, b_store, ldb, c_store, ldc, n, alpha, beta, b_row_major=b_row,
                      op_b_transpose=op_t, c_row_major=c_row)
    assert_fp32_forward_bound(unlayout(gold, m, n, ldc, c_row), truth, rp, ci, va, b, alpha, beta, c0,
                              name + " (fp32 golden)")
    # the default algorithm value on the same storage: the same strict tolerance
    sd = SpmmCase(rp + base, ci + base, va, k, n, b_store, ldb, c_store, ldc, base=base,
                  order_b=L.ORDER_ROW if b_row else L.ORDER_COL, order_c=L.ORDER_ROW if c_row else L.ORDER_COL,
                  op_b=L.OP_T if op_t else L.OP_N)
    assert_close(unlayout(sd.run(alpha, beta, preprocess=pre), m, n, ldc, c_row), truth, name + " (default alg)")


def test_device_scalars_and_plan_reuse():
    rng = np.random.default_rng(21)
    m, k, n = 300, 200, 64
    rp, ci = random_csr(rng, rng.integers(0, 30, m), k)
    va = rng.uniform(-1, 1, ci.size).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    sc = SpmmCase(rp, ci, va, k, n, b, n, c0, n, alg=HP)
    sc.handle.set_pointer_mode(L.POINTER_MODE_DEVICE)
    alpha, beta = dev(np.array([0.75], np.float32)), dev(np.array([-0.25], np.float32))
    got = sc.run(alpha, beta, preprocess=False).reshape(m, n)
    assert_close(got, O.spmm_f64(rp, ci, va, b, n, c0, n, n, k, 0.75, -0.25), "device scalars")
    # new B and C on the same plan
    b2 = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c2 = np.full((m, n), np.nan, np.float32)  # beta == 0 never reads C
    d_b2, d_c2 = dev(b2), dev(c2)
    sc.mb.set_values(d_b2)
    sc.mc.set_values(d_c2)
    sc.handle.set_pointer_mode(L.POINTER_MODE_HOST)
    sc.op(1.0, 0.0)
    torch.cuda.synchronize()
    assert_close(d_c2.cpu().numpy(), O.spmm_f64(rp, ci, va, b2, n, np.zeros((m, n), np.float32), n, n, k), "rebind")


@pytest.mark.parametrize("name,rows", [("c4", 1 << 15), ("c5", 1 << 17)])
def test_benchmark_configs_vs_oracle(name, rows):
    cfg = workloads.make(name, rows=rows)
    n, m = cfg["n"], cfg["rows"]
    sc = SpmmCase(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["cols"], n, cfg["b"], n, cfg["c"], n)
    got = sc.run(cfg["alpha"], cfg["beta"]).reshape(m, n)
    truth = O.spmm_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["b"], n, cfg["c"], n, n, cfg["cols"],
                       cfg["alpha"], cfg["beta"], threads=O.max_threads())
    assert_close(got, truth, name)
    for _ in range(2):  # bit-reproducible
        again = sc.run(cfg["alpha"], cfg["beta"], preprocess=False).reshape(m, n)
        assert np.array_equal(again.view(np.uint32), got.view(np.uint32))


def test_plan_metadata_bit_exact():
    rng = np.random.default_rng(31)
    for lengths in (np.clip(rng.zipf(2.0, 15000) * 3, 1, 9000), rng.poisson(16, 20000), np.zeros(3000, int),
                    np.array([40000])):
        cols, n = int(max(lengths.max(), 1)) + 5, 32
        rp, ci = random_csr(rng, lengths, cols)
        rows, nnz = len(lengths), ci.size
        sc = SpmmCase(rp, ci, np.ones(nnz, np.float32), cols, n, np.ones((cols, n), np.float32), n,
                      np.zeros((rows, n), np.float32), n)
        sc.op.preprocess()
        torch.cuda.synchronize()
        ws = sc.op.buffer.cpu().numpy()
        lay = O.spmm_plan_layout(rows, nnz, n)
        assert ws.size == lay["total_bytes"]
        head = O.plan_header(2, rows, cols, nnz, 0, n, lay, O.SPMM_TILE_ITEMS)
        assert np.array_equal(ws[:head.size], head)
        tile_row, tile_class = O.plan_tiles(rp, nnz, O.SPMM_TILE_ITEMS, 1)
        nt = lay["num_tiles"]
        assert np.array_equal(ws[lay["row_ptr_off"]:lay["row_ptr_off"] + 4 * (rows + 1)].view(np.int32), rp)
        assert np.array_equal(ws[lay["tile_row_off"]:lay["tile_row_off"] + 4 * (nt + 1)].view(np.int32), tile_row)
        assert np.array_equal(ws[lay["tile_class_off"]:lay["tile_class_off"] + 4 * nt].view(np.int32), tile_class)


@pytest.mark.parametrize("n", [1, 4, 31, 32, 33, 64, 96, 128, 160, 256])
def test_long_and_empty_rows_all_widths(n):
    """Rows that span many warps and tiles, runs of empty rows, every vector width."""
    rng = np.random.default_rng(40 + n)
    k = 5000
    lengths = np.concatenate([rng.integers(0, 6, 300), [4000], np.zeros(1500, int), [1024, 1023, 1025, 127, 128, 129],
                              rng.integers(0, 40, 200), [3000, 3000]])
    rp, ci = random_csr(rng, lengths, k)
    m = lengths.size
    va = rng.uniform(-1, 1, ci.size).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    truth = O.spmm_f64(rp, ci, va, b, n, c0, n, n, k, 1.5, -0.5)
    got = SpmmCase(rp, ci, va, k, n, b, n, c0, n, alg=HP).run(1.5, -0.5).reshape(m, n)
    assert_close(got, truth, f"n={n} high-precision alg")
    got = SpmmCase(rp, ci, va, k, n, b, n, c0, n).run(1.5, -0.5).reshape(m, n)
    assert_close(got, truth, f"n={n} default alg")


def test_shared_workspace_between_spmv_and_spmm(kats):
    """SpMV and SpMM handed the same allocation invalidate each other's plan (reference: spmv_test.cpp:386-472)."""
    from ops_sparse_b200 import api
    k = kats["spmv"][4]
    rp, ci, va = (np.array(k[s]) for s in ("row_ptr", "col_ind", "values"))
    d_rp, d_ci, d_va = dev(rp, np.int32), dev(ci, np.int32), dev(va, np.float32)
    d_x, d_y = dev(np.array([1, 2, 3], np.float32)), dev(np.zeros(2, np.float32))
    h = api.Handle()
    mat = api.CsrMatrix(2, 3, d_rp, d_ci, d_va)
    mv = api.SpMV(h, mat, api.DnVec(d_x), api.DnVec(d_y))
    mm = api.SpMM(h, mat, api.DnMat(3, 1, 1, d_x), api.DnMat(2, 1, 1, d_y))
    ws = torch.empty(max(mv.buffer_size(), mm.buffer_size()), dtype=torch.uint8, device="cuda:0")
    mv.buffer = ws
    mm.buffer = ws
    for mm_pre in (False, True):
        mv.preprocess()
        d_y.zero_()
        if mm_pre:
            mm.preprocess()
        mm()
        torch.cuda.synchronize()
        np.testing.assert_allclose(d_y.cpu().numpy(), [11, 8], atol=1e-5)
        d_y.zero_()
        mv()  # must not trust SpMM metadata in the buffer
        torch.cuda.synchronize()
        np.testing.assert_allclose(d_y.cpu().numpy(), [11, 8], atol=1e-5)


# ------------------------------------------------------------------ op(A) = transpose --

def _transpose_host(rp, ci, va, cols):
    """A^T as CSR on the host (stable counting sort by column), for the oracle."""
    rpt, cit, perm = O.transpose_twin(rp, ci, cols)
    return rpt, cit, np.asarray(va, np.float32)[perm]


@pytest.mark.parametrize("op_a", [L.OP_T, L.OP_H])
@pytest.mark.parametrize("n", [1, 7, 64, 128])
def test_transposed_a_vs_oracle(op_a, n):
    """C = alpha * A^T * B + beta * C (reference cases: test/spmm/arch35/spmm_transpose_test.cpp): A is m x k,
    B has m rows and C has k."""
    rng = np.random.default_rng(50 + n)
    m, k = 700, 500
    lengths = np.concatenate([rng.integers(0, 25, m - 2), [400, 0]])
    rp, ci = random_csr(rng, lengths, k)
    va = rng.uniform(-1, 1, ci.size).astype(np.float32)
    b = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    from ops_sparse_b200 import api
    d_rp, d_ci, d_va, d_b, d_c = dev(rp, np.int32), dev(ci, np.int32), dev(va), dev(b), dev(c0)
    h = api.Handle()
    mat = api.CsrMatrix(m, k, d_rp, d_ci, d_va, nnz=ci.size)
    op = api.SpMM(h, mat, api.DnMat(m, n, n, d_b), api.DnMat(k, n, n, d_c), op_a=op_a)
    rpt, cit, vat = _transpose_host(rp, ci, va, k)
    truth = O.spmm_f64(rpt, cit, vat, b, n, c0, n, n, m, 0.75, -0.5)
    for pre in (True, False):
        d_c.copy_(torch.from_numpy(c0))
        if pre:
            op.preprocess(0.75, -0.5)
        op(0.75, -0.5)
        torch.cuda.synchronize()
        assert_close(d_c.cpu().numpy(), truth, f"A^T n={n} preprocess={pre}")
    # new values through the same plan
    va2 = (va * 0.5 + 0.25).astype(np.float32)
    d_va.copy_(torch.from_numpy(va2))
    d_c.copy_(torch.from_numpy(c0))
    op(0.75, -0.5)
    torch.cuda.synchronize()
    assert_close(d_c.cpu().numpy(), O.spmm_f64(rpt, cit, va2[O.transpose_twin(rp, ci, k)[2]], b, n, c0, n, n, m,
                                               0.75, -0.5), f"A^T n={n}, new values")
