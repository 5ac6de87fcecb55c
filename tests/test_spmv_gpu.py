"""SpMV parity on the GPU, through the C ABI, against the oracle and the reference's golden vectors.

Tolerance of every fp32 output against the fp64-accumulated truth: |got - truth| <= 1e-6 + 1e-5*|truth|
on every element.  Preprocessing metadata is compared bit for bit with the oracle's CPU twin.
"""
import ctypes
from ctypes import c_void_p

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from ops_sparse_b200 import _lib as L  # noqa: E402
from ops_sparse_b200 import api, workloads  # noqa: E402
from tests.gpu_util import DEV, SpmvCase, dev, random_csr  # noqa: E402

RTOL, ATOL = 1e-5, 1e-6


def assert_close(got, truth, what=""):
    bad, max_abs, max_rel = O.check_tolerance(got, truth, RTOL, ATOL)
    assert bad == 0, f"{what}: {bad} of {got.size} outside tolerance (max abs {max_abs:.3e}, max rel {max_rel:.3e})"


def test_reference_known_answers(kats):
    for k in kats["spmv"]:
        for alg in (L.SPMV_ALG_DEFAULT, L.SPMV_CSR_ALG1, L.SPMV_CSR_ALG2):
            case = SpmvCase(k["row_ptr"], k["col_ind"], k["values"], k["x"], k["y"], cols=k["cols"], base=k["base"],
                            alg=alg)
            got = case.run(k["alpha"], k["beta"])
            np.testing.assert_allclose(got, np.array(k["expect"], np.float32), rtol=0, atol=1e-5, err_msg=k["name"])
            if "expect_second" in k:  # the same pattern and workspace must stay valid for a second call
                got = case.run(k["alpha"], k["beta"], preprocess=False)
                np.testing.assert_allclose(got, np.array(k["expect_second"], np.float32), rtol=0, atol=1e-5)


def test_device_pointer_mode(kats):
    k = kats["spmv"][0]
    case = SpmvCase(k["row_ptr"], k["col_ind"], k["values"], k["x"], k["y"], cols=k["cols"])
    case.handle.set_pointer_mode(L.POINTER_MODE_DEVICE)
    alpha, beta = dev(np.array([k["alpha"]], np.float32)), dev(np.array([k["beta"]], np.float32))
    got = case.run(alpha, beta)
    np.testing.assert_allclose(got, np.array(k["expect"], np.float32), rtol=0, atol=1e-5)


def test_without_preprocess_and_rebinding(kats):
    """Preprocess is optional; a plan made before values were bound is not trusted afterwards."""
    k = kats["spmv"][4]
    case = SpmvCase(k["row_ptr"], k["col_ind"], k["values"], k["x"], k["y"], cols=k["cols"])
    np.testing.assert_allclose(case.run(preprocess=False), [11, 8], atol=1e-5)
    # rebind the values: the next call must use the new array
    new_vals = dev(np.array([1, 1, 1], np.float32))
    api.check("SetValues", L.lib().aclsparseSpMatSetValues(case.mat.raw, c_void_p(new_vals.data_ptr())))
    np.testing.assert_allclose(case.run(preprocess=False), [4, 2], atol=1e-5)


def test_two_matrices_sharing_one_workspace():
    """A1, A2, A1 through one external buffer: every product uses its own matrix's plan, with and without
    explicit Preprocess calls (two matrices of equal rows and nnz, so that their plans have the same layout)."""
    rng = np.random.default_rng(31)
    rows, cols = 6000, 5000
    lens1 = rng.integers(0, 40, rows)
    lens2 = rng.permutation(lens1)                 # same rows and nnz, different structure
    x = rng.standard_normal(cols).astype(np.float32)
    y0 = np.zeros(rows, np.float32)
    mats = []
    for lens in (lens1, lens2):
        rp, ci = random_csr(rng, lens, cols)
        va = rng.standard_normal(ci.size).astype(np.float32)
        mats.append((rp, ci, va, O.spmv_f64(rp, ci, va, x, y0)))
    h = api.Handle()
    cases = [SpmvCase(rp, ci, va, x, y0, handle=h) for rp, ci, va, _ in mats]
    shared = cases[0].op.allocate()
    cases[1].op.buffer = shared
    for preprocess in (True, False):
        if preprocess:
            cases[0].op.preprocess()
            cases[1].op.preprocess()               # overwrites the plan of the first matrix
        for which in (0, 1, 0, 0, 1):
            cases[which].d_y.zero_()
            got = cases[which].run(1.0, 0.0, preprocess=False)
            assert_close(got, mats[which][3], f"matrix {which}, preprocess={preprocess}")


def test_beta_zero_never_reads_y():
    rng = np.random.default_rng(1)
    rp, ci = random_csr(rng, rng.integers(0, 40, 3000), 2500)
    va = rng.uniform(-1, 1, ci.size).astype(np.float32)
    x = rng.uniform(-1, 1, 2500).astype(np.float32)
    y = np.full(3000, np.nan, np.float32)
    got = SpmvCase(rp, ci, va, x, y).run(1.0, 0.0)
    assert_close(got, O.spmv_f64(rp, ci, va, x, np.zeros(3000, np.float32)), "beta=0 with NaN y")


def test_reference_goldens(goldens):
    for name, g in goldens.items():
        if g["n"] != 1:
            continue
        case = SpmvCase(g["row_ptr"], g["col_ind"], g["values"], g["b"][:, 0], g["c0"][:, 0], cols=g["cols"],
                        base=g["base"])
        assert_close(case.run(g["alpha"], g["beta"]), g["truth"][:, 0], name)


@pytest.mark.parametrize("name,rows", [("c1", None), ("c2", 40 ** 3), ("c3", 1 << 17)])
def test_benchmark_configs_vs_oracle(name, rows):
    cfg = workloads.make(name, rows=rows)
    truth = O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], cfg["alpha"], cfg["beta"],
                       threads=O.max_threads())
    case = SpmvCase(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"])
    got = case.run(cfg["alpha"], cfg["beta"])
    assert_close(got, truth, name)
    # the reference's fp32 golden is held to the same check and reported, not required
    # determinism: three more runs give the same bits
    for _ in range(3):
        case.d_y.copy_(torch.from_numpy(cfg["y"]))
        again = case.run(cfg["alpha"], cfg["beta"], preprocess=False)
        assert np.array_equal(again.view(np.uint32), got.view(np.uint32))


def test_both_kernels_agree_and_no_wait_runs_out():
    """Matrices with short rows are computed by the row-block kernel, or by the merge-path tile kernel when
    it is switched off (ACLSPARSE_SPMV_ROW_BLOCKS=0): both meet the tolerance against the oracle.  The
    row-block kernel counts bounded waits that ran out in the plan header; the count stays 0."""
    import subprocess, sys, os
    shapes = (("c1", None), ("c2", 50 ** 3), ("c3", 1 << 16))
    code = (
        "import sys, numpy as np, torch; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "from gpu_util import SpmvCase\n"
        "from ops_sparse_b200 import workloads\n"
        "out = []\n"
        "for name, rows in " + repr(shapes) + ":\n"
        "    cfg = workloads.make(name, rows=rows)\n"
        "    case = SpmvCase(cfg['row_ptr'], cfg['col_ind'], cfg['values'], cfg['x'], cfg['y'])\n"
        "    got = case.run(cfg['alpha'], cfg['beta'])\n"
        "    fails = int(case.op.buffer[128:132].view(torch.int32).item())\n"
        "    assert fails == 0, fails\n"
        "    import ctypes; from ops_sparse_b200 import _lib as L\n"
        "    count = ctypes.c_uint32(9)\n"
        "    st = L.lib().aclsparseB200SpMVWaitFailures(0x1, case.op.buffer.data_ptr(), ctypes.byref(count))\n"
        "    assert st == L.SUCCESS and count.value == 0, (st, count.value)\n"
        "    out.append(got)\n"
        "np.save(sys.argv[1], np.concatenate(out))\n"
    ) % (os.path.dirname(os.path.abspath(__file__)), os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import tempfile
    truth = []
    for name, rows in shapes:
        cfg = workloads.make(name, rows=rows)
        truth.append(O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], cfg["alpha"],
                                cfg["beta"], threads=O.max_threads()))
    truth = np.concatenate(truth)
    for mode in ("1", "0"):  # the choice is read once per process
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "y.npy")
            env = dict(os.environ, ACLSPARSE_SPMV_ROW_BLOCKS=mode)
            subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=600)
            assert_close(np.load(path), truth, f"ACLSPARSE_SPMV_ROW_BLOCKS={mode}")


def test_plan_metadata_bit_exact():
    """Header, normalised row offsets, tile splits and row bins == the oracle's CPU twin."""
    rng = np.random.default_rng(4)
    shapes = [np.clip(rng.zipf(2.0, 20000) * 3, 1, 9000), rng.poisson(16, 30000), np.zeros(5000, int),
              np.array([70000]), np.where(rng.random(8000) < 0.5, 0, rng.integers(1, 300, 8000))]
    for base in (0, 1):
        for lengths in shapes:
            cols = int(max(lengths.max(), 1)) + 17
            rp, ci = random_csr(rng, lengths, cols)
            nnz = ci.size
            va = np.ones(nnz, np.float32)
            case = SpmvCase(rp + base, ci + base, va, np.ones(cols, np.float32), np.zeros(len(lengths), np.float32),
                            base=base)
            case.op.preprocess()
            torch.cuda.synchronize()
            ws = case.op.buffer.cpu().numpy()
            lay = O.spmv_plan_layout(len(lengths), nnz)
            assert ws.size == lay["total_bytes"]
            head = O.plan_header(1, len(lengths), cols, nnz, base, 1, lay, O.SPMV_TILE_ITEMS)
            assert np.array_equal(ws[:head.size], head)
            rows = len(lengths)
            got_rp = ws[lay["row_ptr_off"]:lay["row_ptr_off"] + 4 * (rows + 1)].view(np.int32)
            assert np.array_equal(got_rp, O.normalize_row_offsets(rp + base, rows, base))
            # the counters behind the header: no bounded wait ran out; the longest row
            assert ws[128:132].view(np.uint32)[0] == 0
            assert ws[132:136].view(np.uint32)[0] == O.longest_row(rp + base)
            tile_row, tile_class = O.plan_tiles(rp, nnz, O.SPMV_TILE_ITEMS, O.SPMV_CLASS_DIV)
            nt = lay["num_tiles"]
            assert np.array_equal(ws[lay["tile_row_off"]:lay["tile_row_off"] + 4 * (nt + 1)].view(np.int32), tile_row)
            assert np.array_equal(ws[lay["tile_class_off"]:lay["tile_class_off"] + 4 * nt].view(np.int32), tile_class)


@pytest.mark.parametrize("rows", [1, 2, 31, 32, 33, 255, 256, 257, 2047, 2048, 2049, 4097])
@pytest.mark.parametrize("length", [0, 1, 3, 4, 5, 15, 16, 17, 63, 64, 65, 300])
def test_sizes_around_the_bin_thresholds(rows, length):
    rng = np.random.default_rng(rows * 1000 + length)
    cols = 400
    rp, ci = random_csr(rng, np.full(rows, length), cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    y = rng.uniform(-1, 1, rows).astype(np.float32)
    got = SpmvCase(rp, ci, va, x, y).run(1.5, 0.5)
    assert_close(got, O.spmv_f64(rp, ci, va, x, y, 1.5, 0.5), f"rows={rows} len={length}")


def test_long_rows_and_mixed_tiles():
    """Rows that span many tiles next to short and empty rows (the reference's long-tail cases)."""
    rng = np.random.default_rng(8)
    cols = 60000
    lengths = np.concatenate([rng.integers(0, 8, 500), [50000], rng.integers(0, 8, 300), [2048, 2047, 2049, 511, 512],
                              np.zeros(3000, int), [30000, 30000], rng.integers(0, 30, 700)])
    rp, ci = random_csr(rng, lengths, cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    y = rng.uniform(-1, 1, lengths.size).astype(np.float32)
    got = SpmvCase(rp, ci, va, x, y).run(-0.75, 1.25)
    assert_close(got, O.spmv_f64(rp, ci, va, x, y, -0.75, 1.25), "long rows")


def assert_matches_f64_golden(got, truth, what=""):
    """fp32 result against the fp64 golden rounded to fp32: NaN where it is NaN, the same infinity where it is
    infinite, within the tolerance everywhere else."""
    with np.errstate(over="ignore", invalid="ignore"):
        want = truth.astype(np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want)), f"{what}: NaN pattern {got} vs {want}"
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf]), f"{what}: infinities {got[inf]} vs {want[inf]}"
    fin = np.isfinite(want)
    assert_close(got[fin], truth[fin], what)


def test_extreme_and_non_finite_values():
    """The reference's extreme-value regression (test/spmv/arch22/spmv_test.cpp:1923-1936: 2^116 and 1e35 entries,
    alpha = 2^-116), fp32 products that overflow while the fp64 sum is finite, and Inf / NaN in A and in x, in short
    rows (row-block kernel) and in rows that span tiles (merge-path kernel): all equal to the fp64 golden."""
    rng = np.random.default_rng(21)
    rp = np.array([0, 1, 3, 3, 5], np.int32)
    ci = np.array([0, 1, 7, 2, 5], np.int32)
    va = np.array([2.0 ** 116, 1.0e35, 2.0, 1.0e35, -3.0], np.float32)
    x = rng.uniform(-5, 5, 8).astype(np.float32)
    y = np.zeros(4, np.float32)
    alpha = float(2.0 ** -116)
    got = SpmvCase(rp, ci, va, x, y).run(alpha, 0.0)
    assert_matches_f64_golden(got, O.spmv_f64(rp, ci, va, x, y, alpha, 0.0), "extreme-large-val")

    big = np.float32(3.0e38)
    for long_len in (0, 6000):  # 0: short rows only; 6000: one row over three tiles in front of them
        rows_v = [[big, -big, 1.0], [big, 2.0], [np.inf, 1.0, 1.0], [-np.inf, 1.0], [np.inf, -np.inf], [np.nan, 1.0],
                  [1.0, 2.0, 3.0], [0.0, 5.0], [1.0, 1.0]]
        rows_x = [[2.0, 2.0, 1.0], [2.0, 1.0], [1.0, 1.0, 1.0], [2.0, 1.0], [1.0, 1.0], [1.0, 1.0],
                  [np.inf, 1.0, 1.0], [np.inf, 1.0], [np.nan, 1.0]]
        if long_len:
            # The overflowing pair leads the row: the golden adds in array order, and a 6e38 term met later
            # would swallow whatever it had summed before, which is an artefact of that order, not the product.
            lv = rng.standard_normal(long_len).astype(np.float32)
            lx = rng.standard_normal(long_len).astype(np.float32)
            lv[0], lv[1], lx[0], lx[1] = big, -big, 2.0, 2.0   # cancels in fp64, overflows in fp32
            li = lv.copy()
            li[4000] = np.inf                                   # a row over three tiles that is +Inf
            rows_v, rows_x = [list(lv)] + rows_v + [list(li)], [list(lx)] + rows_x + [list(np.abs(lx) + 1)]
        # every entry gets its own column, so that x can hold the factor meant for it
        lens = [len(r) for r in rows_v]
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        nnz = int(rp[-1])
        ci = np.arange(nnz, dtype=np.int32)
        va = np.concatenate(rows_v).astype(np.float32)
        x = np.concatenate(rows_x).astype(np.float32)
        y = np.ones(len(lens), np.float32)
        for a, b in ((1.0, 0.0), (0.5, 2.0)):
            got = SpmvCase(rp, ci, va, x, y).run(a, b)
            assert_matches_f64_golden(got, O.spmv_f64(rp, ci, va, x, y, a, b), f"non-finite long={long_len} {a},{b}")


def test_strided_storage_preserves_padding():
    """Strided CSR / x / y with sentinels between elements (reference: spmv_test.cpp:283-378, N cases)."""
    sentinel = -1234.0
    for rows in (2, 65):
        row_ptr, col, val = [1], [], []
        for r in range(rows):
            if r % 2 == 0:
                col += [1, 3]; val += [2.0, 3.0]
            else:
                col += [2]; val += [4.0]
            row_ptr.append(len(val) + 1)

        def strided(a, stride, fill, dt):
            out = np.full(len(a) * stride, fill, dt)
            out[::stride] = a
            return out
        rp = dev(strided(row_ptr, 2, -999, np.int32)); ci = dev(strided(col, 3, -999, np.int32))
        va = dev(strided(val, 4, sentinel, np.float32)); x = dev(strided([1, 2, 3], 5, sentinel, np.float32))
        y0 = strided([5.0] * rows, 6, sentinel, np.float32)
        y = dev(y0)
        h = api.Handle()
        mat = api.CsrMatrix(rows, 3, rp, ci, va, L.BASE_ONE, nnz=len(val))
        vx, vy = api.DnVec(x, 3), api.DnVec(y, rows)
        lib = L.lib()
        api.check("strides", lib.aclsparseCsrSetStrides(mat.raw, 2, 3, 4))
        api.check("xstride", lib.aclsparseDnVecSetStride(vx.raw, 5))
        api.check("ystride", lib.aclsparseDnVecSetStride(vy.raw, 6))
        op = api.SpMV(h, mat, vx, vy)
        for pre in (False, True):
            y.copy_(torch.from_numpy(y0))
            if pre:
                op.preprocess(2.0, 3.0)
            op(2.0, 3.0)
            torch.cuda.synchronize()
            got = y.cpu().numpy()
            expect = y0.copy()
            expect[::6] = [37.0 if r % 2 == 0 else 31.0 for r in range(rows)]
            np.testing.assert_array_equal(got, expect)


def test_guard_bytes_and_misaligned_arrays():
    """Nothing is written outside y, and unaligned colInd / values (sub-array views) still work."""
    rng = np.random.default_rng(12)
    rows, cols = 5000, 4000
    rp, ci = random_csr(rng, rng.integers(0, 50, rows), cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    truth = O.spmv_f64(rp, ci, va, x, np.zeros(rows, np.float32))
    guard = 64
    ybuf = torch.full((rows + 2 * guard,), 777.0, device=DEV)
    cbuf = dev(np.concatenate([[0], ci]).astype(np.int32))      # colInd starts 4 bytes off alignment
    vbuf = dev(np.concatenate([[0, 0, 0], va]).astype(np.float32))  # values start 12 bytes off alignment
    d_rp, d_x = dev(rp), dev(x)
    h = api.Handle()
    mat = api.CsrMatrix(rows, cols, d_rp, cbuf[1:], vbuf[3:], nnz=ci.size)
    op = api.SpMV(h, mat, api.DnVec(d_x), api.DnVec(ybuf[guard:guard + rows]))
    op(1.0, 0.0)
    torch.cuda.synchronize()
    out = ybuf.cpu().numpy()
    assert (out[:guard] == 777.0).all() and (out[-guard:] == 777.0).all()
    assert_close(out[guard:-guard], truth, "misaligned")


def test_garbage_indices_do_not_fault():
    """Out-of-range columns are skipped and wild row offsets are clamped: no fault, finite output."""
    rng = np.random.default_rng(13)
    rows, cols = 3000, 1000
    rp, ci = random_csr(rng, rng.integers(0, 20, rows), cols)
    va = np.ones(ci.size, np.float32)
    bad_ci = ci.copy()
    bad_ci[::7] = cols + 5
    bad_ci[3::11] = -4
    x = np.ones(cols, np.float32)
    got = SpmvCase(rp, bad_ci, va, x, np.zeros(rows, np.float32)).run()
    ok = (bad_ci >= 0) & (bad_ci < cols)
    expect = np.add.reduceat(np.concatenate([ok.astype(np.float64), [0]]), rp[:-1].astype(np.int64))
    expect[np.diff(rp) == 0] = 0
    np.testing.assert_allclose(got, expect, atol=1e-5)
    bad_rp = rp.copy()
    bad_rp[100:200] = rng.integers(-50, ci.size + 50, 100)
    out = SpmvCase(bad_rp, ci, va, x, np.zeros(rows, np.float32)).run()
    assert np.isfinite(out).all()


def test_full_size_stencil_properties():
    """160^3 stencil, the benchmark workload: x = 1 gives y = 27 - len(row) exactly; then the oracle on random x."""
    cfg = workloads.make("c2")
    assert cfg["nnz"] == 478 ** 3
    ones = np.ones(cfg["rows"], np.float32)
    case = SpmvCase(cfg["row_ptr"], cfg["col_ind"], cfg["values"], ones, cfg["y"])
    got = case.run(1.0, 0.0)
    np.testing.assert_array_equal(got, (27 - np.diff(cfg["row_ptr"])).astype(np.float32))
    case.d_x.copy_(torch.from_numpy(cfg["x"]))
    got = case.run(1.0, 0.0, preprocess=False)
    truth = O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], threads=O.max_threads())
    assert_close(got, truth, "c2 full size")
    # linearity: A(2x) == 2*A(x) exactly in floating point
    case.d_x.mul_(2.0)
    twice = case.run(1.0, 0.0, preprocess=False)
    np.testing.assert_array_equal(twice, 2.0 * got)


# ------------------------------------------------------------------ op(A) = transpose --

def _transposed_case(rp, ci, va, x, y, cols, base=0, op=L.OP_T, alg=L.SPMV_ALG_DEFAULT):
    """SpMV with op(A) = T: x has one entry per row of A, y one per column."""
    case = SpmvCase.__new__(SpmvCase)
    case.rows, case.cols, case.nnz = len(rp) - 1, cols, len(ci)
    case.d_rp = dev(np.asarray(rp), np.int32)
    case.d_ci = dev(np.asarray(ci), np.int32) if case.nnz else None
    case.d_va = dev(np.asarray(va), np.float32) if case.nnz else None
    case.d_x, case.d_y = dev(np.asarray(x), np.float32), dev(np.asarray(y), np.float32)
    case.handle = api.Handle()
    case.mat = api.CsrMatrix(case.rows, cols, case.d_rp, case.d_ci, case.d_va, base, nnz=case.nnz)
    case.vx, case.vy = api.DnVec(case.d_x), api.DnVec(case.d_y)
    case.op = api.SpMV(case.handle, case.mat, case.vx, case.vy, alg=alg, op=op)
    return case


def test_transposed_reference_fixture(kats):
    """The reference's transposed cases of its 2x3 fixture (test/spmv/arch35/spmv_test.cpp:69-86, CSV rows with T)."""
    hit = 0
    for k in kats["spmv"]:
        if k.get("op", "N") == "N":
            continue
        hit += 1
        case = _transposed_case(k["row_ptr"], k["col_ind"], k["values"], k["x"], k["y"], k["cols"], base=k["base"])
        got = case.run(k["alpha"], k["beta"])
        np.testing.assert_allclose(got, np.array(k["expect"], np.float32), rtol=0, atol=1e-5, err_msg=k["name"])
    # the fixture itself, spelled out, in case the known-answer file carries no transposed row
    rp, ci, va = [0, 2, 3], [0, 2, 1], [2.0, 3.0, 4.0]
    x, y = [1.0, 2.0], [1.0, 1.0, 1.0]
    for op in (L.OP_T, L.OP_H):
        got = _transposed_case(rp, ci, va, x, y, 3, op=op).run(2.0, 3.0)
        np.testing.assert_allclose(got, [2 * 2 + 3, 2 * 8 + 3, 2 * 3 + 3], atol=1e-5)


def test_transposed_plan_bit_exact():
    """Row offsets, column indices and permutation of the transpose built on the device == the CPU twin."""
    rng = np.random.default_rng(41)
    shapes = [(rng.integers(0, 30, 5000), 3000), (np.clip(rng.zipf(2.0, 4000) * 3, 1, 2500), 2600),
              (np.full(3000, 40), 50), (np.full(200, 900), 1000), (np.zeros(100, int), 70)]
    for base in (0, 1):
        for lengths, cols in shapes:
            rp, ci = random_csr(rng, lengths, cols)
            if ci.size:
                ci = ci.copy()
                ci[::97] = cols + 3            # out-of-range entries are left out of the transpose
            case = _transposed_case(rp + base, ci + base, np.ones(ci.size, np.float32), np.ones(len(lengths), np.float32),
                                    np.zeros(cols, np.float32), cols, base=base)
            case.op.preprocess()
            torch.cuda.synchronize()
            ws = case.op.buffer.cpu().numpy()
            plan = O.spmv_plan_layout(cols, ci.size)
            lay = O.transpose_plan_layout(cols, ci.size, plan["total_bytes"])
            assert ws.size == lay["total_bytes"]
            rpt, cit, perm = O.transpose_twin(rp + base, ci + base, cols, base)
            kept = int(rpt[-1])
            assert np.array_equal(ws[lay["row_ptr_off"]:lay["row_ptr_off"] + 4 * (cols + 1)].view(np.int32), rpt)
            assert np.array_equal(ws[lay["perm_off"]:lay["perm_off"] + 4 * kept].view(np.int32), perm)
            assert np.array_equal(ws[lay["col_ind_off"]:lay["col_ind_off"] + 4 * kept].view(np.int32), cit)


@pytest.mark.parametrize("name,rows", [("c1", None), ("c2", 40 ** 3), ("c3", 1 << 16)])
def test_transposed_benchmark_shapes_vs_oracle(name, rows):
    cfg = workloads.make(name, rows=rows)
    rng = np.random.default_rng(7)
    x = rng.standard_normal(cfg["rows"]).astype(np.float32)
    y = rng.uniform(-1, 1, cfg["cols"]).astype(np.float32)
    truth = O.spmv_transpose_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], x, y, cfg["cols"], 1.5, 0.5)
    case = _transposed_case(cfg["row_ptr"], cfg["col_ind"], cfg["values"], x, y, cfg["cols"])
    got = case.run(1.5, 0.5)
    assert_close(got, truth, name + " transposed")
    for _ in range(3):  # bit-wise reproducible (reference: test/spmv/arch22/spmv_test.cpp:1184)
        case.d_y.copy_(torch.from_numpy(y))
        again = case.run(1.5, 0.5, preprocess=False)
        assert np.array_equal(again.view(np.uint32), got.view(np.uint32))
    # new values through the same plan: the permutation is applied at every product
    va2 = (cfg["values"] * 0.5 + 1.0).astype(np.float32)
    case.d_va.copy_(torch.from_numpy(va2))
    case.d_y.copy_(torch.from_numpy(y))
    got = case.run(1.5, 0.5, preprocess=False)
    assert_close(got, O.spmv_transpose_f64(cfg["row_ptr"], cfg["col_ind"], va2, x, y, cfg["cols"], 1.5, 0.5),
                 name + " transposed, new values")


def test_transposed_long_columns():
    """Columns with far more than 32 and than 2048 entries: every tier of the in-column sort."""
    rng = np.random.default_rng(43)
    rows, cols = 9000, 40
    lengths = rng.integers(20, 40, rows)                     # every column gets about 6000 entries
    rp, ci = random_csr(rng, lengths, cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    x = rng.standard_normal(rows).astype(np.float32)
    y = np.zeros(cols, np.float32)
    got = _transposed_case(rp, ci, va, x, y, cols).run(1.0, 0.0)
    assert_close(got, O.spmv_transpose_f64(rp, ci, va, x, y, cols, 1.0, 0.0), "long columns")
