"""The CPU oracle against the reference's golden vectors and known answers (no GPU)."""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _arr(v, dt):
    return np.array(v, dtype=dt)


def test_spmv_known_answers(kats):
    for k in kats["spmv"]:
        rp, ci, va = _arr(k["row_ptr"], np.int32), _arr(k["col_ind"], np.int32), _arr(k["values"], np.float32)
        x, y = _arr(k["x"], np.float32), _arr(k["y"], np.float32)
        got = O.spmv_f64(rp, ci, va, x, y, k["alpha"], k["beta"], k["base"])
        np.testing.assert_array_equal(got, np.array(k["expect"], dtype=np.float64), err_msg=k["name"])
        got32 = O.spmv_f32(rp, ci, va, x, y, k["alpha"], k["beta"], k["base"])
        expect32 = k.get("expect_fp32_rounded", k["expect"])
        np.testing.assert_array_equal(got32, np.array(expect32, dtype=np.float32), err_msg=k["name"])
        if "expect_second" in k:  # the same call again, on the output of the first
            again = O.spmv_f64(rp, ci, va, x, got.astype(np.float32), k["alpha"], k["beta"], k["base"])
            np.testing.assert_array_equal(again, np.array(k["expect_second"], dtype=np.float64))


def test_spmv_transpose_known_answers(kats):
    for k in kats["spmv_transpose"]:
        got = O.spmv_transpose_f64(_arr(k["row_ptr"], np.int32), _arr(k["col_ind"], np.int32),
                                   _arr(k["values"], np.float32), _arr(k["x"], np.float32),
                                   _arr(k["y"], np.float32), k["cols"], k["alpha"], k["beta"], k["base"])
        np.testing.assert_array_equal(got, np.array(k["expect"], dtype=np.float64))


def test_spmm_known_answers(kats):
    for k in kats["spmm"]:
        rp, ci, va = _arr(k["row_ptr"], np.int32), _arr(k["col_ind"], np.int32), _arr(k["values"], np.float32)
        b, c = _arr(k["b"], np.float32), _arr(k["c"], np.float32)
        n = k["n"]
        got = O.spmm_f32(rp, ci, va, b, n, c, n, n, k["alpha"], k["beta"], index_base=k["base"]).reshape(k["m"], n)
        np.testing.assert_array_equal(got, np.array(k["expect"], dtype=np.float32))
        got64 = O.spmm_f64(rp, ci, va, b, n, c, n, n, k["k"], k["alpha"], k["beta"], index_base=k["base"])
        np.testing.assert_array_equal(got64, np.array(k["expect"], dtype=np.float64))


def test_spmm_layouts_agree():
    """Column-major B / C and op(B) = T are views of the same product (SpmmCpuFp32's index rules)."""
    rng = np.random.default_rng(3)
    m, k, n = 19, 13, 7
    lens = rng.integers(0, 6, m)
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(k, l, replace=False)) for l in lens]).astype(np.int32)
    va = rng.uniform(-1, 1, ci.size).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    base = O.spmm_f32(rp, ci, va, b, n, c, n, n, -0.75, 0.5).reshape(m, n)
    # column-major B with padding, column-major C with padding
    ldb, ldc = k + 3, m + 2
    b_col = np.zeros((n, ldb), np.float32); b_col[:, :k] = b.T
    c_col = np.zeros((n, ldc), np.float32); c_col[:, :m] = c.T
    got = O.spmm_f32(rp, ci, va, b_col, ldb, c_col, ldc, n, -0.75, 0.5, b_row_major=False, c_row_major=False)
    np.testing.assert_array_equal(got.reshape(n, ldc)[:, :m].T, base)
    # op(B) = T: B stored n x k row-major
    got_t = O.spmm_f32(rp, ci, va, np.ascontiguousarray(b.T), k, c, n, n, -0.75, 0.5, op_b_transpose=True)
    np.testing.assert_array_equal(got_t.reshape(m, n), base)


def test_oracle_matches_reference_goldens(goldens):
    """fp64 truth of the oracle == the reference's SpmmGolden on inputs from the reference's generator."""
    for name, g in goldens.items():
        n = g["n"]
        got = O.spmm_f64(g["row_ptr"], g["col_ind"], g["values"], g["b"], n, g["c0"], n, n, g["cols"], g["alpha"],
                         g["beta"], index_base=g["base"])
        np.testing.assert_array_equal(got, g["truth"], err_msg=name)
        if n == 1:  # one dense column: the SpMV golden
            y = O.spmv_f64(g["row_ptr"], g["col_ind"], g["values"], g["b"][:, 0], g["c0"][:, 0], g["alpha"],
                           g["beta"], g["base"])
            np.testing.assert_array_equal(y, g["truth"][:, 0], err_msg=name)
            # the fp32 golden stays within the reference's own fp32 tolerance of the truth
            y32 = O.spmv_f32(g["row_ptr"], g["col_ind"], g["values"], g["b"][:, 0], g["c0"][:, 0], g["alpha"],
                             g["beta"], g["base"])
            bad, _, _ = O.check_tolerance(y32, g["truth"][:, 0], rtol=2.0 ** -10, atol=2.0 ** -16)
            assert bad <= 0.01 * y32.size


def test_row_reorder_matches_reference():
    data = np.load(os.path.join(GOLDEN_DIR, "reference_row_reorder.npz"))
    keys = sorted({k.rsplit(".", 1)[0] for k in data.files})
    assert keys
    for key in keys:
        bins = int(key.split(".")[1])
        rp = data[key + ".row_ptr"]
        reorder, edges, identity, uniform = O.greedy_row_bin_pack(np.diff(rp), bins)
        np.testing.assert_array_equal(reorder, data[key + ".reorder"], err_msg=key)
        np.testing.assert_array_equal(edges, data[key + ".edges"], err_msg=key)
        assert [int(identity), uniform] == list(data[key + ".flags"]), key


def test_reference_workspace_sizes(kats):
    data = np.load(os.path.join(GOLDEN_DIR, "reference_spmv_workspace_bytes.npz"))
    for rows, expect in zip(data["rows"], data["bytes"]):
        assert O.ref_spmv_workspace_bytes(int(rows)) == int(expect)
    k = kats["ref_spmm_buffer_size"]
    assert O.ref_spmm_workspace_bytes(k["m"], k["bins"]) == k["bytes"]


def test_normalize_row_offsets():
    rp = np.array([1, -9, 3, -9, 4, -9], dtype=np.int32)  # stride 2, base 1
    np.testing.assert_array_equal(O.normalize_row_offsets(rp, 2, index_base=1, stride=2), [0, 2, 3])


def test_verifier_self_checks():
    """The tolerance check itself: exact, at the limit, just outside, NaN (as spmv_test_verification.h:111-165 does)."""
    truth = np.array([1.0, 100.0, 0.0, 5.0])
    ok = truth.astype(np.float32)
    assert O.check_tolerance(ok, truth)[0] == 0
    off = ok.copy(); off[1] = np.float32(100.0 * (1 + 3e-5))
    assert O.check_tolerance(off, truth)[0] == 1
    nan = ok.copy(); nan[3] = np.nan
    assert O.check_tolerance(nan, truth)[0] == 1
    tiny = ok.copy(); tiny[2] = np.float32(9e-7)
    assert O.check_tolerance(tiny, truth)[0] == 0


def test_plan_twin_invariants():
    """Merge-path splits: monotone, cover everything, at most T items per tile, classes in range."""
    rng = np.random.default_rng(5)
    for lens in (rng.poisson(16, 5000), np.clip(rng.zipf(2.0, 3000), 1, 9000), np.zeros(5000, int),
                 np.array([30000]), np.array([0, 0, 5000, 0])):
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        nnz, rows = int(rp[-1]), lens.size
        for tile, div in ((2048, 16), (1024, 1)):
            tile_row, tile_class = O.plan_tiles(rp, nnz, tile, div)
            nt = tile_row.size - 1
            assert nt == (rows + nnz + tile - 1) // tile
            assert tile_row[0] == 0 and tile_row[-1] == rows
            assert (np.diff(tile_row) >= 0).all()
            d = np.minimum(np.arange(nt + 1, dtype=np.int64) * tile, rows + nnz)
            j = d - tile_row
            assert (np.diff(j) >= 0).all() and j[-1] == nnz
            # every row that ends before a tile really ends at or before the tile's first non-zero
            assert (rp[tile_row] <= np.maximum(j, rp[tile_row])).all()
            assert ((tile_class >= 0) & (tile_class <= 5)).all()


def test_row_block_bounds_twin():
    rng = np.random.default_rng(9)
    lens = np.clip(rng.zipf(2.0, 4000), 1, 3000)
    lens[-7:] = 0  # trailing empty rows still belong to the last block
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    nnz = int(rp[-1])
    for parts in (1, 2, 4, 8):
        b = O.row_block_bounds(rp, nnz, parts)
        assert b[0] == 0 and b[-1] == lens.size and (np.diff(b) >= 0).all()
        per = np.diff(rp[b])
        assert per.sum() == nnz and per.max() <= nnz / parts + lens.max()
        b1 = O.row_block_bounds(rp + 1, nnz, parts, index_base=1)
        np.testing.assert_array_equal(b, b1)


@pytest.mark.skipif(not O.have_ref(), reason="reference-backed library was not built (no reference checkout)")
def test_oracle_against_live_reference():
    """Where the reference's sources were compiled, compare on fresh inputs beyond the committed fixtures."""
    for seed in (101, 102, 103):
        rows, cols, n = 150 + seed % 7, 211, 1 + seed % 5
        rp, ci, va = O.ref_fill_csr(rows, cols, 0.93, seed, empty_row_prob=0.1)
        b = O.ref_fill_dense(cols * n, seed + 1).reshape(cols, n)
        c0 = O.ref_fill_dense(rows * n, seed + 2).reshape(rows, n)
        ref = O.ref_spmm_golden_f64(rp, ci, va, b, c0, rows, n, cols, 1.25, -0.5)
        got = O.spmm_f64(rp, ci, va, b, n, c0, n, n, cols, 1.25, -0.5)
        np.testing.assert_array_equal(got, ref)
        r, e, ident, uni = O.ref_spmm_row_reorder(rp, cols, 24)
        r2, e2, ident2, uni2 = O.greedy_row_bin_pack(np.diff(rp), 24)
        np.testing.assert_array_equal(r, r2)
        np.testing.assert_array_equal(e, e2)
        assert (ident, uni) == (ident2, uni2)


def test_narrow_roundings_are_single_and_to_nearest_even():
    """The oracle's fp64 -> bf16 / fp16 conversions (what the narrow-type GPU results are compared with) against
    exact rational arithmetic: nearest bf16 / fp16 value, ties to even, including values a hair off a tie, where a
    detour through fp32 rounds the wrong way.  int8 -> int32: exact integers, saturated."""
    from fractions import Fraction
    rng = np.random.default_rng(12)

    def nearest(v, values):
        """Index of the value nearest to v in the ascending list `values`, ties to the even index."""
        lo, hi = 0, len(values) - 1
        a = Fraction(float(v))
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if values[mid] <= a:
                lo = mid
            else:
                hi = mid
        dl, dh = a - values[lo], values[hi] - a
        return lo if dl < dh or (dl == dh and lo % 2 == 0) else hi

    # all positive finite bf16 values from 2^-20 to 2^20, as exact fractions
    bits = np.arange(0x3580, 0x4980, dtype=np.uint16)
    grid = [Fraction(float(f)) for f in O.bf16_bits_to_f32(bits)]
    base = np.array([float(g) for g in grid[:-1]])
    mid = (base + np.array([float(g) for g in grid[1:]])) / 2          # exact: one more bit
    probes = np.concatenate([rng.uniform(float(grid[0]), float(grid[-1]), 300), mid[::16],
                             mid[::16] * (1 + 2.0 ** -40), mid[::16] * (1 - 2.0 ** -40)])
    got = O.f64_to_bf16_bits(probes)
    want = np.array([bits[nearest(v, grid)] for v in probes], dtype=np.uint16)
    assert np.array_equal(got, want)
    assert np.array_equal(O.f64_to_bf16_bits(-probes), want | np.uint16(0x8000))
    # fp16 the same way, around 1.0
    hbits = np.arange(0x3800, 0x4000, dtype=np.uint16)
    hgrid = [Fraction(float(f)) for f in hbits.view(np.float16)]
    hmid = np.array([float((a + b) / 2) for a, b in zip(hgrid[:-1], hgrid[1:])])
    hprobes = np.concatenate([hmid[::8], hmid[::8] * (1 + 2.0 ** -40), hmid[::8] * (1 - 2.0 ** -40)])
    assert np.array_equal(O.f64_to_f16(hprobes).view(np.uint16),
                          np.array([hbits[nearest(v, hgrid)] for v in hprobes], dtype=np.uint16))
    # the reference's own known answers (test/spmv/arch35/spmv_test.cpp:665-697): 1 + 2^-11 -> 1 in fp16
    assert O.f64_to_f16(np.array([1 + 2.0 ** -11, -(1 + 2.0 ** -11)])).view(np.uint16).tolist() == [0x3C00, 0xBC00]
    # int8 x int8 -> int32 with saturation (test/spmv/arch35/spmv_test.cpp:617-663)
    got = O.spmv_i8_i32([0, 1, 2, 2], [0, 1], np.array([127, -127], np.int8), np.array([127, 127], np.int8),
                        np.zeros(3, np.int32), 2 ** 31 - 1, 0)
    assert got.tolist() == [2 ** 31 - 1, -2 ** 31, 0]
