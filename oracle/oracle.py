"""TEST INFRASTRUCTURE ONLY: Python face of the CPU oracle.

Loads ``oracle/liboracle.so`` (the C restatement in ``oracle.c``) and, when it
was built, ``oracle/_ref/libref_host.so`` (a few of the reference's own host
sources compiled where they lie).  Only the tests, the smoke run and the
benchmark's CPU-baseline leg import this module; the shipped library never does.

Every function takes and returns numpy arrays.  The reference file:line each
one follows is given in ``oracle.c`` next to the C function it calls.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_host.so")

RTOL = 1e-5  # tolerance of the fp32 outputs against the fp64 truth
ATOL = 1e-6


def build(ref: bool = True) -> None:
    """Compile the oracle (and the reference-backed library when the reference checkout exists)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    if ref:
        where = os.environ.get("OPS_SPARSE_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={where}"], check=True, capture_output=True)


def _load():
    if not os.path.exists(_LIB_PATH):
        build(ref=False)
    return ctypes.CDLL(_LIB_PATH)


_lib = _load()


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


_lib.oracle_spmv_f64.argtypes = [c_int64] + [c_void_p] * 6 + [c_float, c_float, c_int32, c_int]
_lib.oracle_spmv_f32.argtypes = [c_int64] + [c_void_p] * 6 + [c_float, c_float, c_int32]
_lib.oracle_spmv_transpose_f64.argtypes = [c_int64, c_int64] + [c_void_p] * 6 + [c_float, c_float, c_int32]
_lib.oracle_spmm_f32.argtypes = [c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                 c_void_p, c_int64, c_int, c_float, c_float, c_int32, c_int]
_lib.oracle_spmm_f64.argtypes = [c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                 c_int, c_void_p, c_int64, c_int, c_void_p, c_float, c_float, c_int32, c_int64,
                                 c_int64, c_int]
_lib.oracle_normalize_row_offsets.argtypes = [c_void_p, c_int64, c_int32, c_int64, c_void_p]
_lib.oracle_ref_spmv_workspace_bytes.argtypes = [c_uint64]
_lib.oracle_ref_spmv_workspace_bytes.restype = c_uint64
_lib.oracle_ref_spmm_workspace_bytes.argtypes = [c_uint64, c_uint64]
_lib.oracle_ref_spmm_workspace_bytes.restype = c_uint64
_lib.oracle_greedy_row_bin_pack.argtypes = [c_void_p, c_int32, c_int32, c_void_p, c_void_p, POINTER(c_int32)]
_lib.oracle_greedy_row_bin_pack.restype = c_int
_lib.oracle_plan_tiles.argtypes = [c_void_p, c_int64, c_int64, c_uint32, c_uint32, c_void_p, c_void_p]
_lib.oracle_row_block_bounds.argtypes = [c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p]
_lib.oracle_check_tolerance.argtypes = [c_void_p, c_void_p, c_int64, c_double, c_double, POINTER(c_double),
                                        POINTER(c_double)]
_lib.oracle_check_tolerance.restype = c_int64
_lib.oracle_max_threads.restype = c_int


def max_threads() -> int:
    return int(_lib.oracle_max_threads())


# ------------------------------------------------------------------ SpMV --

def spmv_f64(row_ptr, col_ind, values, x, y, alpha=1.0, beta=0.0, index_base=0, threads=1) -> np.ndarray:
    """fp64-accumulated truth of alpha*A*x + beta*y (what the reference's tests compare fp32 SpMV against)."""
    row_ptr, col_ind, values, x, y = _i32(row_ptr), _i32(col_ind), _f32(values), _f32(x), _f32(y)
    rows = row_ptr.size - 1
    out = np.empty(rows, dtype=np.float64)
    _lib.oracle_spmv_f64(rows, _ptr(row_ptr), _ptr(col_ind), _ptr(values), _ptr(x), _ptr(y), _ptr(out),
                         alpha, beta, index_base, threads)
    return out


def spmv_f32(row_ptr, col_ind, values, x, y, alpha=1.0, beta=0.0, index_base=0) -> np.ndarray:
    row_ptr, col_ind, values, x, y = _i32(row_ptr), _i32(col_ind), _f32(values), _f32(x), _f32(y)
    rows = row_ptr.size - 1
    out = np.empty(rows, dtype=np.float32)
    _lib.oracle_spmv_f32(rows, _ptr(row_ptr), _ptr(col_ind), _ptr(values), _ptr(x), _ptr(y), _ptr(out),
                         alpha, beta, index_base)
    return out


def spmv_transpose_f64(row_ptr, col_ind, values, x, y, cols, alpha=1.0, beta=0.0, index_base=0) -> np.ndarray:
    row_ptr, col_ind, values, x, y = _i32(row_ptr), _i32(col_ind), _f32(values), _f32(x), _f32(y)
    out = np.empty(cols, dtype=np.float64)
    _lib.oracle_spmv_transpose_f64(row_ptr.size - 1, cols, _ptr(row_ptr), _ptr(col_ind), _ptr(values), _ptr(x),
                                   _ptr(y), _ptr(out), alpha, beta, index_base)
    return out


# ------------------------------------------------------------------ SpMM --

def spmm_f32(row_ptr, col_ind, values, b, ldb, c, ldc, n, alpha=1.0, beta=0.0, b_row_major=True,
             op_b_transpose=False, c_row_major=True, index_base=0, threads=1) -> np.ndarray:
    """fp32 golden; ``b`` and ``c`` are flat storage arrays, the updated copy of ``c`` is returned."""
    row_ptr, col_ind, values, b = _i32(row_ptr), _i32(col_ind), _f32(values), _f32(b)
    out = np.array(c, dtype=np.float32, copy=True).ravel()
    _lib.oracle_spmm_f32(row_ptr.size - 1, n, _ptr(row_ptr), _ptr(col_ind), _ptr(values), _ptr(b), ldb,
                         int(b_row_major), int(op_b_transpose), _ptr(out), ldc, int(c_row_major), alpha, beta,
                         index_base, threads)
    return out


def spmm_f64(row_ptr, col_ind, values, b, ldb, c, ldc, n, k, alpha=1.0, beta=0.0, b_row_major=True,
             op_b_transpose=False, c_row_major=True, index_base=0, row_begin=0, row_end=None,
             threads=1) -> np.ndarray:
    """fp64 truth of rows [row_begin, row_end), returned row-major with n columns."""
    row_ptr, col_ind, values, b = _i32(row_ptr), _i32(col_ind), _f32(values), _f32(b)
    c = _f32(c).ravel()
    m = row_ptr.size - 1
    row_end = m if row_end is None else row_end
    out = np.empty((row_end - row_begin, n), dtype=np.float64)
    _lib.oracle_spmm_f64(m, n, k, _ptr(row_ptr), _ptr(col_ind), _ptr(values), _ptr(b), ldb, int(b_row_major),
                         int(op_b_transpose), _ptr(c), ldc, int(c_row_major), _ptr(out), alpha, beta, index_base,
                         row_begin, row_end, threads)
    return out


# -------------------------------------------------------------- metadata --

def normalize_row_offsets(row_ptr, rows, index_base=0, stride=1) -> np.ndarray:
    row_ptr = _i32(row_ptr)
    out = np.empty(rows + 1, dtype=np.int32)
    _lib.oracle_normalize_row_offsets(_ptr(row_ptr), rows, index_base, stride, _ptr(out))
    return out


def ref_spmv_workspace_bytes(rows: int) -> int:
    return int(_lib.oracle_ref_spmv_workspace_bytes(rows))


def ref_spmm_workspace_bytes(m: int, bins: int) -> int:
    return int(_lib.oracle_ref_spmm_workspace_bytes(m, bins))


def greedy_row_bin_pack(row_nnz, bins: int):
    """Returns (reorder, bin_edges, identity_reorder, uniform_degree) of the reference's SpMM preprocessing."""
    row_nnz = _i32(row_nnz)
    reorder = np.empty(row_nnz.size, dtype=np.int32)
    edges = np.empty(bins + 1, dtype=np.int32)
    uniform = c_int32(0)
    identity = _lib.oracle_greedy_row_bin_pack(_ptr(row_nnz), row_nnz.size, bins, _ptr(reorder), _ptr(edges),
                                               ctypes.byref(uniform))
    return reorder, edges, bool(identity), int(uniform.value)


SPMV_TILE_ITEMS = 2048
SPMM_TILE_ITEMS = 1024
SPMV_CLASS_DIV = 16
HEADER_BYTES = 192
PLAN_MAGIC = 0x30303242


def _align64(v: int) -> int:
    return (v + 63) & ~63


def plan_layout(rows: int, nnz: int, tile_items: int, carry_bytes_per_tile: int) -> dict:
    """Offsets of the B200 plan inside the external buffer (twin of plan_layout.h)."""
    num_tiles = (rows + nnz + tile_items - 1) // tile_items
    row_ptr_off = HEADER_BYTES
    tile_row_off = _align64(row_ptr_off + 4 * (rows + 1))
    tile_class_off = _align64(tile_row_off + 4 * (num_tiles + 1))
    carry_off = _align64(tile_class_off + 4 * num_tiles)
    total = _align64(carry_off + carry_bytes_per_tile * num_tiles)
    return dict(num_tiles=num_tiles, row_ptr_off=row_ptr_off, tile_row_off=tile_row_off,
                tile_class_off=tile_class_off, carry_off=carry_off, total_bytes=total)


def spmv_plan_layout(rows: int, nnz: int) -> dict:
    return plan_layout(rows, nnz, SPMV_TILE_ITEMS, 16)


def spmm_plan_layout(rows: int, nnz: int, dense_cols: int) -> dict:
    return plan_layout(rows, nnz, SPMM_TILE_ITEMS, 16 * dense_cols)


def plan_tiles(row_ptr_n, nnz: int, tile_items: int, class_div: int):
    """Merge-path tile splits and per-tile row bins (twin of the device preprocessing pass)."""
    row_ptr_n = _i32(row_ptr_n)
    rows = row_ptr_n.size - 1
    num_tiles = (rows + nnz + tile_items - 1) // tile_items
    tile_row = np.empty(num_tiles + 1, dtype=np.int32)
    tile_class = np.empty(num_tiles, dtype=np.int32)
    _lib.oracle_plan_tiles(_ptr(row_ptr_n), rows, nnz, tile_items, class_div, _ptr(tile_row), _ptr(tile_class))
    return tile_row, tile_class


def plan_header(kind: int, rows: int, cols: int, nnz: int, index_base: int, dense_cols: int, layout: dict,
                tile_items: int) -> np.ndarray:
    """The 80 meaningful bytes of the plan header, as the device writes them."""
    head = np.zeros(10, dtype=np.uint32)
    head[:] = [PLAN_MAGIC, 1, kind, tile_items, rows, cols, nnz, index_base, layout["num_tiles"], dense_cols]
    tail = np.array([layout["row_ptr_off"], layout["tile_row_off"], layout["tile_class_off"], layout["carry_off"],
                     layout["total_bytes"]], dtype=np.uint64)
    return np.concatenate([head.view(np.uint8), tail.view(np.uint8)])


def longest_row(row_ptr) -> int:
    """Longest row as the SpMV preprocessing pass records it in the plan header (a negative length counts as 0)."""
    d = np.diff(np.asarray(row_ptr, dtype=np.int64))
    return int(max(d.max(), 0)) if d.size else 0


def transpose_plan_layout(rows_t: int, nnz: int, plan_bytes: int) -> dict:
    """Offsets of the transpose behind the plan of the transposed matrix (twin of aclspTransposeLayout)."""
    col_ind_off = _align64(plan_bytes)
    perm_off = _align64(col_ind_off + 4 * nnz)
    values_off = _align64(perm_off + 4 * nnz)
    cursor_off = _align64(values_off + 4 * nnz)
    scan_off = _align64(cursor_off + 4 * (rows_t + 2))
    total = _align64(scan_off + 4 * (rows_t // 512 + 16))
    return dict(row_ptr_off=HEADER_BYTES, col_ind_off=col_ind_off, perm_off=perm_off, values_off=values_off,
                cursor_off=cursor_off, scan_off=scan_off, total_bytes=total)


def transpose_twin(row_ptr, col_ind, cols: int, index_base=0):
    """CPU twin of the device transpose build: (row offsets, column indices, permutation) of A^T as CSR.
    A stable counting sort by column: entries of one column keep their original order, entries whose
    column is out of range are left out."""
    rp = np.clip(np.asarray(row_ptr, dtype=np.int64) - index_base, 0, len(col_ind))
    rows = rp.size - 1
    lens = np.maximum(np.diff(rp), 0)
    row_of = np.full(len(col_ind), -1, dtype=np.int64)
    for r in np.flatnonzero(lens):
        row_of[rp[r]:rp[r] + lens[r]] = r
    c = np.asarray(col_ind, dtype=np.int64) - index_base
    kept = np.flatnonzero((row_of >= 0) & (c >= 0) & (c < cols))
    perm = kept[np.argsort(c[kept], kind="stable")]
    row_ptr_t = np.concatenate([[0], np.cumsum(np.bincount(c[kept], minlength=cols))]).astype(np.int32)
    return row_ptr_t, row_of[perm].astype(np.int32), perm.astype(np.int32)


def coo2csr_twin(coo_rows, m: int, index_base=0) -> np.ndarray:
    """Row offsets of sorted COO row indices (twin of aclsparseXcoo2csr; reference semantics:
    include/cann_ops_sparse.h:2783-2799, counting + prefix sum)."""
    rows = np.asarray(coo_rows, dtype=np.int64) - index_base
    return (np.searchsorted(rows, np.arange(m + 1), side="left") + index_base).astype(np.int32)


def csrsort_twin(row_ptr, col_ind, perm, index_base=0):
    """Stable in-row sort of CSR column indices and the same permutation applied to perm (twin of
    aclsparseXcsrsort; reference semantics: include/cann_ops_sparse.h:2531-2544)."""
    rp = np.asarray(row_ptr, dtype=np.int64) - index_base
    col = np.array(col_ind, dtype=np.int32, copy=True)
    out = np.array(perm, dtype=np.int32, copy=True)
    for r in range(rp.size - 1):
        b, e = int(rp[r]), int(rp[r + 1])
        if e - b > 1:
            order = np.argsort(col[b:e], kind="stable")
            col[b:e] = col[b:e][order]
            out[b:e] = out[b:e][order]
    return col, out


def row_block_bounds(row_ptr, nnz: int, parts: int, index_base=0) -> np.ndarray:
    row_ptr = _i32(row_ptr)
    bounds = np.empty(parts + 1, dtype=np.int32)
    _lib.oracle_row_block_bounds(_ptr(row_ptr), row_ptr.size - 1, nnz, index_base, parts, _ptr(bounds))
    return bounds


# ---------------------------------------------------------- narrow types --
# fp16 / bf16 / int8 storage (the reference's table, sparse/spmv/arch35/spmv_host.cpp:44-66).  Every such
# value is exactly an fp32 number, so the fp64 truth of a narrow product is spmv_f64 on the widened arrays;
# what differs is the rounding of the result, restated here: to nearest, ties to even, once
# (sparse/spmv/arch35/spmv_kernel.cpp:104-160 for the two 16-bit formats), and the saturating integer form.

def bf16_bits_to_f32(bits) -> np.ndarray:
    """bf16 bit patterns (uint16) as fp32 numbers: a bf16 is the upper half of an fp32."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(v) -> np.ndarray:
    """fp32 -> bf16 bit patterns, to nearest even (NaN stays NaN)."""
    b = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32)
    rounded = ((b.astype(np.uint64) + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(v, dtype=np.float32))
    return np.where(nan, np.uint16(0x7FC0), rounded)


def f64_to_bf16_bits(v) -> np.ndarray:
    """fp64 -> bf16 with ONE rounding to nearest even: the double is first rounded to fp32 to odd (truncate
    toward zero, set the last bit when inexact), which keeps enough information for the final rounding."""
    v = np.ascontiguousarray(v, dtype=np.float64)
    with np.errstate(over="ignore", invalid="ignore"):
        f = v.astype(np.float32)
        too_big = np.isfinite(f) & (np.abs(f.astype(np.float64)) > np.abs(v))
        f = np.where(too_big, np.nextafter(f, np.float32(0)), f).astype(np.float32)
        inexact = np.isfinite(f) & (f.astype(np.float64) != v)
    bits = f.view(np.uint32) | inexact.astype(np.uint32)
    # a finite double beyond the fp32 range rounds to infinity in bf16 as well
    with np.errstate(over="ignore"):
        overflow = np.isfinite(v) & np.isinf(v.astype(np.float32))
    out = f32_to_bf16_bits(bits.view(np.float32))
    sign = (np.signbit(v).astype(np.uint16) << 15)
    return np.where(overflow, sign | np.uint16(0x7F80), out)


def f64_to_f16(v) -> np.ndarray:
    """fp64 -> fp16, one rounding to nearest even (numpy converts from the double directly)."""
    with np.errstate(over="ignore"):
        return np.ascontiguousarray(v, dtype=np.float64).astype(np.float16)


def spmv_i8_i32(row_ptr, col_ind, values, x, y, alpha: int, beta: int, index_base=0) -> np.ndarray:
    """int8 data, int32 scalars and result: the exact integer alpha*sum + beta*y saturated to the int32 range
    (the reference forms the same value by case analysis, sparse/spmv/arch35/spmv_kernel.cpp:347-375).
    beta == 0 does not read y.  Python integers: exact at any size."""
    row_ptr, col_ind = _i32(row_ptr), _i32(col_ind)
    va = np.asarray(values, dtype=np.int64)
    xv = np.asarray(x, dtype=np.int64)
    rows = row_ptr.size - 1
    out = np.empty(rows, dtype=np.int32)
    for r in range(rows):
        b, e = int(row_ptr[r]) - index_base, int(row_ptr[r + 1]) - index_base
        cols = col_ind[b:e].astype(np.int64) - index_base
        ok = (cols >= 0) & (cols < xv.size)
        total = int(np.sum(va[b:e][ok] * xv[cols[ok]]))
        val = int(alpha) * total + (int(beta) * int(y[r]) if beta != 0 else 0)
        out[r] = max(-2**31, min(2**31 - 1, val))
    return out


# -------------------------------------------------------------- verifier --

def check_tolerance(got, truth, rtol=RTOL, atol=ATOL):
    """Returns (violations, max_abs_err, max_rel_err) of |got - truth| <= atol + rtol*|truth| per element."""
    got = _f32(got).ravel()
    truth = np.ascontiguousarray(truth, dtype=np.float64).ravel()
    assert got.size == truth.size
    max_abs, max_rel = c_double(0.0), c_double(0.0)
    bad = _lib.oracle_check_tolerance(_ptr(got), _ptr(truth), got.size, rtol, atol, ctypes.byref(max_abs),
                                      ctypes.byref(max_rel))
    return int(bad), float(max_abs.value), float(max_rel.value)


# ------------------------------------------- the reference's own code --

def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


_ref = None


def ref():
    """The reference-backed library (only exists where the reference checkout was available at build time)."""
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF_PATH)
        _ref.ref_spmm_golden_f64.argtypes = [c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                             c_void_p, c_void_p, c_double, c_double, c_int, c_int32, c_void_p]
        _ref.ref_fill_csr.argtypes = [c_int64, c_int64, c_double, c_double, c_double, c_double, c_uint32, c_void_p,
                                      c_void_p, c_void_p, c_int64]
        _ref.ref_fill_csr.restype = c_int64
        _ref.ref_fill_dense.argtypes = [c_int64, c_double, c_double, c_uint32, c_void_p]
        _ref.ref_spmv_workspace_bytes.argtypes = [c_uint64, c_uint64, c_int]
        _ref.ref_spmv_workspace_bytes.restype = c_uint64
        _ref.ref_spmm_row_reorder.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p,
                                              POINTER(c_int), POINTER(c_int32)]
        _ref.ref_spmm_row_reorder.restype = c_uint32
    return _ref


def ref_spmm_golden_f64(row_ptr, col_ind, values, b, c_init, m, n, k, alpha, beta, op_b_transpose=False,
                        index_base=0) -> np.ndarray:
    row_ptr, col_ind, values = _i32(row_ptr), _i32(col_ind), _f32(values)
    b, c_init = _f32(b).ravel(), _f32(c_init).ravel()
    out = np.empty((m, n), dtype=np.float64)
    ref().ref_spmm_golden_f64(m, n, k, _ptr(row_ptr), _ptr(col_ind), _ptr(values), values.size, _ptr(b),
                              _ptr(c_init), alpha, beta, int(op_b_transpose), index_base, _ptr(out))
    return out


def ref_fill_csr(rows, cols, sparsity, seed, empty_row_prob=0.0, lo=-2.0, hi=2.0):
    cap = max(16, int(rows * cols * (1.0 - sparsity) * 1.5) + 4 * int(rows) + 64)
    while True:
        rp = np.empty(rows + 1, dtype=np.int32)
        ci = np.empty(cap, dtype=np.int32)
        va = np.empty(cap, dtype=np.float32)
        nnz = ref().ref_fill_csr(rows, cols, sparsity, empty_row_prob, lo, hi, seed, _ptr(rp), _ptr(ci), _ptr(va),
                                 cap)
        if nnz <= cap:
            return rp, ci[:nnz].copy(), va[:nnz].copy()
        cap = int(nnz)


def ref_fill_dense(size, seed, lo=-2.0, hi=2.0) -> np.ndarray:
    out = np.empty(size, dtype=np.float32)
    ref().ref_fill_dense(size, lo, hi, seed, _ptr(out))
    return out


def ref_spmv_workspace_bytes_real(rows: int, cols: int, transpose=False) -> int:
    return int(ref().ref_spmv_workspace_bytes(rows, cols, int(transpose)))


def ref_spmm_row_reorder(row_ptr, k: int, bins: int):
    row_ptr = _i32(row_ptr)
    m = row_ptr.size - 1
    nnz = int(row_ptr[-1] - row_ptr[0])
    reorder = np.empty(m, dtype=np.int32)
    edges = np.empty(bins + 1, dtype=np.int32)
    identity, uniform = c_int(0), c_int32(0)
    st = ref().ref_spmm_row_reorder(_ptr(row_ptr), m, k, nnz, bins, _ptr(reorder), _ptr(edges),
                                    ctypes.byref(identity), ctypes.byref(uniform))
    assert st == 0, st
    return reorder, edges, bool(identity.value), int(uniform.value)
