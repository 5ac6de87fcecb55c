"""Seeded synthetic inputs for the five benchmark configurations.

The reference's acceptance cases are shaped like public graph datasets that
are not available here; these generators stand in for them with the shapes,
sizes and value distributions the benchmark names:

  c1  SpMV  16384 x 16384, row lengths Poisson(16) clamped to [1, 64], values and x U[-1, 1)
  c2  SpMV  27-point stencil on a 160^3 grid (centre 26, neighbours -1), x U[-1, 1)
  c3  SpMV  4 194 304 rows, Zipf(2.0) row lengths rescaled to mean 32 and capped at 200 000,
            values and x N(0, 1), alpha 1.5, beta 0.5, y U[-1, 1)
  c4  SpMM  1 048 576 rows, Poisson(16) row lengths, values U[0, 1), B 1 048 576 x 128 U[-1, 1)
  c5  SpMM  8 388 608 rows, Zipf(2.1) row lengths rescaled to mean 20 and capped at 500 000,
            values 1/len(row), B 8 388 608 x 64 N(0, 1)

Every array comes from ``numpy.random.Generator(PCG64(seed))`` with one seed per
array.  Column indices are distinct and sorted inside every row.  ``rows`` can
be lowered to get a small case of the same distribution for tests.
"""
from __future__ import annotations

import numpy as np

FULL_ROWS = {"c1": 16384, "c2": 160 ** 3, "c3": 4194304, "c4": 1048576, "c5": 8388608}


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def unique_sorted_columns(lengths: np.ndarray, cols: int, seed: int):
    """CSR structure with ``lengths[i]`` distinct, sorted, uniformly drawn columns in row i."""
    lengths = np.minimum(lengths.astype(np.int64), cols)
    rows = lengths.size
    row_ptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(lengths, out=row_ptr[1:])
    nnz = int(row_ptr[-1])
    rng = _rng(seed)
    row_of = np.repeat(np.arange(rows, dtype=np.int64), lengths)
    key = row_of * cols + rng.integers(0, cols, nnz, dtype=np.int64)
    # Rows that hold a large share of all columns are drawn without replacement
    # one by one: redrawing collisions would take very long for them.  (None of
    # the full-size configurations has such a row; scaled-down cases do.)
    for r in np.flatnonzero(lengths > max(cols // 16, 1)):
        key[row_ptr[r]:row_ptr[r + 1]] = r * cols + rng.choice(cols, int(lengths[r]), replace=False)
    key.sort()
    # Redraw duplicates until every row holds distinct columns.  A redrawn
    # column is uniform over [0, cols), so the row stays a uniform sample.
    while True:
        dup = np.flatnonzero(key[1:] == key[:-1]) + 1
        if dup.size == 0:
            break
        key[dup] = row_of[dup] * cols + rng.integers(0, cols, dup.size, dtype=np.int64)
        key.sort()
    col_ind = (key - row_of * cols).astype(np.int32)
    return row_ptr.astype(np.int32), col_ind


def zipf_lengths(rows: int, exponent: float, mean: float, cap: int, seed: int):
    """Zipf(exponent) draws scaled by one factor s so that the clamped lengths average ``mean``.

    Returns (lengths, s); s is found by bisection to within 0.1 % of the mean.
    """
    raw = _rng(seed).zipf(exponent, rows).astype(np.float64)

    def lengths_for(s: float) -> np.ndarray:
        return np.clip(np.rint(s * raw), 1, cap)

    lo, hi = 1e-3, 1e3
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        m = lengths_for(mid).mean()
        if abs(m - mean) <= 1e-3 * mean:
            break
        if m < mean:
            lo = mid
        else:
            hi = mid
    return lengths_for(mid).astype(np.int64), float(mid)


def stencil27(grid: int):
    """27-point stencil on a grid^3 lattice: CSR with ascending columns, centre 26, neighbours -1."""
    g = grid
    m = g ** 3
    idx = np.arange(m, dtype=np.int64)
    x = idx % g
    y = (idx // g) % g
    z = idx // (g * g)
    offsets = [(dz, dy, dx) for dz in (-1, 0, 1) for dy in (-1, 0, 1) for dx in (-1, 0, 1)]
    masks = []
    count = np.zeros(m, dtype=np.int32)
    for dz, dy, dx in offsets:
        ok = ((z + dz >= 0) & (z + dz < g) & (y + dy >= 0) & (y + dy < g) & (x + dx >= 0) & (x + dx < g))
        masks.append(ok)
        count += ok
    row_ptr = np.zeros(m + 1, dtype=np.int64)
    np.cumsum(count, out=row_ptr[1:])
    nnz = int(row_ptr[-1])
    col_ind = np.empty(nnz, dtype=np.int32)
    values = np.empty(nnz, dtype=np.float32)
    cursor = row_ptr[:-1].copy()
    for (dz, dy, dx), ok in zip(offsets, masks):
        rows_ok = np.flatnonzero(ok)
        pos = cursor[rows_ok]
        col_ind[pos] = (rows_ok + (dz * g + dy) * g + dx).astype(np.int32)
        values[pos] = 26.0 if (dz, dy, dx) == (0, 0, 0) else -1.0
        cursor[rows_ok] += 1
    return row_ptr.astype(np.int32), col_ind, values


def make(name: str, rows: "int | None" = None, seed: int = 2026) -> dict:
    """Inputs of configuration ``name`` ('c1'..'c5'); ``rows`` overrides the row count (c2: rounded to a cube)."""
    name = name.lower()
    m = FULL_ROWS[name] if rows is None else int(rows)
    out = {"name": name, "index_base": 0}
    if name == "c1":
        lengths = np.clip(_rng(seed).poisson(16.0, m), 1, 64)
        rp, ci = unique_sorted_columns(lengths, m, seed + 1)
        out.update(kind="spmv", rows=m, cols=m, row_ptr=rp, col_ind=ci,
                   values=_rng(seed + 2).uniform(-1.0, 1.0, ci.size).astype(np.float32),
                   x=_rng(seed + 3).uniform(-1.0, 1.0, m).astype(np.float32),
                   y=np.zeros(m, dtype=np.float32), alpha=1.0, beta=0.0)
    elif name == "c2":
        grid = int(round(m ** (1.0 / 3.0)))
        rp, ci, va = stencil27(grid)
        m = grid ** 3
        out.update(kind="spmv", rows=m, cols=m, row_ptr=rp, col_ind=ci, values=va, grid=grid,
                   x=_rng(seed + 3).uniform(-1.0, 1.0, m).astype(np.float32),
                   y=np.zeros(m, dtype=np.float32), alpha=1.0, beta=0.0)
    elif name == "c3":
        cap = min(200000, max(m // 2, 1))
        lengths, s = zipf_lengths(m, 2.0, 32.0, cap, seed)
        rp, ci = unique_sorted_columns(lengths, m, seed + 1)
        out.update(kind="spmv", rows=m, cols=m, row_ptr=rp, col_ind=ci, zipf_scale=s,
                   values=_rng(seed + 2).standard_normal(ci.size, dtype=np.float32),
                   x=_rng(seed + 3).standard_normal(m, dtype=np.float32),
                   y=_rng(seed + 4).uniform(-1.0, 1.0, m).astype(np.float32), alpha=1.5, beta=0.5)
    elif name == "c4":
        lengths = _rng(seed).poisson(16.0, m)
        rp, ci = unique_sorted_columns(lengths, m, seed + 1)
        n = 128
        out.update(kind="spmm", rows=m, cols=m, n=n, row_ptr=rp, col_ind=ci,
                   values=_rng(seed + 2).uniform(0.0, 1.0, ci.size).astype(np.float32),
                   b=_rng(seed + 3).uniform(-1.0, 1.0, (m, n)).astype(np.float32),
                   c=np.zeros((m, n), dtype=np.float32), alpha=1.0, beta=0.0)
    elif name == "c5":
        cap = min(500000, max(m // 2, 1))
        lengths, s = zipf_lengths(m, 2.1, 20.0, cap, seed)
        rp, ci = unique_sorted_columns(lengths, m, seed + 1)
        n = 64
        deg = np.diff(rp).astype(np.float32)
        out.update(kind="spmm", rows=m, cols=m, n=n, row_ptr=rp, col_ind=ci, zipf_scale=s,
                   values=np.repeat((1.0 / np.maximum(deg, 1.0)).astype(np.float32), np.diff(rp)),
                   b=_rng(seed + 3).standard_normal((m, n), dtype=np.float32),
                   c=np.zeros((m, n), dtype=np.float32), alpha=1.0, beta=0.0)
    else:
        raise ValueError(name)
    out["nnz"] = int(out["col_ind"].size)
    return out


def algorithmic_bytes(cfg: dict) -> int:
    """Bytes that have to move at least once: the CSR arrays, x or B, and y or C (read too when beta != 0)."""
    m, nnz = cfg["rows"], cfg["nnz"]
    out_passes = 2 if cfg["beta"] != 0.0 else 1
    if cfg["kind"] == "spmv":
        return nnz * 8 + (m + 1) * 4 + cfg["cols"] * 4 + m * 4 * out_passes
    n = cfg["n"]
    return nnz * 8 + (m + 1) * 4 + cfg["cols"] * n * 4 + m * n * 4 * out_passes


def flops(cfg: dict) -> int:
    return 2 * cfg["nnz"] * (cfg["n"] if cfg["kind"] == "spmm" else 1)
