"""Generates the golden fixtures in this directory from the reference's own code.

Run where the reference checkout is available (it builds oracle/_ref/libref_host.so
from the reference's sources, see oracle/Makefile):

    python tests/golden/make_golden.py

Inputs come from the reference's test generator (SparseFillGenerator,
test/frame/fill.h:55-195) and outputs from the reference's fp64 golden
(SpmmGolden, test/spmm_op/spmm_op_golden.h:177-205; one dense column makes it
the SpMV golden) and from its SpMM row reorder (SpmmCsrMat::DoPreProcess,
sparse/spmm/arch35/host/spmm_csr_mat.cpp:180-210).  The fixtures are small on
purpose; the tests replay them against the oracle (CPU) and the CUDA path (GPU).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402

# name, rows, cols, sparsity, empty-row probability, n (1 = SpMV), alpha, beta, index base, seed
CASES = [
    ("spmv_512x1024_s90", 512, 1024, 0.90, 0.0, 1, 1.0, 0.0, 0, 11),
    ("spmv_512x1024_dense", 64, 256, 0.0, 0.0, 1, 1.0, 0.0, 0, 12),
    ("spmv_10x1024_s999", 10, 1024, 0.999, 0.0, 1, 1.0, 0.0, 0, 13),
    ("spmv_1x1024", 1, 1024, 0.9, 0.0, 1, 2.0, 0.0, 0, 14),
    ("spmv_256x2048_ab", 256, 2048, 0.95, 0.0, 1, 1.5, 0.2, 0, 15),
    ("spmv_emptyrows", 300, 700, 0.97, 0.5, 1, -1.0, 1.0, 0, 16),
    ("spmv_base1", 200, 333, 0.9, 0.1, 1, 0.5, 0.5, 1, 17),
    ("spmv_longrow", 128, 20480, 0.999, 0.0, 1, 1.0, 0.0, 0, 18),
    ("spmm_37x23x11", 37, 23, 0.8, 0.0, 11, 1.0, 0.0, 0, 42),
    ("spmm_41x29x13_ab", 41, 29, 0.83, 0.0, 13, -0.75, 0.5, 0, 50),
    ("spmm_256x256x64", 256, 256, 0.95, 0.0, 64, 1.0, 0.5, 0, 45),
    ("spmm_300x500x128", 300, 500, 0.97, 0.2, 128, 1.0, 0.0, 0, 46),
    ("spmm_base1_17x11x5", 17, 11, 0.75, 0.0, 5, 0.5, -0.25, 1, 53),
]


def main():
    O.build(ref=True)
    assert O.have_ref(), "the reference checkout is needed to generate fixtures"
    out = {}
    for name, rows, cols, sparsity, empty, n, alpha, beta, base, seed in CASES:
        # scalars are fp32 in the API; the golden widens them to double as the reference's tests do
        alpha, beta = float(np.float32(alpha)), float(np.float32(beta))
        rp, ci, va = O.ref_fill_csr(rows, cols, sparsity, seed, empty_row_prob=empty)
        if name == "spmv_longrow":
            # one row with 20 000 entries among sparse ones, as the reference's long-tail cases
            # (test/spmv/arch22/spmv_test.cpp:926-963)
            extra = np.sort(np.random.Generator(np.random.PCG64(seed)).choice(cols, 20000, replace=False))
            lens = np.diff(rp)
            row = 77
            s, e = rp[row], rp[row + 1]
            ci = np.concatenate([ci[:s], extra.astype(np.int32), ci[e:]])
            va = np.concatenate([va[:s], O.ref_fill_dense(20000, seed + 5), va[e:]])
            lens[row] = 20000
            rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        b = O.ref_fill_dense(cols * n, seed + 1).reshape(cols, n)
        c0 = O.ref_fill_dense(rows * n, seed + 2).reshape(rows, n)
        truth = O.ref_spmm_golden_f64(rp + base, ci + base, va, b, c0, rows, n, cols, alpha, beta, index_base=base)
        out[name + ".row_ptr"] = (rp + base).astype(np.int32)
        out[name + ".col_ind"] = (ci + base).astype(np.int32)
        out[name + ".values"] = va
        out[name + ".b"] = b
        out[name + ".c0"] = c0
        out[name + ".truth"] = truth
        out[name + ".meta"] = np.array([rows, cols, n, base], dtype=np.int64)
        out[name + ".scalars"] = np.array([alpha, beta], dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_goldens.npz"), **out)

    # Row reorder / bin edges of the reference's SpMM preprocessing for several row-length shapes.
    reorder = {}
    rng = np.random.Generator(np.random.PCG64(7))
    shapes = {
        "uniform16": np.full(1000, 16),
        "near_uniform": 16 + (np.arange(777) % 2),
        "poisson16": rng.poisson(16.0, 1500),
        "zipf": np.clip(rng.zipf(2.0, 1200), 1, 600),
        "with_empty": np.where(rng.random(900) < 0.4, 0, rng.integers(1, 40, 900)),
        "tiny": np.array([3, 0, 7]),
    }
    for name, lens in shapes.items():
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        for bins in (24, 148):
            r, e, ident, uni = O.ref_spmm_row_reorder(rp, int(max(lens.max(), 1)) + 700, bins)
            reorder[f"{name}.{bins}.row_ptr"] = rp
            reorder[f"{name}.{bins}.reorder"] = r
            reorder[f"{name}.{bins}.edges"] = e
            reorder[f"{name}.{bins}.flags"] = np.array([int(ident), uni], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "reference_row_reorder.npz"), **reorder)

    sizes = {str(r): O.ref_spmv_workspace_bytes_real(r, r) for r in (0, 1, 2, 15, 16, 17, 1000, 4096000)}
    np.savez(os.path.join(HERE, "reference_spmv_workspace_bytes.npz"),
             rows=np.array([int(k) for k in sizes], dtype=np.int64),
             bytes=np.array(list(sizes.values()), dtype=np.int64))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
