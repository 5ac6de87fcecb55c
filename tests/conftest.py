"""Shared test set-up.

``-m "not gpu"`` covers the oracle against the reference's golden vectors, the host
logic of the C API (status codes are decided before anything is launched) and the
exported symbols; ``-m gpu`` holds the parity tests proper, all through the C ABI.
"""
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(GOLDEN_DIR, "reference_kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def goldens():
    data = np.load(os.path.join(GOLDEN_DIR, "reference_goldens.npz"))
    names = sorted({k.split(".")[0] for k in data.files})
    out = {}
    for n in names:
        rows, cols, ncols, base = (int(v) for v in data[n + ".meta"])
        alpha, beta = (float(v) for v in data[n + ".scalars"])
        out[n] = dict(rows=rows, cols=cols, n=ncols, base=base, alpha=alpha, beta=beta,
                      row_ptr=data[n + ".row_ptr"], col_ind=data[n + ".col_ind"], values=data[n + ".values"],
                      b=data[n + ".b"], c0=data[n + ".c0"], truth=data[n + ".truth"])
    return out


@pytest.fixture(scope="session")
def lib():
    from ops_sparse_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        _lib.build()
    return _lib.lib()
