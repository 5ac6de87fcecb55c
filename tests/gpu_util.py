"""Helpers for the GPU parity tests: everything goes through the C ABI (ops_sparse_b200.api)."""
import numpy as np
import torch

from oracle import oracle as O
from ops_sparse_b200 import _lib as L
from ops_sparse_b200 import api

DEV = "cuda:0"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a if dtype is None else a.astype(dtype)))
    return t.to(DEV)


class SpmvCase:
    """Device copies + descriptors of one SpMV problem."""

    def __init__(self, row_ptr, col_ind, values, x, y, cols=None, base=0, alg=L.SPMV_ALG_DEFAULT, handle=None):
        self.rows = len(row_ptr) - 1
        self.cols = len(x) if cols is None else cols
        self.nnz = len(col_ind)
        self.d_rp = dev(np.asarray(row_ptr), np.int32)
        self.d_ci = dev(np.asarray(col_ind), np.int32) if self.nnz else None
        self.d_va = dev(np.asarray(values), np.float32) if self.nnz else None
        self.d_x = dev(np.asarray(x), np.float32)
        self.d_y = dev(np.asarray(y), np.float32)
        self.handle = handle or api.Handle()
        self.mat = api.CsrMatrix(self.rows, self.cols, self.d_rp, self.d_ci, self.d_va, base, nnz=self.nnz)
        self.vx = api.DnVec(self.d_x)
        self.vy = api.DnVec(self.d_y)
        self.op = api.SpMV(self.handle, self.mat, self.vx, self.vy, alg=alg)

    def run(self, alpha=1.0, beta=0.0, preprocess=True):
        if preprocess:
            self.op.preprocess(alpha, beta)
        self.op(alpha, beta)
        torch.cuda.synchronize()
        return self.d_y.cpu().numpy()


class SpmmCase:
    """Device copies + descriptors of one SpMM problem; b and c are storage arrays (any layout)."""

    def __init__(self, row_ptr, col_ind, values, k, n, b, ldb, c, ldc, base=0, order_b=L.ORDER_ROW,
                 order_c=L.ORDER_ROW, op_b=L.OP_N, alg=L.SPMM_ALG_DEFAULT, handle=None):
        self.m = len(row_ptr) - 1
        self.nnz = len(col_ind)
        self.d_rp = dev(np.asarray(row_ptr), np.int32)
        self.d_ci = dev(np.asarray(col_ind), np.int32) if self.nnz else None
        self.d_va = dev(np.asarray(values), np.float32) if self.nnz else None
        self.d_b = dev(np.asarray(b), np.float32)
        self.d_c = dev(np.asarray(c), np.float32)
        self.handle = handle or api.Handle()
        self.mat = api.CsrMatrix(self.m, k, self.d_rp, self.d_ci, self.d_va, base, nnz=self.nnz)
        b_rows, b_cols = (k, n) if op_b == L.OP_N else (n, k)
        self.mb = api.DnMat(b_rows, b_cols, ldb, self.d_b, order_b)
        self.mc = api.DnMat(self.m, n, ldc, self.d_c, order_c)
        self.op = api.SpMM(self.handle, self.mat, self.mb, self.mc, alg=alg, op_b=op_b)

    def run(self, alpha=1.0, beta=0.0, preprocess=True):
        if preprocess:
            self.op.preprocess(alpha, beta)
        self.op(alpha, beta)
        torch.cuda.synchronize()
        return self.d_c.cpu().numpy()


def random_csr(rng, lengths, cols):
    lengths = np.minimum(np.asarray(lengths, dtype=np.int64), cols)
    rp = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols, int(l), replace=False)) for l in lengths] or [[]]).astype(np.int32)
    return rp, ci


# ---- narrow storage types: "f32", "f16", "bf16", "i8", "i32" ----

def to_device(a, kind):
    """A numpy array of exactly representable numbers as a device tensor of the named element type."""
    if kind == "bf16":
        bits = O.f32_to_bf16_bits(np.asarray(a, np.float32)).view(np.int16)
        return dev(bits).view(torch.bfloat16)
    np_type = {"f32": np.float32, "f16": np.float16, "i8": np.int8, "i32": np.int32}[kind]
    return dev(np.asarray(a).astype(np_type))


def bits_of(t):
    """Result tensor -> numpy: 16-bit types as their bit patterns, the others as they are."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def quantize(a, kind):
    """Round test data to the storage type and return it as fp32 (every narrow value is an fp32 number)."""
    a = np.asarray(a, np.float32)
    if kind == "f16":
        return a.astype(np.float16).astype(np.float32)
    if kind == "bf16":
        return O.bf16_bits_to_f32(O.f32_to_bf16_bits(a))
    if kind == "i8":
        return np.clip(np.rint(a), -127, 127).astype(np.float32)
    return a


def expected_bits(truth, kind):
    if kind == "f16":
        return O.f64_to_f16(truth).view(np.uint16)
    if kind == "bf16":
        return O.f64_to_bf16_bits(truth)
    return truth.astype(np.float32)
