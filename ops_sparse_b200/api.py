"""Python face of the aclsparse C API (``libops_sparse.so``) for CUDA tensors.

Thin wrappers that keep the reference's call sequence visible — create a
handle, describe the operands, ``GetBufferSize`` -> ``Preprocess`` -> execute —
so that tests written against this module read like the reference's own
(test/spmv/arch35/spmv_test.cpp:169-221, test/spmm/arch35/spmm_test.cpp).
PyTorch only provides device memory and streams here; every operator call
goes through the C ABI.  Failing calls raise ``AclsparseError`` with the
status the C function returned.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_size_t, c_void_p

import torch

from . import _lib as L


class AclsparseError(RuntimeError):
    def __init__(self, fn: str, status: int):
        super().__init__(f"{fn} returned {L.STATUS_NAMES.get(status, status)} ({status})")
        self.status = status


def check(fn: str, status: int) -> None:
    if status != L.SUCCESS:
        raise AclsparseError(fn, status)


def _ptr(t) -> c_void_p:
    if t is None:
        return c_void_p(None)
    if isinstance(t, int):
        return c_void_p(t)
    return c_void_p(t.data_ptr())


class Handle:
    """aclsparseHandle_t bound to a CUDA stream (the current torch stream by default)."""

    def __init__(self, stream: "torch.cuda.Stream | None" = None, set_stream: bool = True):
        self._h = c_void_p(None)
        check("aclsparseCreate", L.lib().aclsparseCreate(byref(self._h)))
        if set_stream:
            s = stream if stream is not None else torch.cuda.current_stream()
            self.set_stream(s.cuda_stream)

    @property
    def raw(self) -> c_void_p:
        return self._h

    def set_stream(self, cuda_stream: int) -> None:
        # SpMV insists on a non-NULL stream, as the reference does.  PyTorch's default stream is the
        # NULL stream; cudaStreamLegacy (0x1) is the explicit, non-NULL handle of that same stream.
        check("aclsparseSetStream", L.lib().aclsparseSetStream(self._h, c_void_p(cuda_stream or 0x1)))

    def set_pointer_mode(self, mode: int) -> None:
        check("aclsparseSetPointerMode", L.lib().aclsparseSetPointerMode(self._h, mode))

    def close(self) -> None:
        if self._h:
            L.lib().aclsparseDestroy(self._h)
            self._h = c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def acl_type(tensor) -> int:
    """aclDataType of a tensor's elements (the value types the library's dtype tables name)."""
    table = {torch.float32: L.ACL_FLOAT, torch.float16: L.ACL_FLOAT16, torch.bfloat16: L.ACL_BF16,
             torch.int8: L.ACL_INT8, torch.int32: L.ACL_INT32}
    if tensor is None:  # unbound storage (an empty matrix, or values bound later): fp32 unless said otherwise
        return L.ACL_FLOAT
    if tensor.dtype not in table:
        raise TypeError(f"no aclDataType for {tensor.dtype}")
    return table[tensor.dtype]


class CsrMatrix:
    """CSR descriptor over three CUDA tensors (int32 row offsets / column indices; fp32, fp16, bf16 or int8 values)."""

    def __init__(self, rows: int, cols: int, row_offsets, col_indices, values, index_base: int = L.BASE_ZERO,
                 nnz: "int | None" = None):
        self.rows, self.cols = rows, cols
        self.nnz = int(values.numel()) if nnz is None else nnz
        self.row_offsets, self.col_indices, self.values = row_offsets, col_indices, values
        self.index_base = index_base
        self._d = c_void_p(None)
        check("aclsparseCreateCsr", L.lib().aclsparseCreateCsr(
            byref(self._d), rows, cols, self.nnz, _ptr(row_offsets), _ptr(col_indices), _ptr(values), L.INDEX_32I,
            L.INDEX_32I, index_base, acl_type(values)))

    @property
    def raw(self) -> c_void_p:
        return self._d

    def close(self) -> None:
        if self._d:
            L.lib().aclsparseDestroySpMat(self._d)
            self._d = c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DnVec:
    def __init__(self, values, size: "int | None" = None):
        self.values = values
        self.size = int(values.numel()) if size is None else size
        self._d = c_void_p(None)
        check("aclsparseCreateDnVec", L.lib().aclsparseCreateDnVec(byref(self._d), self.size, _ptr(values),
                                                                  acl_type(values)))

    @property
    def raw(self) -> c_void_p:
        return self._d

    def set_values(self, values) -> None:
        self.values = values
        check("aclsparseDnVecSetValues", L.lib().aclsparseDnVecSetValues(self._d, _ptr(values)))

    def set_mirrors(self, pointers) -> None:
        """Device addresses (ints) of buffers that receive every element SpMV writes to this vector."""
        arr = (c_void_p * max(len(pointers), 1))(*[int(p) for p in pointers])
        check("aclsparseB200DnVecSetMirrors", L.lib().aclsparseB200DnVecSetMirrors(self._d, len(pointers), arr))

    def set_multicast_mirror(self, pointer: int) -> None:
        """NVLink multicast address that receives (on every GPU bound to it) each element SpMV writes."""
        check("aclsparseB200DnVecSetMulticastMirror",
              L.lib().aclsparseB200DnVecSetMulticastMirror(self._d, c_void_p(int(pointer))))

    def set_closing_barrier(self, local_state: int, peer_states, world: int, rank: int, spin_limit: int = 0) -> None:
        """Ends every SpMV into this vector with the node barrier (aclsparseB200DnVecSetClosingBarrier);
        ``world <= 1`` removes it.  ``peer_states``: a ctypes array of ``world`` device addresses."""
        check("aclsparseB200DnVecSetClosingBarrier", L.lib().aclsparseB200DnVecSetClosingBarrier(
            self._d, c_void_p(int(local_state)), peer_states, world, rank, spin_limit))

    def close(self) -> None:
        if self._d:
            L.lib().aclsparseDestroyDnVec(self._d)
            self._d = c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DnMat:
    def __init__(self, rows: int, cols: int, ld: int, values, order: int = L.ORDER_ROW):
        self.rows, self.cols, self.ld, self.values, self.order = rows, cols, ld, values, order
        self._d = c_void_p(None)
        check("aclsparseCreateDnMat", L.lib().aclsparseCreateDnMat(byref(self._d), rows, cols, ld, _ptr(values),
                                                                  acl_type(values), order))

    @property
    def raw(self) -> c_void_p:
        return self._d

    def set_values(self, values) -> None:
        self.values = values
        check("aclsparseDnMatSetValues", L.lib().aclsparseDnMatSetValues(self._d, _ptr(values)))

    def set_mirrors(self, pointers) -> None:
        """Device addresses (ints) of buffers that receive every element SpMM writes to this matrix."""
        arr = (c_void_p * max(len(pointers), 1))(*[int(p) for p in pointers])
        check("aclsparseB200DnMatSetMirrors", L.lib().aclsparseB200DnMatSetMirrors(self._d, len(pointers), arr))

    def set_closing_barrier(self, local_state: int, peer_states, world: int, rank: int, spin_limit: int = 0) -> None:
        """Ends every SpMM into this matrix with the node barrier (aclsparseB200DnMatSetClosingBarrier);
        ``world <= 1`` removes it.  ``peer_states``: a ctypes array of ``world`` device addresses."""
        check("aclsparseB200DnMatSetClosingBarrier", L.lib().aclsparseB200DnMatSetClosingBarrier(
            self._d, c_void_p(int(local_state)), peer_states, world, rank, spin_limit))

    def set_multicast_mirror(self, pointer: int) -> None:
        """NVLink multicast address that receives (on every GPU bound to it) each element SpMM writes."""
        check("aclsparseB200DnMatSetMulticastMirror",
              L.lib().aclsparseB200DnMatSetMulticastMirror(self._d, c_void_p(int(pointer))))

    def close(self) -> None:
        if self._d:
            L.lib().aclsparseDestroyDnMat(self._d)
            self._d = c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _scalars(alpha, beta, integer: bool = False):
    """Host scalars as C floats (int32 for the integer compute type), or device tensors passed through for
    DEVICE pointer mode."""
    if isinstance(alpha, torch.Tensor):
        return _ptr(alpha), _ptr(beta), None
    a, b = (ctypes.c_int32(alpha), ctypes.c_int32(beta)) if integer else (c_float(alpha), c_float(beta))
    return ctypes.cast(byref(a), c_void_p), ctypes.cast(byref(b), c_void_p), (a, b)


class SpMV:
    """y = alpha * A * x + beta * y with the reference's three-phase call sequence."""

    def __init__(self, handle: Handle, mat: CsrMatrix, x: DnVec, y: DnVec, alg: int = L.SPMV_ALG_DEFAULT,
                 op: int = L.OP_N):
        self.handle, self.mat, self.x, self.y, self.alg, self.op = handle, mat, x, y, alg, op
        self.buffer = None
        # int8 data with an int32 result computes in int32 (integer alpha / beta, saturating); all else in fp32.
        self.integer = y.values.dtype == torch.int32
        self.compute_type = L.ACL_INT32 if self.integer else L.ACL_FLOAT

    def buffer_size(self, alpha=1.0, beta=0.0) -> int:
        pa, pb, _keep = _scalars(alpha, beta, self.integer)
        size = c_size_t(0)
        check("aclsparseSpMVGetBufferSize", L.lib().aclsparseSpMVGetBufferSize(
            self.handle.raw, self.op, pa, self.mat.raw, self.x.raw, pb, self.y.raw, self.compute_type, self.alg,
            byref(size)))
        return int(size.value)

    def allocate(self, alpha=1.0, beta=0.0):
        n = self.buffer_size(alpha, beta)
        self.buffer = torch.empty(max(n, 64), dtype=torch.uint8, device=self.y.values.device)
        return self.buffer

    def preprocess(self, alpha=1.0, beta=0.0) -> None:
        if self.buffer is None:
            self.allocate(alpha, beta)
        pa, pb, _keep = _scalars(alpha, beta, self.integer)
        check("aclsparseSpMVPreprocess", L.lib().aclsparseSpMVPreprocess(
            self.handle.raw, self.op, pa, self.mat.raw, self.x.raw, pb, self.y.raw, self.compute_type, self.alg,
            _ptr(self.buffer)))

    def __call__(self, alpha=1.0, beta=0.0) -> None:
        if self.buffer is None:
            self.allocate(alpha, beta)
        pa, pb, _keep = _scalars(alpha, beta, self.integer)
        check("aclsparseSpMV", L.lib().aclsparseSpMV(
            self.handle.raw, self.op, pa, self.mat.raw, self.x.raw, pb, self.y.raw, self.compute_type, self.alg,
            _ptr(self.buffer)))


class SpMM:
    """C = alpha * A * op(B) + beta * C with the reference's three-phase call sequence."""

    def __init__(self, handle: Handle, mat: CsrMatrix, b: DnMat, c: DnMat, alg: int = L.SPMM_ALG_DEFAULT,
                 op_a: int = L.OP_N, op_b: int = L.OP_N):
        self.handle, self.mat, self.b, self.c, self.alg, self.op_a, self.op_b = handle, mat, b, c, alg, op_a, op_b
        self.buffer = None
        # int8 data with an int32 result computes in int32 (integer alpha / beta, saturating); all else in fp32.
        self.integer = c.values.dtype == torch.int32
        self.compute_type = L.ACL_INT32 if self.integer else L.ACL_FLOAT

    def buffer_size(self, alpha=1.0, beta=0.0) -> int:
        pa, pb, _keep = _scalars(alpha, beta, self.integer)
        size = c_size_t(0)
        check("aclsparseSpMMGetBufferSize", L.lib().aclsparseSpMMGetBufferSize(
            self.handle.raw, self.op_a, self.op_b, pa, self.mat.raw, self.b.raw, pb, self.c.raw, self.compute_type,
            self.alg, byref(size)))
        return int(size.value)

    def allocate(self, alpha=1.0, beta=0.0):
        n = self.buffer_size(alpha, beta)
        self.buffer = torch.empty(max(n, 64), dtype=torch.uint8, device=self.c.values.device)
        return self.buffer

    def preprocess(self, alpha=1.0, beta=0.0) -> None:
        if self.buffer is None:
            self.allocate(alpha, beta)
        pa, pb, _keep = _scalars(alpha, beta, self.integer)
        check("aclsparseSpMMPreprocess", L.lib().aclsparseSpMMPreprocess(
            self.handle.raw, self.op_a, self.op_b, pa, self.mat.raw, self.b.raw, pb, self.c.raw, self.compute_type,
            self.alg, _ptr(self.buffer)))

    def __call__(self, alpha=1.0, beta=0.0) -> None:
        if self.buffer is None:
            self.allocate(alpha, beta)
        pa, pb, _keep = _scalars(alpha, beta, self.integer)
        check("aclsparseSpMM", L.lib().aclsparseSpMM(
            self.handle.raw, self.op_a, self.op_b, pa, self.mat.raw, self.b.raw, pb, self.c.raw, self.compute_type,
            self.alg, _ptr(self.buffer)))


def kernel_launches() -> int:
    """Kernels the library has launched in this process so far (aclsp_b200_kernel_launches)."""
    return int(L.lib().aclsp_b200_kernel_launches())


def row_block_bounds(handle: Handle, mat: CsrMatrix, parts: int) -> torch.Tensor:
    """Device tensor of parts+1 row boundaries that balance the non-zeros of ``mat`` over ``parts`` devices."""
    out = torch.empty(parts + 1, dtype=torch.int32, device=mat.row_offsets.device)
    check("aclsparseB200RowBlockBounds", L.lib().aclsparseB200RowBlockBounds(handle.raw, mat.raw, parts, _ptr(out)))
    return out
