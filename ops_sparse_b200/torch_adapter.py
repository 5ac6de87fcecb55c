"""PyTorch adapter: ``torch.mv`` / ``torch.addmm`` semantics on CSR CUDA tensors, served by this library.

Counterpart of the reference's torch extension (sparse/spmv/torch_extension/csrc/spmv.cpp:255-330,
sparse/spmv/torch_extension/spmv.py:44-47 and the SpMM twin under sparse/spmm/torch_extension), which routes
``aten::mv`` for CSR tensors of its device to ``aclsparseSpMV`` and exposes two test entries that take the CSR
arrays directly.  Same entry names and argument meaning here:

    mv(mat, vec)                                          y = A @ vec        (alpha = 1, beta = 0)
    addmm(input, mat, dense, beta=1, alpha=1)             beta * input + alpha * A @ dense
    spmv_csr(row_ptr, col_ind, values, x, y, alpha, beta, base=0, trans="N", cols=None)   in place on y
    spmv_workspace(...)                                   bytes aclsparseSpMVGetBufferSize asks for

Argument errors are raised as ``ValueError`` / ``TypeError`` before anything is launched, in the order the reference
checks them; the product itself runs through the C API on the current CUDA stream.  Like the reference's adapter,
every call builds its descriptors and preprocesses (the plan build is tens of microseconds on the device and needs
no host round trip).  ``install()`` additionally registers ``mv`` as the ``aten::mv`` kernel of CSR CUDA tensors.
"""
from __future__ import annotations

import torch

from . import _lib as L

INT32_MAX = 2 ** 31 - 1
_OPS = {"N": L.OP_N, "T": L.OP_T, "H": L.OP_H}


def _check_matrix_and_operand(mat: torch.Tensor, other: torch.Tensor, other_name: str, other_dim: int) -> None:
    """The reference's CheckMvInputs (spmv.cpp:261-287), CUDA in place of its device type."""
    if not isinstance(mat, torch.Tensor):
        raise TypeError("mat must be a defined tensor")
    if mat.layout != torch.sparse_csr:
        raise ValueError(f"mat must use the sparse CSR layout, but got {mat.layout}")
    if mat.device.type != "cuda":
        raise ValueError(f"mat must be on a CUDA device, but got {mat.device}")
    if mat.dim() != 2:
        raise ValueError(f"mat must be a 2-D sparse matrix, but got {mat.dim()} dimensions")
    if not isinstance(other, torch.Tensor):
        raise TypeError(f"{other_name} must be a defined tensor")
    if other.layout != torch.strided:
        raise ValueError(f"{other_name} must be a dense tensor, but got layout {other.layout}")
    if other.device.type != "cuda":
        raise ValueError(f"{other_name} must be on a CUDA device, but got {other.device}")
    if other.dim() != other_dim:
        raise ValueError(f"{other_name} must be a {other_dim}-D dense tensor, but got {other.dim()} dimensions")
    if mat.device != other.device:
        raise ValueError(f"mat and {other_name} must be on the same device, but got {mat.device} and {other.device}")
    if mat.dtype != other.dtype:
        raise TypeError(f"mat and {other_name} must have the same dtype, but got {mat.dtype} and {other.dtype}")
    if mat.dtype != torch.float32:
        raise TypeError(f"this build computes in float32 only, but got {mat.dtype}")
    if mat.size(1) != other.size(0):
        raise ValueError(f"size mismatch: mat is {tuple(mat.shape)}, {other_name} has {other.size(0)} rows")
    if mat.size(0) > INT32_MAX or mat.size(1) > INT32_MAX or mat._nnz() > INT32_MAX:
        raise ValueError("rows, columns and non-zeros must fit int32")


def _csr_arrays(mat: torch.Tensor):
    """int32 row offsets / column indices (PyTorch keeps int64 by default) and contiguous values."""
    crow = mat.crow_indices()
    col = mat.col_indices()
    if crow.dtype != torch.int32:
        crow = crow.to(torch.int32)
    if col.dtype != torch.int32:
        col = col.to(torch.int32)
    return crow.contiguous(), col.contiguous(), mat.values().contiguous()


def _handle():
    from . import api
    return api.Handle()  # bound to the current torch stream


def mv(mat: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
    """``A @ vec`` for a CSR sparse matrix and a dense vector on the GPU (aten::mv semantics)."""
    _check_matrix_and_operand(mat, vec, "vec", 1)
    from . import api
    rows, cols = mat.shape
    crow, col, val = _csr_arrays(mat)
    y = torch.empty(rows, dtype=torch.float32, device=mat.device)
    if rows == 0:
        return y
    if mat._nnz() == 0 or cols == 0:
        return y.zero_()
    with torch.cuda.device(mat.device):
        a = api.CsrMatrix(rows, cols, crow, col, val, L.BASE_ZERO, nnz=int(val.numel()))
        op = api.SpMV(_handle(), a, api.DnVec(vec.contiguous()), api.DnVec(y))
        op.preprocess(1.0, 0.0)
        op(1.0, 0.0)
    return y


def addmm(input: torch.Tensor, mat: torch.Tensor, dense: torch.Tensor, *, beta: float = 1.0,
          alpha: float = 1.0) -> torch.Tensor:
    """``beta * input + alpha * (A @ dense)`` for a CSR ``A`` and row-major dense operands (aten::addmm semantics)."""
    _check_matrix_and_operand(mat, dense, "dense", 2)
    from . import api
    rows, cols = mat.shape
    n = dense.size(1)
    if not isinstance(input, torch.Tensor) or input.device != mat.device or input.dtype != torch.float32:
        raise TypeError("input must be a float32 tensor on the device of mat")
    c = input.expand(rows, n).contiguous().clone() if beta != 0.0 else torch.empty(rows, n, dtype=torch.float32,
                                                                                   device=mat.device)
    if rows == 0 or n == 0:
        return c
    if mat._nnz() == 0 or cols == 0:
        return c.mul_(beta) if beta != 0.0 else c.zero_()
    crow, col, val = _csr_arrays(mat)
    b = dense.contiguous()
    with torch.cuda.device(mat.device):
        a = api.CsrMatrix(rows, cols, crow, col, val, L.BASE_ZERO, nnz=int(val.numel()))
        op = api.SpMM(_handle(), a, api.DnMat(cols, n, n, b), api.DnMat(rows, n, n, c))
        op.preprocess(alpha, beta)
        op(alpha, beta)
    return c


def mm(mat: torch.Tensor, dense: torch.Tensor) -> torch.Tensor:
    """``A @ dense``."""
    _check_matrix_and_operand(mat, dense, "dense", 2)
    zero = torch.empty(0, dtype=torch.float32, device=mat.device)
    return addmm(zero, mat, dense, beta=0.0, alpha=1.0)


def _check_arrays(row_ptr, col_ind, values, x, y, base, trans, cols):
    """The reference's CheckSpmvNpuInputs (spmv.cpp:336-377)."""
    tensors = dict(row_ptr=row_ptr, col_ind=col_ind, values=values, x=x, y=y)
    for name, t in tensors.items():
        if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
            raise ValueError(f"{name} must be a CUDA tensor")
    if len({t.device for t in tensors.values()}) != 1:
        raise ValueError("row_ptr, col_ind, values, x and y must be on the same device")
    if row_ptr.dtype != torch.int32 or col_ind.dtype != torch.int32:
        raise TypeError("row_ptr and col_ind must be int32")
    if col_ind.numel() != values.numel():
        raise ValueError(f"col_ind and values length mismatch: {col_ind.numel()} vs {values.numel()}")
    if x.dtype != values.dtype:
        raise TypeError(f"x and values must have the same dtype, but got {x.dtype} and {values.dtype}")
    if base not in (0, 1):
        raise ValueError(f"base must be 0 or 1, but got {base}")
    if trans not in _OPS:
        raise ValueError(f"trans must be N, T or H, but got {trans}")
    if x.dim() != 1 or y.dim() != 1:
        raise ValueError("x and y must be one-dimensional")
    if row_ptr.numel() < 1:
        raise ValueError("row_ptr must not be empty")
    rows = row_ptr.numel() - 1
    if max(rows, x.numel(), y.numel(), values.numel()) > INT32_MAX:
        raise ValueError("sizes must fit int32")
    if values.dtype != torch.float32 or y.dtype != torch.float32:
        raise TypeError("this build computes in float32 only")
    is_trans = trans != "N"
    cols = (y.numel() if is_trans else x.numel()) if cols is None else cols
    x_size, y_size = (rows, cols) if is_trans else (cols, rows)
    if x.size(0) < x_size:
        raise ValueError(f"x is too small for the requested op: need {x_size}, got {x.size(0)}")
    if y.size(0) < y_size:
        raise ValueError(f"y is too small for the requested op: need {y_size}, got {y.size(0)}")
    return rows, cols, x_size, y_size


def _spmv_op(row_ptr, col_ind, values, x, y, base, trans, cols, sizes):
    from . import api
    rows, cols, x_size, y_size = sizes
    a = api.CsrMatrix(rows, cols, row_ptr, col_ind if col_ind.numel() else None, values if values.numel() else None,
                      base, nnz=int(values.numel()))
    return api.SpMV(_handle(), a, api.DnVec(x, size=x_size), api.DnVec(y, size=y_size), op=_OPS[trans])


def spmv_csr(row_ptr, col_ind, values, x, y, alpha: float = 1.0, beta: float = 0.0, base: int = 0, trans: str = "N",
             cols: "int | None" = None) -> torch.Tensor:
    """``y = alpha * op(A) * x + beta * y`` from explicit CSR arrays, in place on ``y`` (the reference's ``spmv_npu``).

    op(A) = T / H is answered with the library's NOT_SUPPORTED status (an ``AclsparseError``) in this build.
    """
    sizes = _check_arrays(row_ptr, col_ind, values, x, y, base, trans, cols)
    with torch.cuda.device(y.device):
        op = _spmv_op(row_ptr, col_ind, values, x, y, base, trans, cols, sizes)
        op.preprocess(alpha, beta)
        op(alpha, beta)
    return y


def spmv_workspace(row_ptr, col_ind, values, x, y, alpha: float = 1.0, beta: float = 0.0, base: int = 0,
                   trans: str = "N", cols: "int | None" = None) -> int:
    """Bytes of external buffer ``aclsparseSpMVGetBufferSize`` asks for (the reference's ``spmv_npu_workspace``)."""
    sizes = _check_arrays(row_ptr, col_ind, values, x, y, base, trans, cols)
    with torch.cuda.device(y.device):
        return _spmv_op(row_ptr, col_ind, values, x, y, base, trans, cols, sizes).buffer_size(alpha, beta)


_installed = []


def install() -> None:
    """Registers ``mv`` as the ``aten::mv`` implementation for CSR CUDA tensors (replacing PyTorch's own)."""
    if _installed:
        return
    lib = torch.library.Library("aten", "IMPL")
    lib.impl("mv", mv, "SparseCsrCUDA")
    _installed.append(lib)  # the registration lives as long as the Library object


__all__ = ["mv", "mm", "addmm", "spmv_csr", "spmv_workspace", "install"]
