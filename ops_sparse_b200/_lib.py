"""ctypes binding of ``libops_sparse.so``, the aclsparse C API built for B200.

The library is built in-tree by ``ops_sparse_b200/csrc/Makefile``.  Importing
this module loads it and fails loudly when it is missing: there is no other
implementation of the operators to fall back on.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libops_sparse.so")

# aclsparseStatus_t
SUCCESS = 0
NOT_INITIALIZED = 1
ALLOC_FAILED = 2
INVALID_VALUE = 3
ARCH_MISMATCH = 4
EXECUTION_FAILED = 5
INTERNAL_ERROR = 6
MATRIX_TYPE_NOT_SUPPORTED = 7
NOT_SUPPORTED = 8
INSUFFICIENT_RESOURCES = 9
HANDLE_IS_NULLPTR = 10

STATUS_NAMES = {
    0: "SUCCESS", 1: "NOT_INITIALIZED", 2: "ALLOC_FAILED", 3: "INVALID_VALUE", 4: "ARCH_MISMATCH",
    5: "EXECUTION_FAILED", 6: "INTERNAL_ERROR", 7: "MATRIX_TYPE_NOT_SUPPORTED", 8: "NOT_SUPPORTED",
    9: "INSUFFICIENT_RESOURCES", 10: "HANDLE_IS_NULLPTR",
}

# aclsparseOperation_t, aclsparseOrder_t, index types / bases, formats, pointer modes
OP_N, OP_T, OP_H = 0, 1, 2
ORDER_ROW, ORDER_COL = 0, 1
INDEX_32I, INDEX_64I = 0, 1
BASE_ZERO, BASE_ONE = 0, 1
FORMAT_COO, FORMAT_CSR, FORMAT_CSC = 0, 1, 2
POINTER_MODE_HOST, POINTER_MODE_DEVICE = 0, 1
# aclsparseSpMVAlg_t / aclsparseSpMMAlg_t
SPMV_ALG_DEFAULT, SPMV_COO_ALG1, SPMV_COO_ALG2, SPMV_CSR_ALG1, SPMV_CSR_ALG2 = 0, 1, 2, 3, 4
SPMM_ALG_DEFAULT, SPMM_CSR_ALG1, SPMM_CSR_FP32_HIGH_PRECISION_ALG, SPMM_CSR_ALG2, SPMM_CSR_ALG3 = 0, 1, 2, 3, 4
# aclDataType
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_DOUBLE, ACL_COMPLEX64, ACL_BF16 = 0, 1, 2, 3, 11, 16, 27


def build() -> str:
    """Compile the library for sm_100a (nvcc cross-compiles without a GPU)."""
    subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), "-j8"], check=True, capture_output=True)
    return LIB_PATH


class BarrierLink(ctypes.Structure):
    """AclspBarrierLink of include/aclsparse_b200_kernels.h."""
    _fields_ = [("local", c_void_p), ("peers", c_void_p * 16), ("world", c_uint32), ("rank", c_uint32),
                ("spinLimit", c_uint32), ("reserved", c_uint32)]


class SpmvParams(ctypes.Structure):
    """AclspSpmvParams of include/aclsparse_b200_kernels.h."""
    _fields_ = [("rows", c_uint32), ("cols", c_uint32), ("nnz", c_uint32), ("indexBase", c_uint32),
                ("colIndStride", c_int64), ("valuesStride", c_int64), ("xStride", c_int64), ("yStride", c_int64),
                ("alpha", c_float), ("beta", c_float), ("alphaPtr", c_void_p), ("betaPtr", c_void_p),
                ("numMirrors", c_uint32), ("mirrorMulticast", c_uint32), ("mirrorDelta", c_int64 * 7),
                ("maxRowLenHint", c_uint32), ("betaSource", c_void_p), ("betaSourceStride", c_int64),
                ("valueType", c_uint32), ("yType", c_uint32), ("computeInt", c_uint32),
                ("alphaInt", ctypes.c_int32), ("betaInt", ctypes.c_int32), ("barrier", BarrierLink)]


# SpmvParams.valueType / yType
TYPE_F32, TYPE_F16, TYPE_BF16, TYPE_I8, TYPE_I32 = 0, 1, 2, 3, 4


MAX_ROW_LEN_UNKNOWN = 0xFFFFFFFF  # SpmvParams.maxRowLenHint when the host does not know the longest row


class SpmmParams(ctypes.Structure):
    """AclspSpmmParams of include/aclsparse_b200_kernels.h."""
    _fields_ = [("rows", c_uint32), ("cols", c_uint32), ("nnz", c_uint32), ("indexBase", c_uint32),
                ("n", c_uint32), ("opB", c_uint32), ("orderB", c_uint32), ("orderC", c_uint32),
                ("highPrecision", c_uint32), ("reserved", c_uint32), ("ldb", c_int64), ("ldc", c_int64), ("alpha", c_float), ("beta", c_float),
                ("alphaPtr", c_void_p), ("betaPtr", c_void_p),
                ("numMirrors", c_uint32), ("mirrorMulticast", c_uint32), ("mirrorDelta", c_int64 * 7),
                ("valueType", c_uint32), ("cType", c_uint32), ("computeInt", c_uint32),
                ("alphaInt", ctypes.c_int32), ("betaInt", ctypes.c_int32), ("barrier", BarrierLink)]


_P = c_void_p
_PP = POINTER(c_void_p)
_I64P = POINTER(c_int64)

# name -> argtypes; every function returns aclsparseStatus_t (int) unless listed in _VOID.
SIGNATURES = {
    "aclsparseCreate": [_PP],
    "aclsparseDestroy": [_P],
    "aclsparseSetStream": [_P, _P],
    "aclsparseGetStream": [_P, _PP],
    "aclsparseSetWorkspace": [_P, _P, c_size_t],
    "aclsparseGetWorkspace": [_P, _PP, POINTER(c_size_t)],
    "aclsparseGetVersion": [_P, POINTER(c_int)],
    "aclsparseSetPointerMode": [_P, c_int],
    "aclsparseGetPointerMode": [_P, POINTER(c_int)],
    "aclsparseCreateDnVec": [_PP, c_int64, _P, c_int],
    "aclsparseCreateConstDnVec": [_PP, c_int64, _P, c_int],
    "aclsparseDestroyDnVec": [_P],
    "aclsparseDnVecGet": [_P, _I64P, _PP, POINTER(c_int)],
    "aclsparseConstDnVecGet": [_P, _I64P, _PP, POINTER(c_int)],
    "aclsparseDnVecGetValues": [_P, _PP],
    "aclsparseConstDnVecGetValues": [_P, _PP],
    "aclsparseDnVecSetValues": [_P, _P],
    "aclsparseDnVecSetStride": [_P, c_int64],
    "aclsparseDnVecGetStride": [_P, _I64P],
    "aclsparseCreateCsr": [_PP, c_int64, c_int64, c_int64, _P, _P, _P, c_int, c_int, c_int, c_int],
    "aclsparseCreateConstCsr": [_PP, c_int64, c_int64, c_int64, _P, _P, _P, c_int, c_int, c_int, c_int],
    "aclsparseCsrSetPointers": [_P, _P, _P, _P],
    "aclsparseCsrSetStrides": [_P, c_int64, c_int64, c_int64],
    "aclsparseCsrGetStrides": [_P, _I64P, _I64P, _I64P],
    "aclsparseDestroySpMat": [_P],
    "aclsparseSpMatGetFormat": [_P, POINTER(c_int)],
    "aclsparseSpMatGetIndexBase": [_P, POINTER(c_int)],
    "aclsparseSpMatGetValues": [_P, _PP],
    "aclsparseConstSpMatGetValues": [_P, _PP],
    "aclsparseSpMatSetValues": [_P, _P],
    "aclsparseSpMatGetSize": [_P, _I64P, _I64P, _I64P],
    "aclsparseCsrGet": [_P, _I64P, _I64P, _I64P, _PP, _PP, _PP, POINTER(c_int), POINTER(c_int), POINTER(c_int),
                        POINTER(c_int)],
    "aclsparseConstCsrGet": [_P, _I64P, _I64P, _I64P, _PP, _PP, _PP, POINTER(c_int), POINTER(c_int),
                             POINTER(c_int), POINTER(c_int)],
    "aclsparseCreateDnMat": [_PP, c_int64, c_int64, c_int64, _P, c_int, c_int],
    "aclsparseCreateConstDnMat": [_PP, c_int64, c_int64, c_int64, _P, c_int, c_int],
    "aclsparseDestroyDnMat": [_P],
    "aclsparseDnMatGet": [_P, _I64P, _I64P, _I64P, _PP, POINTER(c_int), POINTER(c_int)],
    "aclsparseConstDnMatGet": [_P, _I64P, _I64P, _I64P, _PP, POINTER(c_int), POINTER(c_int)],
    "aclsparseDnMatGetValues": [_P, _PP],
    "aclsparseConstDnMatGetValues": [_P, _PP],
    "aclsparseDnMatSetValues": [_P, _P],
    "aclsparseDnMatGetStridedBatch": [_P, POINTER(c_int), _I64P],
    "aclsparseDnMatSetStridedBatch": [_P, c_int, c_int64],
    "aclsparseSpMVGetBufferSize": [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMVPreprocess": [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P],
    "aclsparseSpMV": [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P],
    "aclsparseSpMMGetBufferSize": [_P, c_int, c_int, _P, _P, _P, _P, _P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMMPreprocess": [_P, c_int, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P],
    "aclsparseSpMM": [_P, c_int, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P],
    "aclsparseCreateMatDescr": [_PP],
    "aclsparseDestroyMatDescr": [_P],
    "aclsparseSetMatType": [_P, c_int],
    "aclsparseSetMatIndexBase": [_P, c_int],
    "aclsparseSetMatDiagType": [_P, c_int],
    "aclsparseSetMatFillMode": [_P, c_int],
    "aclsparseGetMatType": [_P],
    "aclsparseGetMatIndexBase": [_P],
    "aclsparseGetMatDiagType": [_P],
    "aclsparseGetMatFillMode": [_P],
    "aclsparseXcoo2csr": [_P, _P, c_int, c_int, _P, c_int],
    "aclsparseXcsrsort_bufferSizeExt": [_P, c_int, c_int, c_int, _P, _P, POINTER(c_size_t)],
    "aclsparseXcsrsort": [_P, c_int, c_int, c_int, _P, _P, _P, _P, _P],
    "aclsparseSpMVOp_bufferSize": [_P, c_int, _P, _P, _P, _P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMVOp_createDescr": [_P, _PP, c_int, _P, _P, _P, _P, c_int, c_int, _P],
    "aclsparseSpMVOp_destroyDescr": [_P],
    "aclsparseSpMVOp_createPlan": [_P, _P, _PP, _P, c_size_t],
    "aclsparseSpMVOp_destroyPlan": [_P],
    "aclsparseSpMVOp_setGlobalUserData": [_P, _P, ctypes.c_char_p, _P, c_size_t],
    "aclsparseSpMVOp": [_P, _P, _P, _P, _P, _P, _P],
    "aclsparseSpMMOp_bufferSize": [_P, c_int, c_int, _P, _P, _P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMMOp_createDescr": [_P, _PP, c_int, c_int, _P, _P, _P, c_int, c_int, _P],
    "aclsparseSpMMOp_destroyDescr": [_P],
    "aclsparseSpMMOp_createPlan": [_P, _P, _PP, _P, c_size_t],
    "aclsparseSpMMOp_destroyPlan": [_P],
    "aclsparseSpMMOp_setGlobalUserData": [_P, _P, ctypes.c_char_p, _P, c_size_t],
    "aclsparseSpMMOp": [_P, _P, _P, _P, _P, _P],
    # include/aclsparse_b200_ext.h
    "aclsparseB200RowBlockBounds": [_P, _P, c_int, _P],
    "aclsparseB200SpMVNoAlloc": [_P, c_int64, c_int64, c_int64, _P, _P, _P, c_int, _P, _P, c_float, c_float],
    "aclsparseB200DnVecSetMirrors": [_P, c_int, POINTER(c_void_p)],
    "aclsparseB200DnMatSetMirrors": [_P, c_int, POINTER(c_void_p)],
    "aclsparseB200DnVecSetMulticastMirror": [_P, _P],
    "aclsparseB200DnMatSetMulticastMirror": [_P, _P],
    "aclsparseB200NodeBarrier": [_P, _P, POINTER(c_void_p), c_int, c_int, c_uint32],
    "aclsparseB200NodeBarrierStatus": [_P, _P, POINTER(c_int)],
    "aclsparseB200SpMVWaitFailures": [_P, _P, POINTER(c_uint32)],
    "aclsparseB200DnVecSetClosingBarrier": [_P, _P, POINTER(c_void_p), c_int, c_int, c_uint32],
    "aclsparseB200DnMatSetClosingBarrier": [_P, _P, POINTER(c_void_p), c_int, c_int, c_uint32],
    # include/aclsparse_b200_kernels.h
    "spmv_b200_preprocess_kernel_do": [_P, _P, c_uint32, c_uint32, c_uint32, c_int32, c_int64, _P],
    "spmv_b200_kernel_do": [_P, _P, _P, _P, _P, POINTER(SpmvParams), _P],
    "spmm_b200_preprocess_kernel_do": [_P, _P, c_uint32, c_uint32, c_uint32, c_uint32, c_int32, _P],
    "spmm_b200_kernel_do": [_P, _P, _P, _P, _P, POINTER(SpmmParams), _P],
    "aclsp_b200_row_block_bounds_kernel_do": [_P, c_uint32, c_uint32, c_int32, c_uint32, _P, _P],
    "aclsp_b200_push_slice_kernel_do": [_P, POINTER(c_void_p), c_uint32, c_int64, c_int64, _P],
    "aclsp_b200_node_barrier_kernel_do": [_P, POINTER(c_void_p), c_uint32, c_uint32, c_uint32, _P],
    "aclsp_b200_kernel_launches": [],
    "aclsp_b200_transpose_build_kernel_do": [_P, _P, c_uint32, c_uint32, c_uint32, c_int32, c_int64, c_int64, _P, _P, _P],
    "aclsp_b200_transpose_values_kernel_do": [_P, c_int64, c_uint32, c_uint32, _P, _P, c_uint32, _P],
}
_VOID = {"spmv_b200_preprocess_kernel_do", "spmv_b200_kernel_do", "spmm_b200_preprocess_kernel_do",
         "spmm_b200_kernel_do", "aclsp_b200_row_block_bounds_kernel_do", "aclsp_b200_push_slice_kernel_do",
         "aclsp_b200_node_barrier_kernel_do", "aclsp_b200_transpose_build_kernel_do",
         "aclsp_b200_transpose_values_kernel_do", "aclsparseSetMatType", "aclsparseSetMatIndexBase",
         "aclsparseSetMatDiagType", "aclsparseSetMatFillMode"}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library, with argument types declared for every exported entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C ops_sparse_b200/csrc` "
                "(or __graft_entry__.build()); there is no fallback implementation")
        handle = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = args
            fn.restype = None if name in _VOID else (ctypes.c_uint64 if name == "aclsp_b200_kernel_launches" else c_int)
        _lib = handle
    return _lib
