/*
 * aclsparse C API — the CSR SpMV / SpMM slice, implemented for NVIDIA B200.
 *
 * This header declares the subset of the ops-sparse public interface
 * (reference: include/cann_ops_sparse.h) that the CSR sparse-matrix x
 * dense-vector and sparse-matrix x dense-matrix products use: the library
 * handle, CSR / dense-vector / dense-matrix descriptors and the three-phase
 * GetBufferSize -> Preprocess -> execute entry points.  Names, argument order,
 * enum values and status codes are the reference's, so a caller that links
 * against the reference's libops_sparse.so for this path can link against
 * this library instead.  Every "reference:" note gives the file:line of the
 * declaration or definition an entry replaces.
 *
 * Device pointers are CUDA device pointers; `aclrtStream` is a cudaStream_t.
 * All functions return a status and never throw.  Validation finishes before
 * anything is enqueued; execution is asynchronous on the handle's stream.
 */
#ifndef CANN_OPS_SPARSE_H_
#define CANN_OPS_SPARSE_H_

#include <stddef.h>
#include <stdint.h>
#include <acl/acl_base_rt.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility: only what this header declares is exported. */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* ---------------------------------------------------------------- enums -- */

/* reference: include/cann_ops_sparse.h:32-36 */
typedef enum aclsparseOperation_t {
    ACL_SPARSE_OP_NON_TRANSPOSE = 0,
    ACL_SPARSE_OP_TRANSPOSE = 1,
    ACL_SPARSE_OP_CONJUGATE_TRANSPOSE = 2
} aclsparseOperation_t;

/* reference: include/cann_ops_sparse.h:63-66 */
typedef enum aclsparseOrder_t {
    ACL_SPARSE_ORDER_ROW = 0,
    ACL_SPARSE_ORDER_COL = 1
} aclsparseOrder_t;

/* reference: include/cann_ops_sparse.h:94-109 */
typedef enum aclsparseSpMMAlg_t {
    ACL_SPARSE_SPMM_ALG_DEFAULT = 0,
    ACL_SPARSE_SPMM_CSR_ALG1 = 1,
    ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG = 2,
    ACL_SPARSE_SPMM_CSR_ALG2 = 3,
    ACL_SPARSE_SPMM_CSR_ALG3 = 4
} aclsparseSpMMAlg_t;

/* reference: include/cann_ops_sparse.h:124-174 */
typedef enum aclsparseStatus_t {
    ACL_SPARSE_STATUS_SUCCESS = 0,
    ACL_SPARSE_STATUS_NOT_INITIALIZED = 1,
    ACL_SPARSE_STATUS_ALLOC_FAILED = 2,
    ACL_SPARSE_STATUS_INVALID_VALUE = 3,
    ACL_SPARSE_STATUS_ARCH_MISMATCH = 4,
    ACL_SPARSE_STATUS_EXECUTION_FAILED = 5,
    ACL_SPARSE_STATUS_INTERNAL_ERROR = 6,
    ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED = 7,
    ACL_SPARSE_STATUS_NOT_SUPPORTED = 8,
    ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES = 9,
    ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR = 10
} aclsparseStatus_t;

/* reference: include/cann_ops_sparse.h:176-201.  Only DEFAULT, CSR_ALG1 and
 * CSR_ALG2 are accepted by SpMV; every accepted value selects the same
 * deterministic B200 kernels (results are bit-reproducible run to run). */
typedef enum aclsparseSpMVAlg_t {
    ACL_SPARSE_SPMV_ALG_DEFAULT = 0,
    ACL_SPARSE_SPMV_COO_ALG1 = 1,
    ACL_SPARSE_SPMV_COO_ALG2 = 2,
    ACL_SPARSE_SPMV_CSR_ALG1 = 3,
    ACL_SPARSE_SPMV_CSR_ALG2 = 4,
    ACL_SPARSE_SPMV_SELL_ALG1 = 5,
    ACL_SPARSE_SPMV_CSR_ALG_CUBE = 6
} aclsparseSpMVAlg_t;

/* reference: include/cann_ops_sparse.h:244-253 */
typedef enum aclsparseIndexType_t {
    ACL_SPARSE_INDEX_32I = 0,
    ACL_SPARSE_INDEX_64I = 1
} aclsparseIndexType_t;

/* reference: include/cann_ops_sparse.h:258-261 */
typedef enum aclsparseIndexBase_t {
    ACL_SPARSE_INDEX_BASE_ZERO = 0,
    ACL_SPARSE_INDEX_BASE_ONE = 1
} aclsparseIndexBase_t;

/* reference: include/cann_ops_sparse.h:264-277 */
typedef enum aclsparseFormat_t {
    ACL_SPARSE_FORMAT_COO = 0,
    ACL_SPARSE_FORMAT_CSR = 1,
    ACL_SPARSE_FORMAT_CSC = 2,
    ACL_SPARSE_FORMAT_BLOCKED_ELL = 3,
    ACL_SPARSE_FORMAT_SLICED_ELL = 4,
    ACL_SPARSE_FORMAT_BSR = 5
} aclsparseFormat_t;

/* reference: include/cann_ops_sparse.h:1623-1626 */
typedef enum aclsparsePointerMode_t {
    ACL_SPARSE_POINTER_MODE_HOST = 0,
    ACL_SPARSE_POINTER_MODE_DEVICE = 1
} aclsparsePointerMode_t;

/* reference: include/cann_ops_sparse.h:205-213 (scalar layout for complex) */
typedef struct aclsparseComplex {
    float x;
    float y;
} aclsparseComplex;

/* --------------------------------------------------------- opaque types -- */

/* reference: include/cann_ops_sparse.h:38-61 */
struct aclsparseContext;
struct aclsparseSpMatDescr;
struct aclsparseDnVecDescr;
struct aclsparseDnMatDescr;

typedef struct aclsparseContext* aclsparseHandle_t;
typedef struct aclsparseSpMatDescr* aclsparseSpMatDescr_t;
typedef struct aclsparseDnVecDescr* aclsparseDnVecDescr_t;
typedef struct aclsparseDnMatDescr* aclsparseDnMatDescr_t;
typedef struct aclsparseSpMatDescr const* aclsparseConstSpMatDescr_t;
typedef struct aclsparseDnVecDescr const* aclsparseConstDnVecDescr_t;
typedef struct aclsparseDnMatDescr const* aclsparseConstDnMatDescr_t;

/* --------------------------------------------------------------- handle -- */

/* reference: include/cann_ops_sparse.h:1542 (aclsparse_auxiliary.cpp:103-131).
 * *handle must be NULL on entry.  The 4 MiB library workspace of the
 * reference is allocated on first aclsparseGetWorkspace, not here, so that
 * creating a handle touches no device. */
aclsparseStatus_t aclsparseCreate(aclsparseHandle_t* handle);
/* reference: include/cann_ops_sparse.h:1553 (aclsparse_auxiliary.cpp:133-160) */
aclsparseStatus_t aclsparseDestroy(aclsparseHandle_t handle);
/* reference: include/cann_ops_sparse.h:1562 (aclsparse_auxiliary.cpp:162-179) */
aclsparseStatus_t aclsparseSetStream(aclsparseHandle_t handle, aclrtStream stream);
/* reference: include/cann_ops_sparse.h:1572 */
aclsparseStatus_t aclsparseGetStream(aclsparseHandle_t handle, aclrtStream* stream);
/* reference: include/cann_ops_sparse.h:1591 (grow-only, borrowed memory) */
aclsparseStatus_t aclsparseSetWorkspace(aclsparseHandle_t handle, void* workspace, size_t workspaceSize);
/* reference: include/cann_ops_sparse.h:1605 */
aclsparseStatus_t aclsparseGetWorkspace(aclsparseHandle_t handle, void** workspace, size_t* workspaceSize);
/* reference: include/cann_ops_sparse.h:1617 (MAJOR*10000 + MINOR*100 + PATCH) */
aclsparseStatus_t aclsparseGetVersion(aclsparseHandle_t handle, int* version);
/* reference: include/cann_ops_sparse.h:1637 */
aclsparseStatus_t aclsparseSetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t mode);
/* reference: include/cann_ops_sparse.h:1647 */
aclsparseStatus_t aclsparseGetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t* mode);

/* --------------------------------------------------------- dense vector -- */

/* reference: include/cann_ops_sparse.h:288 (aclsparse_descr.cpp:375-401) */
aclsparseStatus_t aclsparseCreateDnVec(aclsparseDnVecDescr_t* dnVecDescr, int64_t size, void* values,
                                       aclDataType valueType);
/* reference: include/cann_ops_sparse.h:294 */
aclsparseStatus_t aclsparseCreateConstDnVec(aclsparseConstDnVecDescr_t* dnVecDescr, int64_t size,
                                            const void* values, aclDataType valueType);
/* reference: include/cann_ops_sparse.h:304 (NULL is a successful no-op) */
aclsparseStatus_t aclsparseDestroyDnVec(aclsparseConstDnVecDescr_t dnVecDescr);
/* reference: include/cann_ops_sparse.h:455 (every OUT pointer is optional) */
aclsparseStatus_t aclsparseDnVecGet(aclsparseDnVecDescr_t dnVecDescr, int64_t* size, void** values,
                                    aclDataType* valueType);
/* reference: include/cann_ops_sparse.h:464 */
aclsparseStatus_t aclsparseConstDnVecGet(aclsparseConstDnVecDescr_t dnVecDescr, int64_t* size,
                                         const void** values, aclDataType* valueType);
/* reference: include/cann_ops_sparse.h:474 */
aclsparseStatus_t aclsparseDnVecGetValues(aclsparseDnVecDescr_t dnVecDescr, void** values);
/* reference: include/cann_ops_sparse.h:479 */
aclsparseStatus_t aclsparseConstDnVecGetValues(aclsparseConstDnVecDescr_t dnVecDescr, const void** values);
/* reference: include/cann_ops_sparse.h:488 */
aclsparseStatus_t aclsparseDnVecSetValues(aclsparseDnVecDescr_t dnVecDescr, void* values);
/* reference: include/cann_ops_sparse.h:497 (element stride, > 0) */
aclsparseStatus_t aclsparseDnVecSetStride(aclsparseDnVecDescr_t dnVecDescr, int64_t stride);
/* reference: include/cann_ops_sparse.h:502 */
aclsparseStatus_t aclsparseDnVecGetStride(aclsparseConstDnVecDescr_t dnVecDescr, int64_t* stride);

/* ----------------------------------------------------------- CSR matrix -- */

/* reference: include/cann_ops_sparse.h:529 (aclsparse_descr.cpp:648-693).
 * Data pointers may be NULL here and bound later with aclsparseCsrSetPointers. */
aclsparseStatus_t aclsparseCreateCsr(aclsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                     void* csrRowOffsets, void* csrColInd, void* csrValues,
                                     aclsparseIndexType_t csrRowOffsetsType, aclsparseIndexType_t csrColIndType,
                                     aclsparseIndexBase_t idxBase, aclDataType valueType);
/* reference: include/cann_ops_sparse.h:535 */
aclsparseStatus_t aclsparseCreateConstCsr(aclsparseConstSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols,
                                          int64_t nnz, const void* csrRowOffsets, const void* csrColInd,
                                          const void* csrValues, aclsparseIndexType_t csrRowOffsetsType,
                                          aclsparseIndexType_t csrColIndType, aclsparseIndexBase_t idxBase,
                                          aclDataType valueType);
/* reference: include/cann_ops_sparse.h:797 (aclsparse_descr.cpp:911-947).
 * Any pointer change drops the cached SpMV / SpMM preprocessing of the
 * descriptor. */
aclsparseStatus_t aclsparseCsrSetPointers(aclsparseSpMatDescr_t descr, void* rowOffsets, void* colIndices,
                                          void* values);
/* reference: include/cann_ops_sparse.h:804 (element strides, all > 0) */
aclsparseStatus_t aclsparseCsrSetStrides(aclsparseSpMatDescr_t descr, int64_t rowOffsetsStride,
                                         int64_t colIndStride, int64_t valuesStride);
/* reference: include/cann_ops_sparse.h:811 */
aclsparseStatus_t aclsparseCsrGetStrides(aclsparseConstSpMatDescr_t descr, int64_t* rowOffsetsStride,
                                         int64_t* colIndStride, int64_t* valuesStride);
/* reference: include/cann_ops_sparse.h:872 (NULL is a successful no-op) */
aclsparseStatus_t aclsparseDestroySpMat(aclsparseConstSpMatDescr_t spMatDescr);
/* reference: include/cann_ops_sparse.h:885 */
aclsparseStatus_t aclsparseSpMatGetFormat(aclsparseConstSpMatDescr_t spMatDescr, aclsparseFormat_t* format);
/* reference: include/cann_ops_sparse.h:893 */
aclsparseStatus_t aclsparseSpMatGetIndexBase(aclsparseConstSpMatDescr_t spMatDescr, aclsparseIndexBase_t* idxBase);
/* reference: include/cann_ops_sparse.h:903 */
aclsparseStatus_t aclsparseSpMatGetValues(aclsparseSpMatDescr_t spMatDescr, void** values);
/* reference: include/cann_ops_sparse.h:908 */
aclsparseStatus_t aclsparseConstSpMatGetValues(aclsparseConstSpMatDescr_t spMatDescr, const void** values);
/* reference: include/cann_ops_sparse.h:920 */
aclsparseStatus_t aclsparseSpMatSetValues(aclsparseSpMatDescr_t spMatDescr, void* values);
/* reference: include/cann_ops_sparse.h:927 */
aclsparseStatus_t aclsparseSpMatGetSize(aclsparseConstSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols,
                                        int64_t* nnz);
/* reference: include/cann_ops_sparse.h:2736 (every OUT pointer is optional) */
aclsparseStatus_t aclsparseCsrGet(aclsparseSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols, int64_t* nnz,
                                  void** csrRowOffsets, void** csrColInd, void** csrValues,
                                  aclsparseIndexType_t* csrRowOffsetsType, aclsparseIndexType_t* csrColIndType,
                                  aclsparseIndexBase_t* idxBase, aclDataType* valueType);
/* reference: include/cann_ops_sparse.h:2746 */
aclsparseStatus_t aclsparseConstCsrGet(aclsparseConstSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols,
                                       int64_t* nnz, const void** csrRowOffsets, const void** csrColInd,
                                       const void** csrValues, aclsparseIndexType_t* csrRowOffsetsType,
                                       aclsparseIndexType_t* csrColIndType, aclsparseIndexBase_t* idxBase,
                                       aclDataType* valueType);

/* --------------------------------------------------------- dense matrix -- */

/* reference: include/cann_ops_sparse.h:1028 (aclsparse_descr.cpp:1102-1152) */
aclsparseStatus_t aclsparseCreateDnMat(aclsparseDnMatDescr_t* dnMatDescr, int64_t rows, int64_t cols, int64_t ld,
                                       void* values, aclDataType valueType, aclsparseOrder_t order);
/* reference: include/cann_ops_sparse.h:1036 */
aclsparseStatus_t aclsparseCreateConstDnMat(aclsparseConstDnMatDescr_t* dnMatDescr, int64_t rows, int64_t cols,
                                            int64_t ld, const void* values, aclDataType valueType,
                                            aclsparseOrder_t order);
/* reference: include/cann_ops_sparse.h:1045 (NULL is a successful no-op) */
aclsparseStatus_t aclsparseDestroyDnMat(aclsparseConstDnMatDescr_t dnMatDescr);
/* reference: include/cann_ops_sparse.h:1061 (every OUT pointer is optional) */
aclsparseStatus_t aclsparseDnMatGet(aclsparseDnMatDescr_t dnMatDescr, int64_t* rows, int64_t* cols, int64_t* ld,
                                    void** values, aclDataType* valueType, aclsparseOrder_t* order);
/* reference: include/cann_ops_sparse.h:1070 */
aclsparseStatus_t aclsparseConstDnMatGet(aclsparseConstDnMatDescr_t dnMatDescr, int64_t* rows, int64_t* cols,
                                         int64_t* ld, const void** values, aclDataType* valueType,
                                         aclsparseOrder_t* order);
/* reference: include/cann_ops_sparse.h:1081 */
aclsparseStatus_t aclsparseDnMatGetValues(aclsparseDnMatDescr_t dnMatDescr, void** values);
/* reference: include/cann_ops_sparse.h:1086 */
aclsparseStatus_t aclsparseConstDnMatGetValues(aclsparseConstDnMatDescr_t dnMatDescr, const void** values);
/* reference: include/cann_ops_sparse.h:1095 */
aclsparseStatus_t aclsparseDnMatSetValues(aclsparseDnMatDescr_t dnMatDescr, void* values);
/* reference: include/cann_ops_sparse.h:1109 */
aclsparseStatus_t aclsparseDnMatGetStridedBatch(aclsparseConstDnMatDescr_t dnMatDescr, int* batchCount,
                                                int64_t* batchStride);
/* reference: include/cann_ops_sparse.h:1126 */
aclsparseStatus_t aclsparseDnMatSetStridedBatch(aclsparseDnMatDescr_t dnMatDescr, int batchCount,
                                                int64_t batchStride);

/* ----------------------------------------------------------------- SpMV -- */

/* y = alpha * op(A) * x + beta * y,  A in CSR with int32 indices, fp32 data.
 *
 * GetBufferSize only looks at descriptor metadata (data pointers may still be
 * unbound) and never touches device memory.  The size it returns is the
 * caller's contract: Preprocess and SpMV write row-partition metadata and
 * per-tile carries into the first `bufferSize` bytes of `externalBuffer`,
 * which must be 64-byte aligned.  Preprocess is optional: SpMV rebuilds the
 * metadata on the handle's stream whenever the buffer does not hold a plan
 * for this matrix.  When beta == 0, y is never read. */

/* reference: include/cann_ops_sparse.h:960 (sparse/spmv/arch35/spmv_host.cpp:636-658) */
aclsparseStatus_t aclsparseSpMVGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA, const void* alpha,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                             const void* beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                             aclsparseSpMVAlg_t alg, size_t* bufferSize);
/* reference: include/cann_ops_sparse.h:983 (sparse/spmv/arch35/spmv_host.cpp:526-583) */
aclsparseStatus_t aclsparseSpMVPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA, const void* alpha,
                                          aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                          const void* beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                          aclsparseSpMVAlg_t alg, void* externalBuffer);
/* reference: include/cann_ops_sparse.h:1003 (sparse/spmv/arch35/spmv_host.cpp:585-632) */
aclsparseStatus_t aclsparseSpMV(aclsparseHandle_t handle, aclsparseOperation_t opA, const void* alpha,
                                aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX, const void* beta,
                                aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                void* externalBuffer);

/* ----------------------------------------------------------------- SpMM -- */

/* C = alpha * op(A) * op(B) + beta * C,  A in CSR (int32, fp32), B and C
 * dense fp32.  Same three-phase contract as SpMV.  When beta == 0, C is
 * never read. */

/* reference: include/cann_ops_sparse.h:1203 (sparse/spmm/arch35/host/spmm_host.cpp:1395-1429) */
aclsparseStatus_t aclsparseSpMMGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseOperation_t opB, const void* alpha,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                             const void* beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                             aclsparseSpMMAlg_t alg, size_t* size);
/* reference: include/cann_ops_sparse.h:1212 (sparse/spmm/arch35/host/spmm_host.cpp:1824-1874) */
aclsparseStatus_t aclsparseSpMMPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                          aclsparseOperation_t opB, const void* alpha,
                                          aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                          const void* beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                          aclsparseSpMMAlg_t alg, void* buffer);
/* reference: include/cann_ops_sparse.h:1220 (sparse/spmm/arch35/host/spmm_host.cpp:1903-1965) */
aclsparseStatus_t aclsparseSpMM(aclsparseHandle_t handle, aclsparseOperation_t opA, aclsparseOperation_t opB,
                                const void* alpha, aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                const void* beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                aclsparseSpMMAlg_t alg, void* buffer);

/* --------------------------------------------------- format producers -- */

/* What feeds the path for callers that start from COO or from unsorted CSR: row offsets from sorted COO
 * row indices, and the in-row sort of CSR column indices (with the permutation to apply to the values).
 * Integer work, asynchronous on the handle's stream. */

/* reference: include/cann_ops_sparse.h:225-241 */
struct aclsparseMatDescr;
typedef struct aclsparseMatDescr* aclsparseMatDescr_t;
typedef enum aclsparseMatrixType_t {
    ACL_SPARSE_MATRIX_TYPE_GENERAL = 0,
    ACL_SPARSE_MATRIX_TYPE_SYMMETRIC,
    ACL_SPARSE_MATRIX_TYPE_HERMITIAN,
    ACL_SPARSE_MATRIX_TYPE_TRIANGULAR
} aclsparseMatrixType_t;
typedef enum aclsparseDiagType_t { ACL_SPARSE_DIAG_TYPE_NON_UNIT = 0, ACL_SPARSE_DIAG_TYPE_UNIT } aclsparseDiagType_t;
typedef enum aclsparseFillMode_t { ACL_SPARSE_FILL_MODE_LOWER = 0, ACL_SPARSE_FILL_MODE_UPPER } aclsparseFillMode_t;

/* reference: include/cann_ops_sparse.h:1659-1673; Destroy(NULL) is SUCCESS; the setters ignore NULL */
aclsparseStatus_t aclsparseCreateMatDescr(aclsparseMatDescr_t* descr);
aclsparseStatus_t aclsparseDestroyMatDescr(aclsparseMatDescr_t descr);
void aclsparseSetMatType(aclsparseMatDescr_t descr, aclsparseMatrixType_t type);
void aclsparseSetMatIndexBase(aclsparseMatDescr_t descr, aclsparseIndexBase_t base);
void aclsparseSetMatDiagType(aclsparseMatDescr_t descr, aclsparseDiagType_t diagType);
void aclsparseSetMatFillMode(aclsparseMatDescr_t descr, aclsparseFillMode_t fillMode);
aclsparseMatrixType_t aclsparseGetMatType(aclsparseMatDescr_t descr);
aclsparseIndexBase_t aclsparseGetMatIndexBase(aclsparseMatDescr_t descr);
aclsparseDiagType_t aclsparseGetMatDiagType(aclsparseMatDescr_t descr);
aclsparseFillMode_t aclsparseGetMatFillMode(aclsparseMatDescr_t descr);

/* csrRowPtr[r] = idxBase + number of entries whose row is below r, r = 0..m, for COO row indices sorted
 * non-decreasing (with idxBase).  reference: include/cann_ops_sparse.h:2800
 * (sparse/coo2csr/arch35/coo2csr_host.cpp:38-77) */
aclsparseStatus_t aclsparseXcoo2csr(aclsparseHandle_t handle, const int* cooRowInd, int nnz, int m, int* csrRowPtr,
                                    aclsparseIndexBase_t idxBase);

/* Sorts the column indices of every CSR row ascending, in place and stably, and applies the same
 * permutation to P (the caller usually starts from the identity and gathers the values through P).
 * The workspace holds 8 bytes per non-zero.  reference: include/cann_ops_sparse.h:2528,2545
 * (sparse/csrsort/arch35/csrsort_host.cpp:40-215) */
aclsparseStatus_t aclsparseXcsrsort_bufferSizeExt(aclsparseHandle_t handle, int m, int n, int nnz, const int* csrRowPtr,
                                                  const int* csrColInd, size_t* pBufferSizeInBytes);
aclsparseStatus_t aclsparseXcsrsort(aclsparseHandle_t handle, int m, int n, int nnz, const aclsparseMatDescr_t descrA,
                                    const int* csrRowPtr, int* csrColInd, int* P, void* pBuffer);

/* ------------------------------------------------------- SpMVOp / SpMMOp -- */

/* The plan API: create once, execute many.
 *   bufferSize -> createDescr (binds A, preprocesses into `buffer`) -> createPlan
 *   -> [setGlobalUserData] -> execute (repeatable) -> destroyPlan -> destroyDescr
 * SpMVOp: Z = alpha*A*X + beta*Y with Z a vector of its own (Z may be Y).  SpMMOp: C = alpha*A*op(B) +
 * beta*C, B and C given at execute.  op(A) is NON_TRANSPOSE, data fp32, indices int32.  Every algorithm
 * value needs the buffer, adds in a fixed order (results are bit-wise reproducible) and picks up new
 * values of A at the next execute.  `buffer` stays the caller's and must outlive the descriptor. */

/* reference: include/cann_ops_sparse.h:69-83 */
typedef enum aclsparseSpMVOpAlg_t {
    ACL_SPARSE_SPMVOP_ALG_DEFAULT = 0,
    ACL_SPARSE_SPMVOP_ALG1,
    ACL_SPARSE_SPMVOP_ALG2
} aclsparseSpMVOpAlg_t;

/* reference: include/cann_ops_sparse.h:2412-2417 */
typedef enum aclsparseSpMMOpAlg_t {
    ACL_SPARSE_SPMMOP_ALG_DEFAULT = 0,
    ACL_SPARSE_SPMMOP_ALG1,
    ACL_SPARSE_SPMMOP_ALG2,
    ACL_SPARSE_SPMMOP_ALG1_HIGH_PRECISION
} aclsparseSpMMOpAlg_t;

/* reference: include/cann_ops_sparse.h:86-91, 2420-2425 */
struct aclsparseSpMVOpDescr;
struct aclsparseSpMVOpPlan;
typedef struct aclsparseSpMVOpDescr* aclsparseSpMVOpDescr_t;
typedef struct aclsparseSpMVOpDescr const* aclsparseConstSpMVOpDescr_t;
typedef struct aclsparseSpMVOpPlan* aclsparseSpMVOpPlan_t;
struct aclsparseSpMMOpDescr;
struct aclsparseSpMMOpPlan;
typedef struct aclsparseSpMMOpDescr* aclsparseSpMMOpDescr_t;
typedef struct aclsparseSpMMOpDescr const* aclsparseConstSpMMOpDescr_t;
typedef struct aclsparseSpMMOpPlan* aclsparseSpMMOpPlan_t;

/* reference: include/cann_ops_sparse.h:2345 (sparse/spmv_op/arch35/spmv_op_host.cpp:520-559) */
aclsparseStatus_t aclsparseSpMVOp_bufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                             aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ,
                                             aclDataType computeType, aclsparseSpMVOpAlg_t alg, size_t* bufferSize);
/* reference: include/cann_ops_sparse.h:2355 (spmv_op_host.cpp:630-673) */
aclsparseStatus_t aclsparseSpMVOp_createDescr(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t* descr,
                                              aclsparseOperation_t opA, aclsparseConstSpMatDescr_t matA,
                                              aclsparseConstDnVecDescr_t vecX, aclsparseConstDnVecDescr_t vecY,
                                              aclsparseDnVecDescr_t vecZ, aclDataType computeType,
                                              aclsparseSpMVOpAlg_t alg, void* buffer);
/* reference: include/cann_ops_sparse.h:2365 (spmv_op_host.cpp:676-683); NULL is SUCCESS */
aclsparseStatus_t aclsparseSpMVOp_destroyDescr(aclsparseSpMVOpDescr_t descr);
/* reference: include/cann_ops_sparse.h:2371 (spmv_op_host.cpp:686-712); the epilogue buffer must be NULL */
aclsparseStatus_t aclsparseSpMVOp_createPlan(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t descr,
                                             aclsparseSpMVOpPlan_t* plan, const void* epilogueLTOBuffer,
                                             size_t epilogueLTOBufferSize);
/* reference: include/cann_ops_sparse.h:2380 (spmv_op_host.cpp:715-722); NULL is SUCCESS */
aclsparseStatus_t aclsparseSpMVOp_destroyPlan(aclsparseSpMVOpPlan_t plan);
/* reference: include/cann_ops_sparse.h:2386 (spmv_op_host.cpp:725-749); identity epilogue: nothing to set */
aclsparseStatus_t aclsparseSpMVOp_setGlobalUserData(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan,
                                                    const char* epilogueDataName, void* epilogueData,
                                                    size_t epilogueDataSize);
/* reference: include/cann_ops_sparse.h:2394 (spmv_op_host.cpp:752-772) */
aclsparseStatus_t aclsparseSpMVOp(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan, const void* alpha,
                                  const void* beta, aclsparseConstDnVecDescr_t vecX, aclsparseConstDnVecDescr_t vecY,
                                  aclsparseDnVecDescr_t vecZ);

/* reference: include/cann_ops_sparse.h:2431 (sparse/spmm_op/arch35/spmm_op_host.cpp:695-730) */
aclsparseStatus_t aclsparseSpMMOp_bufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseOperation_t opB, aclsparseConstSpMatDescr_t matA,
                                             aclsparseConstDnMatDescr_t matB, aclsparseDnMatDescr_t matC,
                                             aclDataType computeType, aclsparseSpMMOpAlg_t alg, size_t* bufferSize);
/* reference: include/cann_ops_sparse.h:2442 */
aclsparseStatus_t aclsparseSpMMOp_createDescr(aclsparseHandle_t handle, aclsparseSpMMOpDescr_t* descr,
                                              aclsparseOperation_t opA, aclsparseOperation_t opB,
                                              aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                              aclsparseDnMatDescr_t matC, aclDataType computeType,
                                              aclsparseSpMMOpAlg_t alg, void* buffer);
/* reference: include/cann_ops_sparse.h:2452; NULL is SUCCESS */
aclsparseStatus_t aclsparseSpMMOp_destroyDescr(aclsparseSpMMOpDescr_t descr);
/* reference: include/cann_ops_sparse.h:2458; the epilogue buffer must be NULL */
aclsparseStatus_t aclsparseSpMMOp_createPlan(aclsparseHandle_t handle, aclsparseSpMMOpDescr_t descr,
                                             aclsparseSpMMOpPlan_t* plan, const void* epilogueLTOBuffer,
                                             size_t epilogueLTOBufferSize);
/* reference: include/cann_ops_sparse.h:2467; NULL is SUCCESS */
aclsparseStatus_t aclsparseSpMMOp_destroyPlan(aclsparseSpMMOpPlan_t plan);
/* reference: include/cann_ops_sparse.h:2473 */
aclsparseStatus_t aclsparseSpMMOp_setGlobalUserData(aclsparseHandle_t handle, aclsparseSpMMOpPlan_t plan,
                                                    const char* epilogueDataName, void* epilogueData,
                                                    size_t epilogueDataSize);
/* reference: include/cann_ops_sparse.h:2484 */
aclsparseStatus_t aclsparseSpMMOp(aclsparseHandle_t handle, aclsparseSpMMOpPlan_t plan, const void* alpha,
                                  const void* beta, aclsparseConstDnMatDescr_t matB, aclsparseDnMatDescr_t matC);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif

#endif /* CANN_OPS_SPARSE_H_ */
