/*
 * Host layer of aclsparseSpMM: validation, buffer sizing, plan bookkeeping and
 * the calls into the CUDA launch shim.  The order of the checks, and therefore
 * which status a bad call gets, follows the reference's
 * sparse/spmm/arch35/host/spmm_host.cpp (entry points :1395-1429, :1824-1874,
 * :1903-1965; ValidateSpmmInputs :474-568).
 *
 * Differences that a caller can observe:
 *  - op(A) = transpose (and conjugate transpose: the data is real) builds the transposed matrix in
 *    the external buffer during preprocessing, on the device, and multiplies with it (the reference
 *    builds a CSC copy on the host, spmm_csr_mat.cpp:212-315); the buffer then needs about 12 bytes
 *    per non-zero more;
 *  - the complex row of the reference's dtype table (spmm_host.cpp:379-387) is answered with NOT_SUPPORTED;
 *    the others (fp32, fp16 / bf16 A and B with C of the same type or fp32, int8 with an int32 C) are computed;
 *  - the buffer must be 64-byte aligned (INVALID_VALUE otherwise) and its size
 *    covers the B200 plan, not the reference's reorder table;
 *  - preprocessing never copies anything to the host, and the plan depends on
 *    the structure of A and the width of C only: calling with another B, C,
 *    alpha or beta reuses it (the reference rebuilds, spmm_host.cpp:63-97,199-215);
 *  - every algorithm value selects the same kernels, which add in a fixed
 *    order (so all of them are deterministic, as the reference's CSR_ALG3 is) and
 *    with fp64 products and fp64 row sums (so all of them are at least as
 *    accurate as the reference's FP32_HIGH_PRECISION, which is Kahan-compensated
 *    fp32, spmm_kernel_simt.cpp:424-431, and equal its fp64 test golden up to
 *    the order of the additions, also in cancelling rows and on Inf / NaN data).
 */
#include <cstdint>
#include <limits>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "internal.h"
#include "plan_layout.h"

namespace {

constexpr const char* kApi = "aclsparseSpMM";
constexpr int64_t kMaxI32 = std::numeric_limits<int32_t>::max();

bool IsOperation(aclsparseOperation_t op)
{
    return op == ACL_SPARSE_OP_NON_TRANSPOSE || op == ACL_SPARSE_OP_TRANSPOSE ||
           op == ACL_SPARSE_OP_CONJUGATE_TRANSPOSE;
}

bool IsAcceptedAlg(aclsparseSpMMAlg_t alg)
{
    return alg == ACL_SPARSE_SPMM_ALG_DEFAULT || alg == ACL_SPARSE_SPMM_CSR_ALG1 ||
           alg == ACL_SPARSE_SPMM_CSR_ALG2 || alg == ACL_SPARSE_SPMM_CSR_ALG3 ||
           alg == ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG;
}

aclsparseStatus_t CheckInputs(const aclsparseSpMatDescr* a, const aclsparseDnMatDescr* b,
                              const aclsparseDnMatDescr* c, aclsparseOperation_t opA, aclsparseOperation_t opB,
                              aclDataType computeType, aclsparseSpMMAlg_t alg)
{
    if (a == nullptr || b == nullptr || c == nullptr) {
        ACLSP_LOGE(kApi, "matA, matB, or matC is nullptr");
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (a->signature != kSpMatSignature || b->signature != kDnMatSignature || c->signature != kDnMatSignature) {
        ACLSP_LOGE(kApi, "invalid descriptor signature");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (!IsAcceptedAlg(alg)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (!IsOperation(opA) || !IsOperation(opB)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (alg == ACL_SPARSE_SPMM_CSR_ALG3 &&
        (opA != ACL_SPARSE_OP_NON_TRANSPOSE || opB == ACL_SPARSE_OP_CONJUGATE_TRANSPOSE)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (a->format != ACL_SPARSE_FORMAT_CSR) {
        ACLSP_LOGE(kApi, "unsupported sparse matrix format %d (CSR required)", static_cast<int>(a->format));
        return ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED;
    }
    if (a->ptrType != ACL_SPARSE_INDEX_32I || a->idxType != ACL_SPARSE_INDEX_32I) {
        ACLSP_LOGE(kApi, "unsupported CSR index types (int32 required)");
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (a->baseType != ACL_SPARSE_INDEX_BASE_ZERO && a->baseType != ACL_SPARSE_INDEX_BASE_ONE) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (a->nnz > static_cast<uint64_t>(kMaxI32)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    // The reference's table (sparse/spmm/arch35/host/spmm_host.cpp:379-387) without its complex row.
    const aclDataType vt = a->valueType;
    const aclDataType ct = c->valueType;
    bool supported = vt == b->valueType;
    if (computeType == ACL_INT32) {
        supported = supported && vt == ACL_INT8 && ct == ACL_INT32;
    } else if (computeType == ACL_FLOAT) {
        supported = supported && ((vt == ACL_FLOAT && ct == ACL_FLOAT) ||
                                  (vt == ACL_FLOAT16 && (ct == ACL_FLOAT16 || ct == ACL_FLOAT)) ||
                                  (vt == ACL_BF16 && (ct == ACL_BF16 || ct == ACL_FLOAT)));
    } else {
        supported = false;
    }
    if (supported && vt != ACL_FLOAT && c->numMirrors != 0) {
        supported = false;  // mirrors of C are for fp32 products
    }
    if (!supported) {
        ACLSP_LOGE(kApi, "unsupported data type combination A=%d B=%d C=%d compute=%d",
                   static_cast<int>(a->valueType), static_cast<int>(b->valueType), static_cast<int>(c->valueType),
                   static_cast<int>(computeType));
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    // C is m x n with m = rows of op(A); op(B) is k x n.
    const uint64_t m = opA == ACL_SPARSE_OP_NON_TRANSPOSE ? a->rows : a->cols;
    const uint64_t k = opA == ACL_SPARSE_OP_NON_TRANSPOSE ? a->cols : a->rows;
    const bool bPlain = opB == ACL_SPARSE_OP_NON_TRANSPOSE;
    const int64_t bK = bPlain ? b->rows : b->cols;
    const int64_t bN = bPlain ? b->cols : b->rows;
    if (m != static_cast<uint64_t>(c->rows) || k != static_cast<uint64_t>(bK) || bN != c->cols) {
        ACLSP_LOGE(kApi, "matrix dimensions do not match");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (a->rows == 0 || a->cols == 0 || c->cols == 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (a->rows > static_cast<uint64_t>(kMaxI32) || a->cols > static_cast<uint64_t>(kMaxI32) || b->rows > kMaxI32 ||
        b->cols > kMaxI32 || b->ld > kMaxI32 || c->rows > kMaxI32 || c->cols > kMaxI32 || c->ld > kMaxI32) {
        ACLSP_LOGE(kApi, "matrix dimension or leading dimension exceeds INT32_MAX");
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if ((a->rows > 0 && a->ptrs == nullptr) || (a->nnz > 0 && (a->idxs == nullptr || a->values == nullptr)) ||
        (b->rows > 0 && b->cols > 0 && b->values == nullptr) || (c->rows > 0 && c->cols > 0 && c->values == nullptr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const int64_t bLd = b->order == ACL_SPARSE_ORDER_ROW ? b->cols : b->rows;
    const int64_t cLd = c->order == ACL_SPARSE_ORDER_ROW ? c->cols : c->rows;
    if (b->ld < bLd || c->ld < cLd) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (a->ptrStride != 1 || a->idxStride != 1 || a->valueStride != 1) {
        ACLSP_LOGE(kApi, "strided CSR arrays are not supported by SpMM");
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// handle and scalar checks shared by the three entry points
aclsparseStatus_t CheckCall(aclsparseHandle_t handle, const void* alpha, const void* beta)
{
    if (handle == nullptr) {
        ACLSP_LOGE(kApi, "handle is nullptr");
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (alpha == nullptr || beta == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (handle->signature != kHandleSignature) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t CheckBuffer(const void* buffer)
{
    if (buffer == nullptr) {
        ACLSP_LOGE(kApi, "buffer is nullptr");
        return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
    }
    if (reinterpret_cast<uintptr_t>(buffer) % ACLSP_WS_ALIGN != 0) {
        ACLSP_LOGE(kApi, "buffer=%p; expected 64-byte alignment", buffer);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// Size and offsets of what the external buffer holds: the plan of A, or for op(A) = transpose the plan of
// the transposed matrix followed by the transpose itself.
uint64_t BufferLayout(const aclsparseSpMatDescr* a, uint64_t denseCols, bool transposed, AclspTransposeLayout* tl)
{
    AclspPlanLayout layout;
    if (!transposed) {
        aclspSpmmLayout(a->rows, a->nnz, denseCols, &layout);
        return layout.totalBytes;
    }
    aclspSpmmLayout(a->cols, a->nnz, denseCols, &layout);
    aclspTransposeLayout(a->cols, a->nnz, layout.totalBytes, tl);
    return tl->totalBytes;
}

bool PlanMatches(const aclsparseSpMatDescr* a, uint64_t denseCols, const void* buffer, const aclsparseContext* h,
                 bool transposed)
{
    const SpmmPlanRecord& p = a->spmm;
    if (p.transposed != transposed || (transposed && p.colIndices != a->idxs)) {
        return false;
    }
    // Only a plan from an explicit Preprocess call is reused, and only while no later plan build (of this
    // or any other descriptor, SpMM or SpMV) went into the same buffer.
    return a->activeBuffer == buffer && p.buffer == buffer && p.fromPreprocess && AclspPlanIsCurrent(buffer, p.serial) &&
           p.rowOffsets == a->ptrs && p.rows == a->rows &&
           p.cols == a->cols && p.nnz == a->nnz && p.denseCols == denseCols && p.base == a->baseType &&
           p.stream == h->stream && p.streamEpoch == h->streamEpoch && p.ownerId == a->workspaceOwnerId;
}

aclsparseStatus_t BuildPlan(aclsparseContext* h, aclsparseSpMatDescr* a, uint64_t denseCols, void* buffer,
                            bool fromPreprocess, bool transposed)
{
    (void)cudaGetLastError();
    if (transposed) {
        // The transpose first (its row offsets land where a plan keeps them), then the plan of the
        // transposed matrix over those offsets, in place.
        AclspTransposeLayout tl;
        (void)BufferLayout(a, denseCols, true, &tl);
        aclsp_b200_transpose_build_kernel_do(a->ptrs, a->idxs, static_cast<uint32_t>(a->rows),
                                             static_cast<uint32_t>(a->cols), static_cast<uint32_t>(a->nnz),
                                             static_cast<int32_t>(a->baseType), 1, 1, buffer, &tl, h->stream);
        spmm_b200_preprocess_kernel_do(static_cast<const unsigned char*>(buffer) + tl.rowPtrOff, buffer,
                                       static_cast<uint32_t>(a->cols), static_cast<uint32_t>(a->rows),
                                       static_cast<uint32_t>(a->nnz), static_cast<uint32_t>(denseCols), 0, h->stream);
    } else {
        spmm_b200_preprocess_kernel_do(a->ptrs, buffer, static_cast<uint32_t>(a->rows),
                                       static_cast<uint32_t>(a->cols), static_cast<uint32_t>(a->nnz),
                                       static_cast<uint32_t>(denseCols), static_cast<int32_t>(a->baseType), h->stream);
    }
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        ACLSP_LOGE(kApi, "preprocess enqueue failed: %s", cudaGetErrorString(err));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    SpmmPlanRecord& p = a->spmm;
    p.serial = AclspPublishPlan(buffer);
    p.fromPreprocess = fromPreprocess;
    p.buffer = buffer;
    p.transposed = transposed;
    p.colIndices = a->idxs;
    p.rowOffsets = a->ptrs;
    p.rows = a->rows;
    p.cols = a->cols;
    p.nnz = a->nnz;
    p.denseCols = denseCols;
    p.base = a->baseType;
    p.stream = h->stream;
    p.streamEpoch = h->streamEpoch;
    p.ownerId = a->workspaceOwnerId;
    a->activeBuffer = buffer;
    // The allocation now holds SpMM metadata: an SpMV plan in it is gone.
    if (a->spmv.buffer == buffer) {
        a->spmv.buffer = nullptr;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

extern "C" aclsparseStatus_t aclsparseSpMMGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                                        aclsparseOperation_t opB, const void* alpha,
                                                        aclsparseConstSpMatDescr_t matA,
                                                        aclsparseConstDnMatDescr_t matB, const void* beta,
                                                        aclsparseDnMatDescr_t matC, aclDataType computeType,
                                                        aclsparseSpMMAlg_t alg, size_t* size)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (size == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    aclsparseStatus_t st = CheckCall(handle, alpha, beta);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckInputs(matA, matB, matC, opA, opB, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    AclspTransposeLayout tl;
    *size = static_cast<size_t>(BufferLayout(matA, static_cast<uint64_t>(matC->cols),
                                             opA != ACL_SPARSE_OP_NON_TRANSPOSE, &tl));
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                                     aclsparseOperation_t opB, const void* alpha,
                                                     aclsparseConstSpMatDescr_t matA,
                                                     aclsparseConstDnMatDescr_t matB, const void* beta,
                                                     aclsparseDnMatDescr_t matC, aclDataType computeType,
                                                     aclsparseSpMMAlg_t alg, void* buffer)
{
    aclsparseStatus_t st = CheckCall(handle, alpha, beta);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckInputs(matA, matB, matC, opA, opB, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckBuffer(buffer);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    return BuildPlan(handle, const_cast<aclsparseSpMatDescr*>(matA), static_cast<uint64_t>(matC->cols), buffer, true,
                     opA != ACL_SPARSE_OP_NON_TRANSPOSE);
}

extern "C" aclsparseStatus_t aclsparseSpMM(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                           aclsparseOperation_t opB, const void* alpha,
                                           aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                           const void* beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                           aclsparseSpMMAlg_t alg, void* buffer)
{
    aclsparseStatus_t st = CheckCall(handle, alpha, beta);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckInputs(matA, matB, matC, opA, opB, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckBuffer(buffer);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    auto* a = const_cast<aclsparseSpMatDescr*>(matA);
    const uint64_t n = static_cast<uint64_t>(matC->cols);
    // Preprocess is optional: without a matching plan in this buffer it is
    // built here, on the same stream, ahead of the product.
    const bool transposed = opA != ACL_SPARSE_OP_NON_TRANSPOSE;
    if (!PlanMatches(a, n, buffer, handle, transposed)) {
        st = BuildPlan(handle, a, n, buffer, false, transposed);
        if (st != ACL_SPARSE_STATUS_SUCCESS) {
            return st;
        }
    }

    (void)cudaGetLastError();  // an enqueue failure below is this call's
    AclspSpmmParams params{};
    const void* colInd = a->idxs;
    const void* values = a->values;
    params.rows = static_cast<uint32_t>(a->rows);
    params.cols = static_cast<uint32_t>(a->cols);
    params.nnz = static_cast<uint32_t>(a->nnz);
    params.indexBase = static_cast<uint32_t>(a->baseType);
    if (transposed) {
        // The product runs on the transposed matrix in the buffer: base 0, its values gathered from the
        // caller's through the permutation, now, so that they are the current ones.
        AclspTransposeLayout tl;
        (void)BufferLayout(a, n, true, &tl);
        aclsp_b200_transpose_values_kernel_do(a->values, 1, static_cast<uint32_t>(a->cols),
                                              static_cast<uint32_t>(a->nnz), buffer, &tl,
                                              a->valueType == ACL_INT8 ? 1u : (a->valueType == ACL_FLOAT ? 4u : 2u),
                                              handle->stream);
        colInd = static_cast<const unsigned char*>(buffer) + tl.colIndOff;
        values = static_cast<const unsigned char*>(buffer) + tl.valuesOff;
        params.rows = static_cast<uint32_t>(a->cols);
        params.cols = static_cast<uint32_t>(a->rows);
        params.indexBase = 0;
    }
    params.n = static_cast<uint32_t>(n);
    params.opB = opB == ACL_SPARSE_OP_NON_TRANSPOSE ? 0u : 1u;  // real data: H is T
    params.orderB = static_cast<uint32_t>(matB->order);
    params.orderC = static_cast<uint32_t>(matC->order);
    params.highPrecision = alg == ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG ? 1u : 0u;
    params.ldb = matB->ld;
    params.ldc = matC->ld;
    auto kernelType = [](aclDataType t) {
        return t == ACL_FLOAT16 ? ACLSP_TYPE_F16
               : t == ACL_BF16  ? ACLSP_TYPE_BF16
               : t == ACL_INT8  ? ACLSP_TYPE_I8
               : t == ACL_INT32 ? ACLSP_TYPE_I32
                                : ACLSP_TYPE_F32;
    };
    params.valueType = kernelType(a->valueType);
    params.cType = kernelType(matC->valueType);
    params.computeInt = computeType == ACL_INT32 ? 1u : 0u;
    if (handle->pointerMode == ACL_SPARSE_POINTER_MODE_DEVICE) {
        params.alphaPtr = static_cast<const float*>(alpha);  // int32 on the device when computeInt
        params.betaPtr = static_cast<const float*>(beta);
    } else if (params.computeInt != 0) {
        params.alphaInt = *static_cast<const int32_t*>(alpha);
        params.betaInt = *static_cast<const int32_t*>(beta);
    } else {
        params.alpha = *static_cast<const float*>(alpha);
        params.beta = *static_cast<const float*>(beta);
    }
    if (params.valueType == ACLSP_TYPE_F32) {
        params.barrier = matC->barrier;
    }
    params.numMirrors = static_cast<uint32_t>(matC->numMirrors);
    params.mirrorMulticast = matC->mirrorMulticast ? 1u : 0u;
    for (int m = 0; m < matC->numMirrors; ++m) {
        params.mirrorDelta[m] = static_cast<const char*>(matC->mirrors[m]) - static_cast<const char*>(matC->values);
        if (params.mirrorDelta[m] % 4 != 0) {
            ACLSP_LOGE(kApi, "mirror %d is not aligned like the output", m);
            return ACL_SPARSE_STATUS_INVALID_VALUE;
        }
    }

    spmm_b200_kernel_do(colInd, values, matB->values, matC->values, buffer, &params, handle->stream);
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        ACLSP_LOGE(kApi, "kernel enqueue failed: %s", cudaGetErrorString(err));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}
