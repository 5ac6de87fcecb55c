/*
 * Host layer of aclsparseSpMV: validation, buffer sizing, plan bookkeeping and
 * the calls into the CUDA launch shim.  The order of the checks, and therefore
 * which status a bad call gets, follows the reference's
 * sparse/spmv/arch35/spmv_host.cpp (descriptor set-up :165-200, matrix
 * metadata :220-294, vector sizes :315-329, storage :331-355, workspace
 * :357-368, three entry points :526-678).
 *
 * Differences that a caller can observe:
 *  - op(A) = transpose (and conjugate transpose, the same thing for real data) builds the transposed
 *    matrix in the external buffer during preprocessing and multiplies with it: the buffer is much
 *    larger (about 12 bytes per non-zero) and the result is bit-reproducible for every algorithm value;
 *  - the complex dtype combinations of the reference's table (spmv_host.cpp:44-66) are answered with
 *    NOT_SUPPORTED; the others (fp32, fp16 / bf16 storage with a result of the same type or fp32, int8 with
 *    an fp32 or a saturating int32 result) are computed;
 *  - the buffer size covers the B200 plan (row offsets + tile splits + row
 *    bins + carries), so it is larger than the reference's for the same matrix.
 */
#include <cstdint>
#include <limits>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "internal.h"
#include "plan_layout.h"

namespace {

constexpr const char* kApi = "aclsparseSpMV";

bool IsTranspose(aclsparseOperation_t op)
{
    return op == ACL_SPARSE_OP_TRANSPOSE || op == ACL_SPARSE_OP_CONJUGATE_TRANSPOSE;
}

bool IsAcceptedAlg(aclsparseSpMVAlg_t alg)
{
    return alg == ACL_SPARSE_SPMV_ALG_DEFAULT || alg == ACL_SPARSE_SPMV_CSR_ALG1 ||
           alg == ACL_SPARSE_SPMV_CSR_ALG2;
}

bool IsScalarComputeType(aclDataType t)
{
    return t == ACL_INT32 || t == ACL_FLOAT || t == ACL_COMPLEX64;
}

size_t ScalarAlignment(aclDataType computeType)
{
    switch (computeType) {
        case ACL_INT32:
            return alignof(int32_t);
        case ACL_COMPLEX64:
            return alignof(aclsparseComplex);
        case ACL_FLOAT:
            return alignof(float);
        default:
            return 0;
    }
}

uint32_t KernelType(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT16:
            return ACLSP_TYPE_F16;
        case ACL_BF16:
            return ACLSP_TYPE_BF16;
        case ACL_INT8:
            return ACLSP_TYPE_I8;
        case ACL_INT32:
            return ACLSP_TYPE_I32;
        default:
            return ACLSP_TYPE_F32;
    }
}

size_t ElementBytes(aclDataType t)
{
    return t == ACL_INT8 ? 1u : (t == ACL_FLOAT16 || t == ACL_BF16) ? 2u : t == ACL_COMPLEX64 ? 8u : 4u;
}

bool StrideFits(uint64_t length, int64_t stride, size_t elementBytes)
{
    if (stride <= 0 || elementBytes == 0) {
        return false;
    }
    const uint64_t maxOffset = static_cast<uint64_t>(std::numeric_limits<int64_t>::max()) / elementBytes;
    return length <= 1u || static_cast<uint64_t>(stride) <= maxOffset / (length - 1u);
}

aclsparseStatus_t CheckHandle(aclsparseHandle_t handle)
{
    if (handle == nullptr) {
        ACLSP_LOGE(kApi, "handle must be non-null");
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (handle->signature != kHandleSignature) {
        ACLSP_LOGE(kApi, "invalid handle signature");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (handle->stream == nullptr) {
        ACLSP_LOGE(kApi, "handle stream must be set before use");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t CheckSetup(aclsparseHandle_t handle, aclsparseOperation_t opA, const void* alpha,
                             const aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x, const void* beta,
                             const aclsparseDnVecDescr* y, aclDataType computeType, aclsparseSpMVAlg_t alg)
{
    aclsparseStatus_t st = CheckHandle(handle);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (mat == nullptr || x == nullptr || y == nullptr || mat->signature != kSpMatSignature ||
        x->signature != kDnVecSignature || y->signature != kDnVecSignature) {
        ACLSP_LOGE(kApi, "matrix and vector descriptors must be valid and non-null");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (opA != ACL_SPARSE_OP_NON_TRANSPOSE && !IsTranspose(opA)) {
        ACLSP_LOGE(kApi, "op=%d; expected N/T/H", static_cast<int>(opA));
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (!IsScalarComputeType(computeType) || !IsAcceptedAlg(alg)) {
        ACLSP_LOGE(kApi, "computeType=%d alg=%d not supported", static_cast<int>(computeType),
                   static_cast<int>(alg));
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (handle->pointerMode != ACL_SPARSE_POINTER_MODE_HOST && handle->pointerMode != ACL_SPARSE_POINTER_MODE_DEVICE) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (alpha == nullptr || beta == nullptr) {
        ACLSP_LOGE(kApi, "alpha and beta must be non-null");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const size_t alignment = ScalarAlignment(computeType);
    if (alignment == 0 || reinterpret_cast<uintptr_t>(alpha) % alignment != 0 ||
        reinterpret_cast<uintptr_t>(beta) % alignment != 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t CheckMatrix(const aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x,
                              const aclsparseDnVecDescr* y, aclsparseOperation_t opA, aclDataType computeType)
{
    if (mat->format != ACL_SPARSE_FORMAT_CSR || mat->ptrType != ACL_SPARSE_INDEX_32I ||
        mat->idxType != ACL_SPARSE_INDEX_32I ||
        (mat->baseType != ACL_SPARSE_INDEX_BASE_ZERO && mat->baseType != ACL_SPARSE_INDEX_BASE_ONE)) {
        ACLSP_LOGE(kApi, "format=%d rowIndexType=%d colIndexType=%d base=%d; expected CSR, int32, base 0/1",
                   static_cast<int>(mat->format), static_cast<int>(mat->ptrType), static_cast<int>(mat->idxType),
                   static_cast<int>(mat->baseType));
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (mat->nnz > 0 && (mat->rows == 0 || mat->cols == 0)) {
        ACLSP_LOGE(kApi, "zero dimensions require nnz=0");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    // Row offsets and column indices are signed 32-bit on the device; a
    // one-based CSR needs one more representable value for the last offset.
    const uint64_t maxI32 = static_cast<uint64_t>(std::numeric_limits<int32_t>::max());
    const uint64_t baseOffset = mat->baseType == ACL_SPARSE_INDEX_BASE_ONE ? 1u : 0u;
    if (mat->rows > maxI32 || mat->cols > maxI32 || mat->nnz > maxI32 - baseOffset) {
        ACLSP_LOGE(kApi, "rows/cols/nnz must fit a signed 32-bit index");
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    // Repeated coordinates are legal, so nnz is not bounded by rows*cols.
    // The reference's table (sparse/spmv/arch35/spmv_host.cpp:44-66) without its complex rows.
    const aclDataType vt = mat->valueType;
    const aclDataType yt = y->valueType;
    bool supported = vt == x->valueType;
    if (computeType == ACL_INT32) {
        supported = supported && vt == ACL_INT8 && yt == ACL_INT32;
    } else if (computeType == ACL_FLOAT) {
        supported = supported && ((vt == ACL_FLOAT && yt == ACL_FLOAT) || (vt == ACL_INT8 && yt == ACL_FLOAT) ||
                                  (vt == ACL_FLOAT16 && (yt == ACL_FLOAT16 || yt == ACL_FLOAT)) ||
                                  (vt == ACL_BF16 && (yt == ACL_BF16 || yt == ACL_FLOAT)));
    } else {
        supported = false;
    }
    if (!supported) {
        ACLSP_LOGE(kApi, "unsupported dtype combination A=%d x=%d y=%d compute=%d",
                   static_cast<int>(mat->valueType), static_cast<int>(x->valueType),
                   static_cast<int>(y->valueType), static_cast<int>(computeType));
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (vt != ACL_FLOAT && y->numMirrors != 0) {
        ACLSP_LOGE(kApi, "mirrors of y are for fp32 products");
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    (void)opA;
    if (!StrideFits(mat->rows + 1u, mat->ptrStride, sizeof(int32_t)) ||
        !StrideFits(mat->nnz, mat->idxStride, sizeof(int32_t)) ||
        !StrideFits(mat->nnz, mat->valueStride, ElementBytes(mat->valueType)) ||
        !StrideFits(x->nums, x->stride, ElementBytes(x->valueType)) ||
        !StrideFits(y->nums, y->stride, ElementBytes(y->valueType))) {
        ACLSP_LOGE(kApi, "strides must be positive and addressable");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// Everything GetBufferSize checks: descriptors and metadata only, so data
// pointers may still be unbound.
aclsparseStatus_t CheckInputs(aclsparseHandle_t handle, aclsparseOperation_t opA, const void* alpha,
                              const aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x, const void* beta,
                              const aclsparseDnVecDescr* y, aclDataType computeType, aclsparseSpMVAlg_t alg)
{
    aclsparseStatus_t st = CheckSetup(handle, opA, alpha, mat, x, beta, y, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckMatrix(mat, x, y, opA, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    const uint64_t xRequired = IsTranspose(opA) ? mat->rows : mat->cols;
    const uint64_t yRequired = IsTranspose(opA) ? mat->cols : mat->rows;
    if (x->nums != xRequired || y->nums != yRequired) {
        ACLSP_LOGE(kApi, "vector sizes x=%llu y=%llu; expected x=%llu y=%llu",
                   static_cast<unsigned long long>(x->nums), static_cast<unsigned long long>(y->nums),
                   static_cast<unsigned long long>(xRequired), static_cast<unsigned long long>(yRequired));
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// y is updated in place while A and x are only read, so none of the five
// arrays may start at the same address.
bool HasAliases(const aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x, const aclsparseDnVecDescr* y)
{
    const void* p[5] = {mat->ptrs, mat->idxs, mat->values, x->values, y->values};
    for (int i = 0; i < 5; ++i) {
        for (int j = i + 1; j < 5; ++j) {
            if (p[i] != nullptr && p[i] == p[j]) {
                return true;
            }
        }
    }
    return false;
}

aclsparseStatus_t CheckStorage(const aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x,
                               const aclsparseDnVecDescr* y)
{
    if ((mat->rows > 0 && mat->ptrs == nullptr) || (mat->nnz > 0 && (mat->idxs == nullptr || mat->values == nullptr)) ||
        (x->nums > 0 && x->values == nullptr) || (y->nums > 0 && y->values == nullptr)) {
        ACLSP_LOGE(kApi, "required storage is unbound");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (HasAliases(mat, x, y)) {
        ACLSP_LOGE(kApi, "CSR, x and y storage must not alias");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t CheckWorkspace(const void* buffer)
{
    if (buffer == nullptr) {
        ACLSP_LOGE(kApi, "workspace must be allocated with the size from GetBufferSize");
        return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
    }
    if (reinterpret_cast<uintptr_t>(buffer) % ACLSP_WS_ALIGN != 0) {
        ACLSP_LOGE(kApi, "workspace=%p; expected 64-byte alignment", buffer);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// Size and offsets of what the external buffer holds: the plan of A, or for op(A) = transpose the plan of
// the transposed matrix followed by the transpose itself.
uint64_t BufferLayout(const aclsparseSpMatDescr* mat, bool transposed, AclspTransposeLayout* tl)
{
    AclspPlanLayout layout;
    if (!transposed) {
        aclspSpmvLayout(mat->rows, mat->nnz, &layout);
        return layout.totalBytes;
    }
    aclspSpmvLayout(mat->cols, mat->nnz, &layout);
    aclspTransposeLayout(mat->cols, mat->nnz, layout.totalBytes, tl);
    return tl->totalBytes;
}

bool PlanMatches(const aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x, const aclsparseDnVecDescr* y,
                 aclsparseOperation_t opA, aclDataType computeType, aclsparseSpMVAlg_t alg, const void* buffer,
                 const aclsparseContext* h)
{
    // Only a plan from an explicit Preprocess call is reused, and only while no later plan build (of this
    // or any other descriptor, SpMV or SpMM) went into the same buffer.
    const SpmvPlanRecord& p = mat->spmv;
    return buffer != nullptr && p.buffer == buffer && p.fromPreprocess && AclspPlanIsCurrent(buffer, p.serial) &&
           mat->activeBuffer != buffer && p.rowOffsets == mat->ptrs &&
           p.colIndices == mat->idxs && p.values == mat->values && p.rowOffsetsStride == mat->ptrStride &&
           p.colIndStride == mat->idxStride && p.valuesStride == mat->valueStride && p.xStride == x->stride &&
           p.yStride == y->stride && p.rows == mat->rows && p.cols == mat->cols && p.nnz == mat->nnz &&
           p.base == mat->baseType && p.valueType == mat->valueType && p.xType == x->valueType &&
           p.yType == y->valueType && p.computeType == computeType && p.op == opA &&
           p.alg == static_cast<int32_t>(alg) && p.stream == h->stream && p.streamEpoch == h->streamEpoch;
}

void RecordPlan(aclsparseSpMatDescr* mat, const aclsparseDnVecDescr* x, const aclsparseDnVecDescr* y,
                aclsparseOperation_t opA, aclDataType computeType, aclsparseSpMVAlg_t alg, const void* buffer,
                const aclsparseContext* h, bool fromPreprocess)
{
    SpmvPlanRecord& p = mat->spmv;
    p.serial = AclspPublishPlan(buffer);
    p.fromPreprocess = fromPreprocess;
    p.buffer = buffer;
    p.rowOffsets = mat->ptrs;
    p.colIndices = mat->idxs;
    p.values = mat->values;
    p.rowOffsetsStride = mat->ptrStride;
    p.colIndStride = mat->idxStride;
    p.valuesStride = mat->valueStride;
    p.xStride = x->stride;
    p.yStride = y->stride;
    p.rows = mat->rows;
    p.cols = mat->cols;
    p.nnz = mat->nnz;
    p.base = mat->baseType;
    p.valueType = mat->valueType;
    p.xType = x->valueType;
    p.yType = y->valueType;
    p.computeType = computeType;
    p.op = opA;
    p.alg = static_cast<int32_t>(alg);
    p.stream = h->stream;
    p.streamEpoch = h->streamEpoch;
}

// Enqueues the plan-building kernels.  An enqueue failure is attributed to
// this launch only: the sticky-free last error is cleared first, then peeked.
aclsparseStatus_t LaunchPreprocess(const aclsparseContext* h, aclsparseSpMatDescr* mat, void* buffer, bool transposed)
{
    (void)cudaGetLastError();
    if (transposed) {
        // The transpose first (its row offsets land where a plan keeps them), then the plan of the
        // transposed matrix over those offsets, in place.
        AclspTransposeLayout tl;
        (void)BufferLayout(mat, true, &tl);
        aclsp_b200_transpose_build_kernel_do(mat->ptrs, mat->idxs, static_cast<uint32_t>(mat->rows),
                                             static_cast<uint32_t>(mat->cols), static_cast<uint32_t>(mat->nnz),
                                             static_cast<int32_t>(mat->baseType), mat->ptrStride, mat->idxStride,
                                             buffer, &tl, h->stream);
        spmv_b200_preprocess_kernel_do(static_cast<const unsigned char*>(buffer) + tl.rowPtrOff, buffer,
                                       static_cast<uint32_t>(mat->cols), static_cast<uint32_t>(mat->rows),
                                       static_cast<uint32_t>(mat->nnz), 0, 1, h->stream);
    } else {
        spmv_b200_preprocess_kernel_do(mat->ptrs, buffer, static_cast<uint32_t>(mat->rows),
                                       static_cast<uint32_t>(mat->cols), static_cast<uint32_t>(mat->nnz),
                                       static_cast<int32_t>(mat->baseType), mat->ptrStride, h->stream);
    }
    // The longest row, which the pass has just written into the plan header, is sent to pinned host
    // memory in stream order; products look there to pick their kernel and never wait for it.
    mat->spmv.longestRow = AclspAcquireHostSlot();
    if (mat->spmv.longestRow.word != nullptr) {
        (void)cudaMemcpyAsync(mat->spmv.longestRow.word,
                              static_cast<const unsigned char*>(buffer) + ACLSP_HEADER_MAX_ROW_LEN_OFF, sizeof(uint32_t),
                              cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(h->stream));
    }
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        ACLSP_LOGE(kApi, "preprocess enqueue failed: %s", cudaGetErrorString(err));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

extern "C" aclsparseStatus_t aclsparseSpMVGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                                        const void* alpha, aclsparseConstSpMatDescr_t matA,
                                                        aclsparseConstDnVecDescr_t vecX, const void* beta,
                                                        aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                                        aclsparseSpMVAlg_t alg, size_t* bufferSize)
{
    if (bufferSize == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *bufferSize = 0;
    const aclsparseStatus_t st = CheckInputs(handle, opA, alpha, matA, vecX, beta, vecY, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    AclspTransposeLayout tl;
    *bufferSize = static_cast<size_t>(BufferLayout(matA, IsTranspose(opA), &tl));
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMVPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                                     const void* alpha, aclsparseConstSpMatDescr_t matA,
                                                     aclsparseConstDnVecDescr_t vecX, const void* beta,
                                                     aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                                     aclsparseSpMVAlg_t alg, void* externalBuffer)
{
    aclsparseStatus_t st = CheckInputs(handle, opA, alpha, matA, vecX, beta, vecY, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    auto* mat = const_cast<aclsparseSpMatDescr*>(matA);
    // Preprocessing reads the row offsets only (and, to build a transpose, the column indices);
    // values and vectors may be bound later.
    if ((mat->rows > 0 && mat->ptrs == nullptr) || (IsTranspose(opA) && mat->nnz > 0 && mat->idxs == nullptr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    st = CheckWorkspace(externalBuffer);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    // The buffer is about to hold SpMV metadata: an SpMM plan cached for the
    // same allocation is gone.
    if (mat->activeBuffer == externalBuffer) {
        mat->activeBuffer = nullptr;
    }
    if (vecY->nums > 0) {
        st = LaunchPreprocess(handle, mat, externalBuffer, IsTranspose(opA));
        if (st != ACL_SPARSE_STATUS_SUCCESS) {
            return st;
        }
    }
    RecordPlan(mat, vecX, vecY, opA, computeType, alg, externalBuffer, handle, true);
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMV(aclsparseHandle_t handle, aclsparseOperation_t opA, const void* alpha,
                                           aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                           const void* beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                           aclsparseSpMVAlg_t alg, void* externalBuffer)
{
    aclsparseStatus_t st = CheckInputs(handle, opA, alpha, matA, vecX, beta, vecY, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    auto* mat = const_cast<aclsparseSpMatDescr*>(matA);
    st = CheckStorage(mat, vecX, vecY);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = CheckWorkspace(externalBuffer);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (vecY->nums == 0) {  // nothing to write
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    const bool transposed = IsTranspose(opA);
    // Preprocess is optional.  Without a matching plan from a Preprocess call in this buffer the
    // plan is (re)built here, on the same stream and ahead of the product (a few O(rows) kernels),
    // so that a caller who never preprocesses, or who let another operator or another matrix
    // overwrite the buffer, still gets the product of the descriptor's current arrays.
    if (!PlanMatches(mat, vecX, vecY, opA, computeType, alg, externalBuffer, handle)) {
        if (mat->activeBuffer == externalBuffer) {
            mat->activeBuffer = nullptr;
        }
        st = LaunchPreprocess(handle, mat, externalBuffer, transposed);
        if (st != ACL_SPARSE_STATUS_SUCCESS) {
            return st;
        }
        RecordPlan(mat, vecX, vecY, opA, computeType, alg, externalBuffer, handle, false);
    }

    (void)cudaGetLastError();  // an enqueue failure below is this call's
    AclspSpmvParams params{};
    const void* colInd = mat->idxs;
    const void* values = mat->values;
    params.rows = static_cast<uint32_t>(mat->rows);
    params.cols = static_cast<uint32_t>(mat->cols);
    params.nnz = static_cast<uint32_t>(mat->nnz);
    params.indexBase = static_cast<uint32_t>(mat->baseType);
    params.colIndStride = mat->idxStride;
    params.valuesStride = mat->valueStride;
    if (transposed) {
        // The product runs on the transposed matrix in the buffer: base 0, unit strides, its values
        // gathered from the caller's through the permutation, now, so that they are the current ones.
        AclspTransposeLayout tl;
        (void)BufferLayout(mat, true, &tl);
        aclsp_b200_transpose_values_kernel_do(mat->values, mat->valueStride, static_cast<uint32_t>(mat->cols),
                                              static_cast<uint32_t>(mat->nnz), externalBuffer, &tl,
                                              static_cast<uint32_t>(ElementBytes(mat->valueType)), handle->stream);
        colInd = static_cast<const unsigned char*>(externalBuffer) + tl.colIndOff;
        values = static_cast<const unsigned char*>(externalBuffer) + tl.valuesOff;
        params.rows = static_cast<uint32_t>(mat->cols);
        params.cols = static_cast<uint32_t>(mat->rows);
        params.indexBase = 0;
        params.colIndStride = 1;
        params.valuesStride = 1;
    }
    params.xStride = vecX->stride;
    params.yStride = vecY->stride;
    params.valueType = KernelType(mat->valueType);
    params.yType = KernelType(vecY->valueType);
    params.computeInt = computeType == ACL_INT32 ? 1u : 0u;
    if (handle->pointerMode == ACL_SPARSE_POINTER_MODE_DEVICE) {
        // The host never dereferences device scalars; the kernels read them (as int32 when computeInt).
        params.alphaPtr = static_cast<const float*>(alpha);
        params.betaPtr = static_cast<const float*>(beta);
    } else if (params.computeInt != 0) {
        params.alphaInt = *static_cast<const int32_t*>(alpha);
        params.betaInt = *static_cast<const int32_t*>(beta);
    } else {
        params.alpha = *static_cast<const float*>(alpha);
        params.beta = *static_cast<const float*>(beta);
    }
    params.maxRowLenHint = ACLSP_MAX_ROW_LEN_UNKNOWN;
    uint32_t longest = 0;
    if (AclspHostSlotValue(mat->spmv.longestRow, &longest)) {
        params.maxRowLenHint = longest;
    }
    if (params.valueType == ACLSP_TYPE_F32) {
        params.barrier = vecY->barrier;
    }
    params.numMirrors = static_cast<uint32_t>(vecY->numMirrors);
    params.mirrorMulticast = vecY->mirrorMulticast ? 1u : 0u;
    for (int m = 0; m < vecY->numMirrors; ++m) {
        params.mirrorDelta[m] = static_cast<const char*>(vecY->mirrors[m]) - static_cast<const char*>(vecY->values);
        if (params.mirrorDelta[m] % 4 != 0) {
            ACLSP_LOGE(kApi, "mirror %d is not aligned like the output", m);
            return ACL_SPARSE_STATUS_INVALID_VALUE;
        }
    }

    spmv_b200_kernel_do(colInd, values, vecX->values, vecY->values, externalBuffer, &params, handle->stream);
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        ACLSP_LOGE(kApi, "kernel enqueue failed: %s", cudaGetErrorString(err));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}
