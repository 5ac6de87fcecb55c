/*
 * The plan API: aclsparseSpMVOp_* and aclsparseSpMMOp_* (create once, execute many).
 *
 *   bufferSize -> createDescr (binds A, preprocesses into the caller's buffer)
 *              -> createPlan -> [setGlobalUserData] -> execute ... -> destroyPlan -> destroyDescr
 *
 * SpMVOp computes Z = alpha*A*X + beta*Y into a vector of its own; SpMMOp computes
 * C = alpha*A*op(B) + beta*C with B and C handed over at every execute.  Both run the kernels of
 * aclsparseSpMV / aclsparseSpMM over a plan that lives in the caller's buffer, so every algorithm
 * value is deterministic (fixed summation order, no atomics: the bit-wise reproducibility the
 * reference promises, include/cann_ops_sparse.h:2391-2393) and sums in fp64.
 *
 * The order of the checks, and therefore which status a bad call gets, follows the reference's
 * sparse/spmv_op/arch35/spmv_op_host.cpp (validation :66-298, entry points :520-772) and
 * sparse/spmm_op/arch35/spmm_op_host.cpp.  Differences a caller can observe:
 *  - every algorithm value needs the buffer (the reference's ALG1 needs none and reports size 0): the
 *    size query says how much, createDescr answers INVALID_VALUE when it gets no buffer;
 *  - row offsets must be int32 (the reference also takes int64 row offsets here);
 *  - new values (aclsparseSpMatSetValues / writing into the bound array) are picked up by the next
 *    execute under every algorithm value, because the plan depends on the structure of A only;
 *  - SpMMOp: the buffer is sized for the width of the C given to bufferSize / createDescr; an execute
 *    with a wider C is answered with INVALID_VALUE.
 */
#include <cstdint>
#include <limits>
#include <new>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "internal.h"
#include "plan_layout.h"

// What createDescr copies out of the matrix descriptor: the CSR arrays stay the caller's.
struct aclsparseSpMVOpDescr {
    uint32_t signature = 0x53564F44u;  // "SVOD"
    uint64_t m = 0;
    uint64_t n = 0;
    uint64_t nnz = 0;
    const void* rowOffsets = nullptr;
    const void* colIndices = nullptr;
    const void* values = nullptr;
    aclsparseConstSpMatDescr_t mat = nullptr;  // values are re-read from it at execute (SetValues)
    aclsparseIndexBase_t base = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseSpMVOpAlg_t alg = ACL_SPARSE_SPMVOP_ALG1;
    void* buffer = nullptr;
    AclspHostSlot longestRow;
};

struct aclsparseSpMVOpPlan {
    uint32_t signature = 0x53564F50u;  // "SVOP"
    aclsparseSpMVOpDescr* descr = nullptr;
};

struct aclsparseSpMMOpDescr {
    uint32_t signature = 0x534D4F44u;  // "SMOD"
    uint64_t m = 0;
    uint64_t k = 0;
    uint64_t nnz = 0;
    uint64_t maxDenseCols = 0;  // the buffer's carry area holds rows of C this wide
    const void* rowOffsets = nullptr;
    const void* colIndices = nullptr;
    aclsparseConstSpMatDescr_t mat = nullptr;
    aclsparseIndexBase_t base = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseOperation_t opB = ACL_SPARSE_OP_NON_TRANSPOSE;
    aclsparseSpMMOpAlg_t alg = ACL_SPARSE_SPMMOP_ALG1;
    void* buffer = nullptr;
};

struct aclsparseSpMMOpPlan {
    uint32_t signature = 0x534D4F50u;  // "SMOP"
    aclsparseSpMMOpDescr* descr = nullptr;
};

namespace {

constexpr const char* kVTag = "aclsparseSpMVOp";
constexpr const char* kMTag = "aclsparseSpMMOp";
constexpr uint64_t kMaxI32 = static_cast<uint64_t>(std::numeric_limits<int32_t>::max());

aclsparseStatus_t ValidateMatrix(const char* tag, aclsparseConstSpMatDescr_t a)
{
    if (a == nullptr) {
        ACLSP_LOGE(tag, "matA is nullptr");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (a->format != ACL_SPARSE_FORMAT_CSR) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (a->valueType != ACL_FLOAT) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (a->idxType != ACL_SPARSE_INDEX_32I || a->ptrType != ACL_SPARSE_INDEX_32I) {
        ACLSP_LOGE(tag, "int32 row offsets and column indices required");
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (a->ptrStride != 1 || a->idxStride != 1 || a->valueStride != 1) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t ValidateSpmvCommon(aclsparseOperation_t opA, aclDataType computeType)
{
    if (opA != ACL_SPARSE_OP_NON_TRANSPOSE || computeType != ACL_FLOAT) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

bool IsSpmvOpAlg(aclsparseSpMVOpAlg_t alg)
{
    return alg == ACL_SPARSE_SPMVOP_ALG_DEFAULT || alg == ACL_SPARSE_SPMVOP_ALG1 || alg == ACL_SPARSE_SPMVOP_ALG2;
}

bool IsSpmmOpAlg(aclsparseSpMMOpAlg_t alg)
{
    return alg == ACL_SPARSE_SPMMOP_ALG_DEFAULT || alg == ACL_SPARSE_SPMMOP_ALG1 || alg == ACL_SPARSE_SPMMOP_ALG2 ||
           alg == ACL_SPARSE_SPMMOP_ALG1_HIGH_PRECISION;
}

bool HandleUsable(aclsparseHandle_t h)
{
    return h->signature == kHandleSignature && h->stream != nullptr;
}

aclsparseStatus_t EnqueueStatus(const char* tag)
{
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        ACLSP_LOGE(tag, "enqueue failed: %s", cudaGetErrorString(err));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

/* ------------------------------------------------------------------ SpMVOp -- */

extern "C" aclsparseStatus_t aclsparseSpMVOp_bufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                                        aclsparseConstSpMatDescr_t matA,
                                                        aclsparseConstDnVecDescr_t vecX,
                                                        aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ,
                                                        aclDataType computeType, aclsparseSpMVOpAlg_t alg,
                                                        size_t* bufferSize)
{
    (void)vecX;
    (void)vecY;
    (void)vecZ;
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    aclsparseStatus_t st = ValidateSpmvCommon(opA, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = ValidateMatrix(kVTag, matA);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (!IsSpmvOpAlg(alg)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (bufferSize == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (matA->rows > kMaxI32 || matA->cols > kMaxI32 || matA->nnz > kMaxI32 - 1u) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    AclspPlanLayout layout;
    aclspSpmvLayout(matA->rows, matA->nnz, &layout);
    *bufferSize = static_cast<size_t>(layout.totalBytes);
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMVOp_createDescr(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t* descr,
                                                         aclsparseOperation_t opA, aclsparseConstSpMatDescr_t matA,
                                                         aclsparseConstDnVecDescr_t vecX,
                                                         aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ,
                                                         aclDataType computeType, aclsparseSpMVOpAlg_t alg,
                                                         void* buffer)
{
    (void)vecX;
    (void)vecY;
    (void)vecZ;
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (descr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    aclsparseStatus_t st = ValidateMatrix(kVTag, matA);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (!IsSpmvOpAlg(alg)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (buffer == nullptr || reinterpret_cast<uintptr_t>(buffer) % ACLSP_WS_ALIGN != 0 || !HandleUsable(handle)) {
        ACLSP_LOGE(kVTag, "createDescr needs a 64-byte aligned buffer of the size bufferSize reports, and a stream");
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    st = ValidateSpmvCommon(opA, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (matA->rows > kMaxI32 || matA->cols > kMaxI32 || matA->nnz > kMaxI32 - 1u) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (matA->rows > 0 && matA->ptrs == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* d = new (std::nothrow) aclsparseSpMVOpDescr;
    if (d == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    d->m = matA->rows;
    d->n = matA->cols;
    d->nnz = matA->nnz;
    d->rowOffsets = matA->ptrs;
    d->colIndices = matA->idxs;
    d->values = matA->values;
    d->mat = matA;
    d->base = matA->baseType;
    d->alg = alg == ACL_SPARSE_SPMVOP_ALG_DEFAULT ? ACL_SPARSE_SPMVOP_ALG1 : alg;
    d->buffer = buffer;
    if (d->m > 0) {
        (void)cudaGetLastError();
        spmv_b200_preprocess_kernel_do(d->rowOffsets, buffer, static_cast<uint32_t>(d->m), static_cast<uint32_t>(d->n),
                                       static_cast<uint32_t>(d->nnz), static_cast<int32_t>(d->base), 1, handle->stream);
        d->longestRow = AclspAcquireHostSlot();
        if (d->longestRow.word != nullptr) {
            (void)cudaMemcpyAsync(d->longestRow.word,
                                  static_cast<const unsigned char*>(buffer) + ACLSP_HEADER_MAX_ROW_LEN_OFF,
                                  sizeof(uint32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(handle->stream));
        }
        st = EnqueueStatus(kVTag);
        if (st != ACL_SPARSE_STATUS_SUCCESS) {
            delete d;
            return st;
        }
        (void)AclspPublishPlan(buffer);  // whatever plan another operator kept in this buffer is gone
    }
    *descr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMVOp_destroyDescr(aclsparseSpMVOpDescr_t descr)
{
    if (descr != nullptr) {
        descr->signature = 0;
        delete descr;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMVOp_createPlan(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t descr,
                                                        aclsparseSpMVOpPlan_t* plan, const void* epilogueLTOBuffer,
                                                        size_t epilogueLTOBufferSize)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (descr == nullptr || plan == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (epilogueLTOBuffer != nullptr || epilogueLTOBufferSize > 0) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;  // identity epilogue only, as in the reference
    }
    auto* p = new (std::nothrow) aclsparseSpMVOpPlan;
    if (p == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    p->descr = descr;
    *plan = p;
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMVOp_destroyPlan(aclsparseSpMVOpPlan_t plan)
{
    if (plan != nullptr) {
        plan->signature = 0;
        delete plan;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMVOp_setGlobalUserData(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan,
                                                               const char* epilogueDataName, void* epilogueData,
                                                               size_t epilogueDataSize)
{
    (void)epilogueDataName;
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (plan == nullptr || (epilogueData == nullptr) != (epilogueDataSize == 0)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;  // the identity epilogue has no data
}

extern "C" aclsparseStatus_t aclsparseSpMVOp(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan, const void* alpha,
                                             const void* beta, aclsparseConstDnVecDescr_t vecX,
                                             aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (plan == nullptr || plan->descr == nullptr || alpha == nullptr || beta == nullptr || vecX == nullptr ||
        vecY == nullptr || vecZ == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const aclsparseSpMVOpDescr* d = plan->descr;
    if (vecX->valueType != ACL_FLOAT || vecY->valueType != ACL_FLOAT || vecZ->valueType != ACL_FLOAT) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (d->n > 0 && vecX->values == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    // beta == 0 never reads Y, which may then be unbound; device scalars cannot be looked at here.
    const bool hostScalars = handle->pointerMode == ACL_SPARSE_POINTER_MODE_HOST;
    const bool skipY = !hostScalars || *static_cast<const float*>(beta) == 0.0f;
    if (!skipY && d->m > 0 && vecY->values == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (d->m > 0 && vecZ->values == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (vecX->nums != d->n || vecY->nums != d->m || vecZ->nums != d->m) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (!HandleUsable(handle)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (d->m == 0) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    const void* values = d->mat != nullptr && d->mat->signature == kSpMatSignature ? d->mat->values : d->values;
    if (d->nnz > 0 && (d->colIndices == nullptr || values == nullptr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }

    AclspSpmvParams params{};
    params.rows = static_cast<uint32_t>(d->m);
    params.cols = static_cast<uint32_t>(d->n);
    params.nnz = static_cast<uint32_t>(d->nnz);
    params.indexBase = static_cast<uint32_t>(d->base);
    params.colIndStride = 1;
    params.valuesStride = 1;
    params.xStride = vecX->stride;
    params.yStride = vecZ->stride;
    if (hostScalars) {
        params.alpha = *static_cast<const float*>(alpha);
        params.beta = *static_cast<const float*>(beta);
    } else {
        params.alphaPtr = static_cast<const float*>(alpha);
        params.betaPtr = static_cast<const float*>(beta);
    }
    if (vecY->values != vecZ->values || vecY->stride != vecZ->stride) {
        // With host scalars and beta == 0 the kernels never look at it, so an unbound Y is fine.
        params.betaSource = static_cast<const float*>(vecY->values);
        params.betaSourceStride = vecY->stride;
        if (params.betaSource == nullptr && !hostScalars) {
            return ACL_SPARSE_STATUS_INVALID_VALUE;  // a device beta might be non-zero
        }
    }
    params.maxRowLenHint = ACLSP_MAX_ROW_LEN_UNKNOWN;
    uint32_t longest = 0;
    if (AclspHostSlotValue(d->longestRow, &longest)) {
        params.maxRowLenHint = longest;
    }
    (void)cudaGetLastError();
    spmv_b200_kernel_do(d->colIndices, values, vecX->values, vecZ->values, d->buffer, &params, handle->stream);
    return EnqueueStatus(kVTag);
}

/* ------------------------------------------------------------------ SpMMOp -- */

namespace {

aclsparseStatus_t ValidateSpmmCommon(aclsparseOperation_t opA, aclsparseOperation_t opB, aclDataType computeType)
{
    if (opA != ACL_SPARSE_OP_NON_TRANSPOSE) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (opB != ACL_SPARSE_OP_NON_TRANSPOSE && opB != ACL_SPARSE_OP_TRANSPOSE) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (computeType != ACL_FLOAT) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// Shapes of B and C against A (m x k) and op(B): C is m x n, op(B) is k x n.
aclsparseStatus_t ValidateDense(uint64_t m, uint64_t k, aclsparseOperation_t opB, aclsparseConstDnMatDescr_t b,
                                aclsparseConstDnMatDescr_t c)
{
    if (b == nullptr || c == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (b->valueType != ACL_FLOAT || c->valueType != ACL_FLOAT) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    const bool plain = opB == ACL_SPARSE_OP_NON_TRANSPOSE;
    const int64_t bRows = plain ? b->rows : b->cols;
    const int64_t bCols = plain ? b->cols : b->rows;
    if (static_cast<uint64_t>(c->rows) != m || static_cast<uint64_t>(bRows) != k || bCols != c->cols) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const int64_t bLd = b->order == ACL_SPARSE_ORDER_ROW ? b->cols : b->rows;
    const int64_t cLd = c->order == ACL_SPARSE_ORDER_ROW ? c->cols : c->rows;
    if (b->ld < bLd || c->ld < cLd) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

extern "C" aclsparseStatus_t aclsparseSpMMOp_bufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                                        aclsparseOperation_t opB, aclsparseConstSpMatDescr_t matA,
                                                        aclsparseConstDnMatDescr_t matB, aclsparseDnMatDescr_t matC,
                                                        aclDataType computeType, aclsparseSpMMOpAlg_t alg,
                                                        size_t* bufferSize)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    aclsparseStatus_t st = ValidateSpmmCommon(opA, opB, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = ValidateMatrix(kMTag, matA);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (!IsSpmmOpAlg(alg)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (bufferSize == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    st = ValidateDense(matA->rows, matA->cols, opB, matB, matC);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (matA->rows > kMaxI32 || matA->cols > kMaxI32 || matA->nnz > kMaxI32 - 1u) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    AclspPlanLayout layout;
    aclspSpmmLayout(matA->rows, matA->nnz, static_cast<uint64_t>(matC->cols), &layout);
    *bufferSize = static_cast<size_t>(layout.totalBytes);
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMOp_createDescr(aclsparseHandle_t handle, aclsparseSpMMOpDescr_t* descr,
                                                         aclsparseOperation_t opA, aclsparseOperation_t opB,
                                                         aclsparseConstSpMatDescr_t matA,
                                                         aclsparseConstDnMatDescr_t matB, aclsparseDnMatDescr_t matC,
                                                         aclDataType computeType, aclsparseSpMMOpAlg_t alg,
                                                         void* buffer)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (descr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    aclsparseStatus_t st = ValidateMatrix(kMTag, matA);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (!IsSpmmOpAlg(alg)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    st = ValidateSpmmCommon(opA, opB, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    st = ValidateDense(matA->rows, matA->cols, opB, matB, matC);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (buffer == nullptr || reinterpret_cast<uintptr_t>(buffer) % ACLSP_WS_ALIGN != 0 || !HandleUsable(handle)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (matA->rows > kMaxI32 || matA->cols > kMaxI32 || matA->nnz > kMaxI32 - 1u) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (matA->rows > 0 && matA->ptrs == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* d = new (std::nothrow) aclsparseSpMMOpDescr;
    if (d == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    d->m = matA->rows;
    d->k = matA->cols;
    d->nnz = matA->nnz;
    d->maxDenseCols = static_cast<uint64_t>(matC->cols);
    d->rowOffsets = matA->ptrs;
    d->colIndices = matA->idxs;
    d->mat = matA;
    d->base = matA->baseType;
    d->opB = opB;
    d->alg = alg == ACL_SPARSE_SPMMOP_ALG_DEFAULT ? ACL_SPARSE_SPMMOP_ALG1 : alg;
    d->buffer = buffer;
    if (d->m > 0 && d->maxDenseCols > 0) {
        (void)cudaGetLastError();
        spmm_b200_preprocess_kernel_do(d->rowOffsets, buffer, static_cast<uint32_t>(d->m), static_cast<uint32_t>(d->k),
                                       static_cast<uint32_t>(d->nnz), static_cast<uint32_t>(d->maxDenseCols),
                                       static_cast<int32_t>(d->base), handle->stream);
        st = EnqueueStatus(kMTag);
        if (st != ACL_SPARSE_STATUS_SUCCESS) {
            delete d;
            return st;
        }
        (void)AclspPublishPlan(buffer);
    }
    *descr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMOp_destroyDescr(aclsparseSpMMOpDescr_t descr)
{
    if (descr != nullptr) {
        descr->signature = 0;
        delete descr;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMOp_createPlan(aclsparseHandle_t handle, aclsparseSpMMOpDescr_t descr,
                                                        aclsparseSpMMOpPlan_t* plan, const void* epilogueLTOBuffer,
                                                        size_t epilogueLTOBufferSize)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (descr == nullptr || plan == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (epilogueLTOBuffer != nullptr || epilogueLTOBufferSize > 0) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    auto* p = new (std::nothrow) aclsparseSpMMOpPlan;
    if (p == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    p->descr = descr;
    *plan = p;
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMOp_destroyPlan(aclsparseSpMMOpPlan_t plan)
{
    if (plan != nullptr) {
        plan->signature = 0;
        delete plan;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMOp_setGlobalUserData(aclsparseHandle_t handle, aclsparseSpMMOpPlan_t plan,
                                                               const char* epilogueDataName, void* epilogueData,
                                                               size_t epilogueDataSize)
{
    (void)epilogueDataName;
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (plan == nullptr || (epilogueData == nullptr) != (epilogueDataSize == 0)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseSpMMOp(aclsparseHandle_t handle, aclsparseSpMMOpPlan_t plan, const void* alpha,
                                             const void* beta, aclsparseConstDnMatDescr_t matB,
                                             aclsparseDnMatDescr_t matC)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (plan == nullptr || plan->descr == nullptr || alpha == nullptr || beta == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const aclsparseSpMMOpDescr* d = plan->descr;
    aclsparseStatus_t st = ValidateDense(d->m, d->k, d->opB, matB, matC);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (static_cast<uint64_t>(matC->cols) > d->maxDenseCols) {
        ACLSP_LOGE(kMTag, "C has %lld columns, the buffer was sized for %llu", static_cast<long long>(matC->cols),
                   static_cast<unsigned long long>(d->maxDenseCols));
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (!HandleUsable(handle)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (d->m == 0 || matC->cols == 0) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    const void* values = d->mat != nullptr && d->mat->signature == kSpMatSignature ? d->mat->values : nullptr;
    if ((matB->values == nullptr && d->k > 0) || matC->values == nullptr ||
        (d->nnz > 0 && (d->colIndices == nullptr || values == nullptr))) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    AclspSpmmParams params{};
    params.rows = static_cast<uint32_t>(d->m);
    params.cols = static_cast<uint32_t>(d->k);
    params.nnz = static_cast<uint32_t>(d->nnz);
    params.indexBase = static_cast<uint32_t>(d->base);
    params.n = static_cast<uint32_t>(matC->cols);
    params.opB = d->opB == ACL_SPARSE_OP_NON_TRANSPOSE ? 0u : 1u;
    params.orderB = static_cast<uint32_t>(matB->order);
    params.orderC = static_cast<uint32_t>(matC->order);
    params.highPrecision = d->alg == ACL_SPARSE_SPMMOP_ALG1_HIGH_PRECISION ? 1u : 0u;
    params.ldb = matB->ld;
    params.ldc = matC->ld;
    if (handle->pointerMode == ACL_SPARSE_POINTER_MODE_DEVICE) {
        params.alphaPtr = static_cast<const float*>(alpha);
        params.betaPtr = static_cast<const float*>(beta);
    } else {
        params.alpha = *static_cast<const float*>(alpha);
        params.beta = *static_cast<const float*>(beta);
    }
    // The offsets of the plan's parts do not depend on the width of C; only the carry area behind them
    // was sized for maxDenseCols columns, which bounds matC->cols above.
    (void)cudaGetLastError();
    spmm_b200_kernel_do(d->colIndices, values, matB->values, matC->values, d->buffer, &params, handle->stream);
    return EnqueueStatus(kMTag);
}
