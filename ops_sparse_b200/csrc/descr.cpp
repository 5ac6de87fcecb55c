/*
 * Descriptors over caller-owned device arrays: CSR matrix, dense vector and
 * dense matrix.  Validation rules and status codes follow the reference's
 * sparse/common/aclsparse_descr.cpp (CreateDnVec :375-431, vector accessors
 * :580-646, CreateCsr :648-712, CsrSetPointers/SetStrides :911-988,
 * DestroySpMat and SpMat accessors :1017-1100, DnMat :1102-1302).
 * Descriptors are plain host objects; none of these functions touches a device.
 */
#include <atomic>
#include <limits>
#include <new>

#include "internal.h"

namespace {

bool IsKnownValueType(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT:
        case ACL_FLOAT16:
        case ACL_DOUBLE:
        case ACL_INT8:
        case ACL_INT16:
        case ACL_INT32:
        case ACL_INT64:
        case ACL_UINT8:
        case ACL_UINT16:
        case ACL_UINT32:
        case ACL_UINT64:
        case ACL_BF16:
        case ACL_FLOAT8_E4M3FN:
        case ACL_FLOAT8_E5M2:
        case ACL_FLOAT4_E2M1:
        case ACL_COMPLEX64:
        case ACL_COMPLEX128:
            return true;
        default:
            return false;
    }
}

int64_t StorageBytes(aclDataType t)
{
    switch (t) {
        case ACL_INT8:
        case ACL_UINT8:
        case ACL_FLOAT8_E4M3FN:
        case ACL_FLOAT8_E5M2:
        case ACL_FLOAT4_E2M1:
            return 1;
        case ACL_FLOAT16:
        case ACL_BF16:
        case ACL_INT16:
        case ACL_UINT16:
            return 2;
        case ACL_FLOAT:
        case ACL_INT32:
        case ACL_UINT32:
            return 4;
        case ACL_DOUBLE:
        case ACL_INT64:
        case ACL_UINT64:
        case ACL_COMPLEX64:
            return 8;
        case ACL_COMPLEX128:
            return 16;
        default:
            return 0;
    }
}

bool IsIndexType(aclsparseIndexType_t t)
{
    return t == ACL_SPARSE_INDEX_32I || t == ACL_SPARSE_INDEX_64I;
}

// An element stride is usable when the last logical element is still
// addressable with a signed 64-bit element offset.
bool IsUsableStride(uint64_t logicalSize, int64_t stride)
{
    if (stride <= 0) {
        return false;
    }
    if (logicalSize <= 1u) {
        return true;
    }
    return static_cast<uint64_t>(stride) <=
           static_cast<uint64_t>(std::numeric_limits<int64_t>::max()) / (logicalSize - 1u);
}

bool MulNonNegative(int64_t a, int64_t b, int64_t* out)
{
    if (a < 0 || b < 0 || (a != 0 && b > std::numeric_limits<int64_t>::max() / a)) {
        return false;
    }
    *out = a * b;
    return true;
}

bool AddNonNegative(int64_t a, int64_t b, int64_t* out)
{
    if (a < 0 || b < 0 || b > std::numeric_limits<int64_t>::max() - a) {
        return false;
    }
    *out = a + b;
    return true;
}

bool IsSpMat(const aclsparseSpMatDescr* d) { return d != nullptr && d->signature == kSpMatSignature; }
bool IsDnVec(const aclsparseDnVecDescr* d) { return d != nullptr && d->signature == kDnVecSignature; }
bool IsDnMat(const aclsparseDnMatDescr* d) { return d != nullptr && d->signature == kDnMatSignature; }

template <typename Out, typename Val>
void Put(Out* out, Val value)
{
    if (out != nullptr) {
        *out = value;
    }
}

void MarkStructureChanged(aclsparseSpMatDescr* d)
{
    ++d->structureGeneration;
    if (d->structureGeneration == 0) {
        d->structureGeneration = 1;
    }
    d->activeBuffer = nullptr;
    d->spmv.buffer = nullptr;
    d->spmm.buffer = nullptr;
}

}  // namespace

uint64_t AclspNextWorkspaceOwnerId()
{
    static std::atomic<uint64_t> next{1};
    return next.fetch_add(1, std::memory_order_relaxed);
}

void AclspResetSpmvPlan(aclsparseSpMatDescr* descr)
{
    descr->activeBuffer = nullptr;
    descr->spmv = SpmvPlanRecord{};
}

extern "C" {

/* ---------------------------------------------------------------- DnVec -- */

aclsparseStatus_t aclsparseCreateDnVec(aclsparseDnVecDescr_t* dnVecDescr, int64_t size, void* values,
                                       aclDataType valueType)
{
    // `values` may be NULL: callers query workspace sizes before binding data.
    if (dnVecDescr == nullptr || size < 0 || !IsKnownValueType(valueType)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* d = new (std::nothrow) aclsparseDnVecDescr();
    if (d == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    d->signature = kDnVecSignature;
    d->nums = static_cast<uint64_t>(size);
    d->values = values;
    d->valueType = valueType;
    *dnVecDescr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCreateConstDnVec(aclsparseConstDnVecDescr_t* dnVecDescr, int64_t size,
                                            const void* values, aclDataType valueType)
{
    if (dnVecDescr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    aclsparseDnVecDescr_t tmp = nullptr;
    const aclsparseStatus_t st = aclsparseCreateDnVec(&tmp, size, const_cast<void*>(values), valueType);
    if (st == ACL_SPARSE_STATUS_SUCCESS) {
        *dnVecDescr = tmp;
    }
    return st;
}

aclsparseStatus_t aclsparseDestroyDnVec(aclsparseConstDnVecDescr_t dnVecDescr)
{
    if (dnVecDescr == nullptr) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    auto* d = const_cast<aclsparseDnVecDescr*>(dnVecDescr);
    if (d->signature != kDnVecSignature) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    d->signature = 0;
    delete d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstDnVecGet(aclsparseConstDnVecDescr_t dnVecDescr, int64_t* size,
                                         const void** values, aclDataType* valueType)
{
    if (!IsDnVec(dnVecDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(size, static_cast<int64_t>(dnVecDescr->nums));
    Put(values, static_cast<const void*>(dnVecDescr->values));
    Put(valueType, dnVecDescr->valueType);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecGet(aclsparseDnVecDescr_t dnVecDescr, int64_t* size, void** values,
                                    aclDataType* valueType)
{
    return aclsparseConstDnVecGet(dnVecDescr, size, const_cast<const void**>(values), valueType);
}

aclsparseStatus_t aclsparseConstDnVecGetValues(aclsparseConstDnVecDescr_t dnVecDescr, const void** values)
{
    if (!IsDnVec(dnVecDescr) || values == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *values = dnVecDescr->values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecGetValues(aclsparseDnVecDescr_t dnVecDescr, void** values)
{
    return aclsparseConstDnVecGetValues(dnVecDescr, const_cast<const void**>(values));
}

aclsparseStatus_t aclsparseDnVecSetValues(aclsparseDnVecDescr_t dnVecDescr, void* values)
{
    if (!IsDnVec(dnVecDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    dnVecDescr->values = values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecSetStride(aclsparseDnVecDescr_t dnVecDescr, int64_t stride)
{
    if (!IsDnVec(dnVecDescr) || !IsUsableStride(dnVecDescr->nums, stride)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    dnVecDescr->stride = stride;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecGetStride(aclsparseConstDnVecDescr_t dnVecDescr, int64_t* stride)
{
    if (!IsDnVec(dnVecDescr) || stride == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *stride = dnVecDescr->stride;
    return ACL_SPARSE_STATUS_SUCCESS;
}

/* ------------------------------------------------------------------ CSR -- */

aclsparseStatus_t aclsparseCreateCsr(aclsparseSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                     void* csrRowOffsets, void* csrColInd, void* csrValues,
                                     aclsparseIndexType_t csrRowOffsetsType, aclsparseIndexType_t csrColIndType,
                                     aclsparseIndexBase_t idxBase, aclDataType valueType)
{
    if (spMatDescr == nullptr || rows < 0 || cols < 0 || nnz < 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    // Unknown index widths are "not supported"; the operators narrow this
    // further (SpMV and SpMM take int32 only).
    if (!IsIndexType(csrRowOffsetsType) || !IsIndexType(csrColIndType)) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (idxBase != ACL_SPARSE_INDEX_BASE_ZERO && idxBase != ACL_SPARSE_INDEX_BASE_ONE) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (!IsKnownValueType(valueType)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* d = new (std::nothrow) aclsparseSpMatDescr();
    if (d == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    d->format = ACL_SPARSE_FORMAT_CSR;
    d->workspaceOwnerId = AclspNextWorkspaceOwnerId();
    d->rows = static_cast<uint64_t>(rows);
    d->cols = static_cast<uint64_t>(cols);
    d->nnz = static_cast<uint64_t>(nnz);
    d->ptrs = csrRowOffsets;
    d->idxs = csrColInd;
    d->values = csrValues;
    d->baseType = idxBase;
    d->ptrType = csrRowOffsetsType;
    d->idxType = csrColIndType;
    d->valueType = valueType;
    *spMatDescr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCreateConstCsr(aclsparseConstSpMatDescr_t* spMatDescr, int64_t rows, int64_t cols,
                                          int64_t nnz, const void* csrRowOffsets, const void* csrColInd,
                                          const void* csrValues, aclsparseIndexType_t csrRowOffsetsType,
                                          aclsparseIndexType_t csrColIndType, aclsparseIndexBase_t idxBase,
                                          aclDataType valueType)
{
    if (spMatDescr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    aclsparseSpMatDescr_t tmp = nullptr;
    const aclsparseStatus_t st =
        aclsparseCreateCsr(&tmp, rows, cols, nnz, const_cast<void*>(csrRowOffsets), const_cast<void*>(csrColInd),
                           const_cast<void*>(csrValues), csrRowOffsetsType, csrColIndType, idxBase, valueType);
    if (st == ACL_SPARSE_STATUS_SUCCESS) {
        *spMatDescr = tmp;
    }
    return st;
}

aclsparseStatus_t aclsparseCsrSetPointers(aclsparseSpMatDescr_t descr, void* rowOffsets, void* colIndices,
                                          void* values)
{
    if (!IsSpMat(descr) || descr->format != ACL_SPARSE_FORMAT_CSR ||
        (rowOffsets == nullptr && descr->rows > 0 && descr->cols > 0) ||
        (descr->nnz > 0 && (colIndices == nullptr || values == nullptr))) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const bool structureChanged = descr->ptrs != rowOffsets || descr->idxs != colIndices;
    if (structureChanged || descr->values != values) {
        AclspResetSpmvPlan(descr);
    }
    descr->ptrs = rowOffsets;
    descr->idxs = colIndices;
    descr->values = values;
    if (structureChanged) {
        MarkStructureChanged(descr);
    }
    descr->workspaceOwnerId = AclspNextWorkspaceOwnerId();
    descr->activeBuffer = nullptr;
    descr->spmv.buffer = nullptr;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCsrSetStrides(aclsparseSpMatDescr_t descr, int64_t rowOffsetsStride,
                                         int64_t colIndStride, int64_t valuesStride)
{
    if (!IsSpMat(descr) || descr->format != ACL_SPARSE_FORMAT_CSR ||
        !IsUsableStride(descr->rows + 1u, rowOffsetsStride) || !IsUsableStride(descr->nnz, colIndStride) ||
        !IsUsableStride(descr->nnz, valuesStride)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const bool changed = descr->ptrStride != rowOffsetsStride || descr->idxStride != colIndStride ||
                         descr->valueStride != valuesStride;
    descr->ptrStride = rowOffsetsStride;
    descr->idxStride = colIndStride;
    descr->valueStride = valuesStride;
    if (changed) {
        MarkStructureChanged(descr);
    }
    descr->workspaceOwnerId = AclspNextWorkspaceOwnerId();
    descr->activeBuffer = nullptr;
    descr->spmv.buffer = nullptr;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCsrGetStrides(aclsparseConstSpMatDescr_t descr, int64_t* rowOffsetsStride,
                                         int64_t* colIndStride, int64_t* valuesStride)
{
    if (!IsSpMat(descr) || descr->format != ACL_SPARSE_FORMAT_CSR || rowOffsetsStride == nullptr ||
        colIndStride == nullptr || valuesStride == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *rowOffsetsStride = descr->ptrStride;
    *colIndStride = descr->idxStride;
    *valuesStride = descr->valueStride;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDestroySpMat(aclsparseConstSpMatDescr_t spMatDescr)
{
    if (spMatDescr == nullptr) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    auto* d = const_cast<aclsparseSpMatDescr*>(spMatDescr);
    if (d->signature != kSpMatSignature) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    d->signature = 0;
    delete d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetFormat(aclsparseConstSpMatDescr_t spMatDescr, aclsparseFormat_t* format)
{
    if (!IsSpMat(spMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(format, spMatDescr->format);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetIndexBase(aclsparseConstSpMatDescr_t spMatDescr, aclsparseIndexBase_t* idxBase)
{
    if (!IsSpMat(spMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(idxBase, spMatDescr->baseType);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstSpMatGetValues(aclsparseConstSpMatDescr_t spMatDescr, const void** values)
{
    if (!IsSpMat(spMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(values, static_cast<const void*>(spMatDescr->values));
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetValues(aclsparseSpMatDescr_t spMatDescr, void** values)
{
    return aclsparseConstSpMatGetValues(spMatDescr, const_cast<const void**>(values));
}

aclsparseStatus_t aclsparseSpMatSetValues(aclsparseSpMatDescr_t spMatDescr, void* values)
{
    if (!IsSpMat(spMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (spMatDescr->values != values) {
        AclspResetSpmvPlan(spMatDescr);
    }
    spMatDescr->values = values;
    spMatDescr->workspaceOwnerId = AclspNextWorkspaceOwnerId();
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetSize(aclsparseConstSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols,
                                        int64_t* nnz)
{
    if (!IsSpMat(spMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(rows, static_cast<int64_t>(spMatDescr->rows));
    Put(cols, static_cast<int64_t>(spMatDescr->cols));
    Put(nnz, static_cast<int64_t>(spMatDescr->nnz));
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstCsrGet(aclsparseConstSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols,
                                       int64_t* nnz, const void** csrRowOffsets, const void** csrColInd,
                                       const void** csrValues, aclsparseIndexType_t* csrRowOffsetsType,
                                       aclsparseIndexType_t* csrColIndType, aclsparseIndexBase_t* idxBase,
                                       aclDataType* valueType)
{
    if (!IsSpMat(spMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (spMatDescr->format != ACL_SPARSE_FORMAT_CSR) {
        return ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED;
    }
    Put(rows, static_cast<int64_t>(spMatDescr->rows));
    Put(cols, static_cast<int64_t>(spMatDescr->cols));
    Put(nnz, static_cast<int64_t>(spMatDescr->nnz));
    Put(csrRowOffsets, static_cast<const void*>(spMatDescr->ptrs));
    Put(csrColInd, static_cast<const void*>(spMatDescr->idxs));
    Put(csrValues, static_cast<const void*>(spMatDescr->values));
    Put(csrRowOffsetsType, spMatDescr->ptrType);
    Put(csrColIndType, spMatDescr->idxType);
    Put(idxBase, spMatDescr->baseType);
    Put(valueType, spMatDescr->valueType);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCsrGet(aclsparseSpMatDescr_t spMatDescr, int64_t* rows, int64_t* cols, int64_t* nnz,
                                  void** csrRowOffsets, void** csrColInd, void** csrValues,
                                  aclsparseIndexType_t* csrRowOffsetsType, aclsparseIndexType_t* csrColIndType,
                                  aclsparseIndexBase_t* idxBase, aclDataType* valueType)
{
    return aclsparseConstCsrGet(spMatDescr, rows, cols, nnz, const_cast<const void**>(csrRowOffsets),
                                const_cast<const void**>(csrColInd), const_cast<const void**>(csrValues),
                                csrRowOffsetsType, csrColIndType, idxBase, valueType);
}

/* ---------------------------------------------------------------- DnMat -- */

aclsparseStatus_t aclsparseCreateDnMat(aclsparseDnMatDescr_t* dnMatDescr, int64_t rows, int64_t cols, int64_t ld,
                                       void* values, aclDataType valueType, aclsparseOrder_t order)
{
    constexpr int64_t kMaxDim = std::numeric_limits<int32_t>::max();
    if (dnMatDescr == nullptr || rows < 0 || cols < 0 || rows > kMaxDim || cols > kMaxDim || ld < 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    // Only a matrix with no elements may come without storage.
    if (rows != 0 && cols != 0 && values == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (!IsKnownValueType(valueType) || (order != ACL_SPARSE_ORDER_ROW && order != ACL_SPARSE_ORDER_COL)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if ((order == ACL_SPARSE_ORDER_ROW && ld < cols) || (order == ACL_SPARSE_ORDER_COL && ld < rows)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* d = new (std::nothrow) aclsparseDnMatDescr();
    if (d == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    d->signature = kDnMatSignature;
    d->rows = rows;
    d->cols = cols;
    d->ld = ld;
    d->order = order;
    d->values = values;
    d->valueType = valueType;
    *dnMatDescr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCreateConstDnMat(aclsparseConstDnMatDescr_t* dnMatDescr, int64_t rows, int64_t cols,
                                            int64_t ld, const void* values, aclDataType valueType,
                                            aclsparseOrder_t order)
{
    if (dnMatDescr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    aclsparseDnMatDescr_t tmp = nullptr;
    const aclsparseStatus_t st =
        aclsparseCreateDnMat(&tmp, rows, cols, ld, const_cast<void*>(values), valueType, order);
    if (st == ACL_SPARSE_STATUS_SUCCESS) {
        *dnMatDescr = tmp;
    }
    return st;
}

aclsparseStatus_t aclsparseDestroyDnMat(aclsparseConstDnMatDescr_t dnMatDescr)
{
    if (dnMatDescr == nullptr) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    auto* d = const_cast<aclsparseDnMatDescr*>(dnMatDescr);
    if (d->signature != kDnMatSignature) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    d->signature = 0;
    delete d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstDnMatGet(aclsparseConstDnMatDescr_t dnMatDescr, int64_t* rows, int64_t* cols,
                                         int64_t* ld, const void** values, aclDataType* valueType,
                                         aclsparseOrder_t* order)
{
    if (!IsDnMat(dnMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(rows, dnMatDescr->rows);
    Put(cols, dnMatDescr->cols);
    Put(ld, dnMatDescr->ld);
    Put(values, static_cast<const void*>(dnMatDescr->values));
    Put(valueType, dnMatDescr->valueType);
    Put(order, dnMatDescr->order);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatGet(aclsparseDnMatDescr_t dnMatDescr, int64_t* rows, int64_t* cols, int64_t* ld,
                                    void** values, aclDataType* valueType, aclsparseOrder_t* order)
{
    return aclsparseConstDnMatGet(dnMatDescr, rows, cols, ld, const_cast<const void**>(values), valueType, order);
}

aclsparseStatus_t aclsparseConstDnMatGetValues(aclsparseConstDnMatDescr_t dnMatDescr, const void** values)
{
    if (!IsDnMat(dnMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    Put(values, static_cast<const void*>(dnMatDescr->values));
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatGetValues(aclsparseDnMatDescr_t dnMatDescr, void** values)
{
    return aclsparseConstDnMatGetValues(dnMatDescr, const_cast<const void**>(values));
}

aclsparseStatus_t aclsparseDnMatSetValues(aclsparseDnMatDescr_t dnMatDescr, void* values)
{
    if (!IsDnMat(dnMatDescr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    dnMatDescr->values = values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatGetStridedBatch(aclsparseConstDnMatDescr_t dnMatDescr, int* batchCount,
                                                int64_t* batchStride)
{
    if (!IsDnMat(dnMatDescr) || batchCount == nullptr || batchStride == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *batchCount = dnMatDescr->batchCount;
    *batchStride = dnMatDescr->batchStride;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatSetStridedBatch(aclsparseDnMatDescr_t dnMatDescr, int batchCount,
                                                int64_t batchStride)
{
    if (!IsDnMat(dnMatDescr) || batchCount < 1 || batchCount > kMaxStridedBatchCount || batchStride < 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const bool rowMajor = dnMatDescr->order == ACL_SPARSE_ORDER_ROW;
    const int64_t major = rowMajor ? dnMatDescr->rows : dnMatDescr->cols;
    const int64_t minor = rowMajor ? dnMatDescr->cols : dnMatDescr->rows;
    // Elements from the first to the last readable one of a single matrix.
    int64_t span = 0;
    if (major != 0 && minor != 0 &&
        (!MulNonNegative(major - 1, dnMatDescr->ld, &span) || !AddNonNegative(span, minor, &span))) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    int64_t bytes = 0;
    const int64_t elementBytes = StorageBytes(dnMatDescr->valueType);
    if (elementBytes <= 0 || !MulNonNegative(span, elementBytes, &bytes) || (batchCount > 1 && batchStride < span)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    int64_t lastBatch = 0;
    int64_t extent = 0;
    if (!MulNonNegative(static_cast<int64_t>(batchCount - 1), batchStride, &lastBatch) ||
        !AddNonNegative(lastBatch, span, &extent) || !MulNonNegative(extent, elementBytes, &bytes)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (dnMatDescr->values != nullptr && bytes > 0 &&
        static_cast<uint64_t>(bytes - 1) >
            std::numeric_limits<uintptr_t>::max() - reinterpret_cast<uintptr_t>(dnMatDescr->values)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    dnMatDescr->batchCount = batchCount;
    dnMatDescr->batchStride = batchStride;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
