/*
 * Host side of the B200-only entry points (include/aclsparse_b200_ext.h).
 */
#include <cuda_runtime.h>

#include "aclsparse_b200_ext.h"
#include "aclsparse_b200_kernels.h"
#include "internal.h"
#include "plan_layout.h"

extern "C" aclsparseStatus_t aclsparseB200RowBlockBounds(aclsparseHandle_t handle, aclsparseConstSpMatDescr_t matA,
                                                         int parts, void* bounds)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (handle->signature != kHandleSignature || handle->stream == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (matA == nullptr || matA->signature != kSpMatSignature || bounds == nullptr || parts < 1 || parts > 65535) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (matA->format != ACL_SPARSE_FORMAT_CSR || matA->ptrType != ACL_SPARSE_INDEX_32I || matA->ptrStride != 1 ||
        matA->rows > 0x7FFFFFFFull || matA->nnz > 0x7FFFFFFFull) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (matA->rows > 0 && matA->ptrs == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    (void)cudaGetLastError();
    aclsp_b200_row_block_bounds_kernel_do(matA->ptrs, static_cast<uint32_t>(matA->rows),
                                          static_cast<uint32_t>(matA->nnz), static_cast<int32_t>(matA->baseType),
                                          static_cast<uint32_t>(parts), bounds, handle->stream);
    if (cudaPeekAtLastError() != cudaSuccess) {
        ACLSP_LOGE("aclsparseB200RowBlockBounds", "kernel enqueue failed");
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

namespace {

template <typename Descr>
aclsparseStatus_t SetMirrors(Descr* d, uint32_t signature, int count, void* const* mirrors)
{
    if (d == nullptr || d->signature != signature || count < 0 || count > ACLSP_MAX_MIRRORS ||
        (count > 0 && mirrors == nullptr)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    for (int m = 0; m < count; ++m) {
        if (mirrors[m] == nullptr) {
            return ACL_SPARSE_STATUS_INVALID_VALUE;
        }
    }
    d->numMirrors = count;
    d->mirrorMulticast = false;
    for (int m = 0; m < ACLSP_MAX_MIRRORS; ++m) {
        d->mirrors[m] = m < count ? mirrors[m] : nullptr;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

template <typename Descr>
aclsparseStatus_t SetMulticastMirror(Descr* d, uint32_t signature, void* multicast)
{
    if (multicast == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    void* const one[1] = {multicast};
    const aclsparseStatus_t st = SetMirrors(d, signature, 1, one);
    if (st == ACL_SPARSE_STATUS_SUCCESS) {
        d->mirrorMulticast = true;
    }
    return st;
}

template <typename Descr>
aclsparseStatus_t SetClosingBarrier(Descr* d, uint32_t signature, void* localState, void* const* peerStates, int world,
                                    int rank, unsigned spinLimit)
{
    if (d == nullptr || d->signature != signature) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (localState == nullptr || world <= 1) {
        d->barrier = AclspBarrierLink{};
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (peerStates == nullptr || world > ACLSP_BARRIER_MAX_RANKS || rank < 0 || rank >= world) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    AclspBarrierLink link{};
    for (int r = 0; r < world; ++r) {
        if (r != rank && peerStates[r] == nullptr) {
            return ACL_SPARSE_STATUS_INVALID_VALUE;
        }
        link.peers[r] = peerStates[r];
    }
    link.local = localState;
    link.world = static_cast<uint32_t>(world);
    link.rank = static_cast<uint32_t>(rank);
    link.spinLimit = spinLimit != 0 ? spinLimit : 4000000u;  // about a second, as for aclsparseB200NodeBarrier
    d->barrier = link;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

extern "C" aclsparseStatus_t aclsparseB200DnVecSetClosingBarrier(aclsparseDnVecDescr_t vec, void* localState,
                                                                 void* const* peerStates, int world, int rank,
                                                                 unsigned spinLimit)
{
    return SetClosingBarrier(vec, kDnVecSignature, localState, peerStates, world, rank, spinLimit);
}

extern "C" aclsparseStatus_t aclsparseB200DnMatSetClosingBarrier(aclsparseDnMatDescr_t mat, void* localState,
                                                                 void* const* peerStates, int world, int rank,
                                                                 unsigned spinLimit)
{
    return SetClosingBarrier(mat, kDnMatSignature, localState, peerStates, world, rank, spinLimit);
}

extern "C" aclsparseStatus_t aclsparseB200DnVecSetMulticastMirror(aclsparseDnVecDescr_t vec, void* multicast)
{
    return SetMulticastMirror(vec, kDnVecSignature, multicast);
}

extern "C" aclsparseStatus_t aclsparseB200DnMatSetMulticastMirror(aclsparseDnMatDescr_t mat, void* multicast)
{
    return SetMulticastMirror(mat, kDnMatSignature, multicast);
}

extern "C" aclsparseStatus_t aclsparseB200DnVecSetMirrors(aclsparseDnVecDescr_t vec, int count, void* const* mirrors)
{
    return SetMirrors(vec, kDnVecSignature, count, mirrors);
}

extern "C" aclsparseStatus_t aclsparseB200DnMatSetMirrors(aclsparseDnMatDescr_t mat, int count, void* const* mirrors)
{
    return SetMirrors(mat, kDnMatSignature, count, mirrors);
}

extern "C" aclsparseStatus_t aclsparseB200NodeBarrier(aclrtStream stream, void* localState, void* const* peerStates,
                                                      int world, int rank, unsigned spinLimit)
{
    if (localState == nullptr || peerStates == nullptr || world < 1 || world > ACLSP_BARRIER_MAX_RANKS || rank < 0 ||
        rank >= world) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    for (int r = 0; r < world; ++r) {
        if (r != rank && peerStates[r] == nullptr) {
            return ACL_SPARSE_STATUS_INVALID_VALUE;
        }
    }
    if (world == 1) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    // About a second: a poll is a system-scope load plus a 64 ns sleep.
    const unsigned limit = spinLimit != 0 ? spinLimit : 4000000u;
    (void)cudaGetLastError();
    aclsp_b200_node_barrier_kernel_do(localState, peerStates, static_cast<uint32_t>(world),
                                      static_cast<uint32_t>(rank), limit, stream);
    if (cudaPeekAtLastError() != cudaSuccess) {
        ACLSP_LOGE("aclsparseB200NodeBarrier", "kernel enqueue failed");
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseB200SpMVWaitFailures(aclrtStream stream, const void* externalBuffer,
                                                           unsigned* count)
{
    if (externalBuffer == nullptr || count == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto s = static_cast<cudaStream_t>(stream);
    uint32_t value = 0;
    const auto* at = static_cast<const unsigned char*>(externalBuffer) + ACLSP_HEADER_WAIT_FAILURES_OFF;
    if (cudaMemcpyAsync(&value, at, sizeof(value), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    *count = value;
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseB200NodeBarrierStatus(aclrtStream stream, void* localState, int* missingRank)
{
    if (localState == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto s = static_cast<cudaStream_t>(stream);
    auto* state = static_cast<AclspNodeBarrierState*>(localState);
    uint32_t status = 0;
    if (cudaMemcpyAsync(&status, &state->status, sizeof(status), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (status == 0) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (missingRank != nullptr) {
        *missingRank = static_cast<int>(status) - 1;
    }
    (void)cudaMemsetAsync(&state->status, 0, sizeof(status), s);
    ACLSP_LOGE("aclsparseB200NodeBarrier", "rank %d did not arrive within the limit", static_cast<int>(status) - 1);
    return ACL_SPARSE_STATUS_EXECUTION_FAILED;
}
