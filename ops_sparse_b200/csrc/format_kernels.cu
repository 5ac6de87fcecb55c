/*
 * The two format producers that feed the SpMV / SpMM path for callers who start from COO or from
 * unsorted CSR (the PyTorch adapter's callers do): aclsparseXcoo2csr and aclsparseXcsrsort, and the
 * legacy matrix descriptor the latter takes its index base from.  Integer work only; every result is
 * reproduced bit for bit by the CPU twin in the test oracle.
 *
 * aclsparseXcoo2csr (reference: sparse/coo2csr/arch35/coo2csr_host.cpp:38-77 for the checks,
 * include/cann_ops_sparse.h:2780-2801): row offsets of sorted COO row indices.  The reference counts
 * and prefix-sums; here thread r looks up the first entry whose row is not below r with a binary
 * search, which needs no scratch memory and no atomics.
 *
 * aclsparseXcsrsort (reference: sparse/csrsort/arch35/csrsort_host.cpp:40-215,
 * include/cann_ops_sparse.h:2513-2546): sorts the column indices of every row ascending, in place and
 * stably (equal columns keep their order: repeated coordinates are legal), and applies the same
 * permutation to P.  A warp ranks rows of up to 32 entries with shuffles; a CTA sorts longer rows with a
 * sorting network on (column, original position) pairs, in shared memory up to 2048 entries and in
 * the caller's workspace beyond.  The workspace is 8 bytes per non-zero, as the reference's.
 */
#include <cstdint>
#include <new>

#include <cuda_runtime.h>

#include "cann_ops_sparse.h"
#include "internal.h"
#include "plan_kernels.h"

struct aclsparseMatDescr {
    uint32_t signature = 0x4D444553u;
    aclsparseMatrixType_t type = ACL_SPARSE_MATRIX_TYPE_GENERAL;
    aclsparseIndexBase_t base = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseDiagType_t diag = ACL_SPARSE_DIAG_TYPE_NON_UNIT;
    aclsparseFillMode_t fill = ACL_SPARSE_FILL_MODE_LOWER;
};

namespace {

constexpr int kSortSmem = 2048;

__global__ void Coo2CsrKernel(const int32_t* __restrict__ cooRowInd, int32_t nnz, int32_t m, int32_t base,
                              int32_t* __restrict__ csrRowPtr)
{
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r <= m; r += step) {
        // first entry whose row (with its base) is at least r + base
        int32_t lo = 0;
        int32_t hi = nnz;
        while (lo < hi) {
            const int32_t mid = lo + ((hi - lo) >> 1);
            if (static_cast<int64_t>(cooRowInd[mid]) < r + base) {
                lo = mid + 1;
            } else {
                hi = mid;
            }
        }
        csrRowPtr[r] = lo + base;
    }
}

__global__ void CopyKernel(const int32_t* __restrict__ src, int32_t* __restrict__ dst, int64_t n)
{
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {
        dst[i] = src[i];
    }
}

__device__ __forceinline__ int ClampOffset(int64_t v, int nnz)
{
    return v < 0 ? 0 : (v > nnz ? nnz : static_cast<int>(v));
}

// Rows of up to 32 entries: lane i holds entry i; its rank is the number of entries that sort before
// it (smaller column, or equal column and earlier position).
__global__ void SortShortRowsKernel(const int32_t* __restrict__ rowPtr, int32_t m, int32_t nnz, int32_t base,
                                    int32_t* __restrict__ colInd, int32_t* __restrict__ perm,
                                    const int32_t* __restrict__ permIn)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < m; r += warps) {
        const int b = ClampOffset(static_cast<int64_t>(rowPtr[r]) - base, nnz);
        const int e = ClampOffset(static_cast<int64_t>(rowPtr[r + 1]) - base, nnz);
        const int len = e - b;
        if (len <= 0 || len > 32) {
            if (len > 32) {
                continue;  // SortLongRowsKernel
            }
            continue;
        }
        const bool has = lane < len;
        const int32_t col = has ? colInd[b + lane] : 0x7fffffff;
        const int32_t p = has ? permIn[b + lane] : 0;
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int32_t other = __shfl_sync(0xffffffffu, col, j);
            rank += (other < col || (other == col && j < lane)) ? 1 : 0;
        }
        __syncwarp();
        if (has) {
            colInd[b + rank] = col;
            perm[b + rank] = p;
        }
    }
}

// Sorting network whose comparators all put the smaller element at the lower index, so that the
// slots above `len` behave like +infinity and are never touched.
template <typename Swap>
__device__ __forceinline__ void NetworkAscending(int len, Swap swapIfGreater)
{
    int padded = 1;
    while (padded < len) {
        padded <<= 1;
    }
    for (int k = 2; k <= padded; k <<= 1) {
        for (int i = threadIdx.x; i < padded; i += blockDim.x) {
            const int l = i ^ (k - 1);
            if (l > i && l < len) {
                swapIfGreater(i, l);
            }
        }
        __syncthreads();
        for (int j = k >> 2; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < padded; i += blockDim.x) {
                const int l = i ^ j;
                if (l > i && l < len) {
                    swapIfGreater(i, l);
                }
            }
            __syncthreads();
        }
    }
}

// Persistent CTAs walk the rows and sort those with more than 32 entries.  `order` is scratch of nnz
// words: the original position of every entry of a row that does not fit shared memory.
__global__ void __launch_bounds__(256)
SortLongRowsKernel(const int32_t* __restrict__ rowPtr, int32_t m, int32_t nnz, int32_t base,
                   int32_t* __restrict__ colInd, int32_t* __restrict__ perm, const int32_t* __restrict__ permIn,
                   int32_t* __restrict__ order)
{
    __shared__ int32_t sCol[kSortSmem];
    __shared__ int32_t sPos[kSortSmem];
    for (int64_t r = blockIdx.x; r < m; r += gridDim.x) {
        const int b = ClampOffset(static_cast<int64_t>(rowPtr[r]) - base, nnz);
        const int e = ClampOffset(static_cast<int64_t>(rowPtr[r + 1]) - base, nnz);
        const int len = e - b;
        if (len <= 32) {
            continue;
        }
        if (len <= kSortSmem) {
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                sCol[i] = colInd[b + i];
                sPos[i] = i;
            }
            __syncthreads();
            NetworkAscending(len, [&](int i, int l) {
                const int32_t ci = sCol[i], cl = sCol[l], pi = sPos[i], pl = sPos[l];
                if (ci > cl || (ci == cl && pi > pl)) {
                    sCol[i] = cl;
                    sCol[l] = ci;
                    sPos[i] = pl;
                    sPos[l] = pi;
                }
            });
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                colInd[b + i] = sCol[i];
                perm[b + i] = permIn[b + sPos[i]];
            }
            __syncthreads();
        } else {
            int32_t* col = colInd + b;
            int32_t* pos = order + b;
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                pos[i] = i;
            }
            __syncthreads();
            NetworkAscending(len, [&](int i, int l) {
                const int32_t ci = col[i], cl = col[l], pi = pos[i], pl = pos[l];
                if (ci > cl || (ci == cl && pi > pl)) {
                    col[i] = cl;
                    col[l] = ci;
                    pos[i] = pl;
                    pos[l] = pi;
                }
            });
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                perm[b + i] = permIn[b + pos[i]];
            }
            __syncthreads();
        }
    }
}

unsigned GridFor(int64_t items, int perBlock)
{
    int64_t blocks = (items + perBlock - 1) / perBlock;
    blocks = blocks < 1 ? 1 : (blocks > 148 * 32 ? 148 * 32 : blocks);
    return static_cast<unsigned>(blocks);
}

aclsparseStatus_t CsrsortCommon(int m, int n, int nnz, const int* csrRowPtr, const int* csrColInd)
{
    if (m < 0 || n < 0 || nnz < 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if ((m == 0 || n == 0) && nnz != 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (m > 0 && csrRowPtr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (nnz > 0 && csrColInd == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

/* --------------------------------------------------- legacy MatDescr -- */

extern "C" aclsparseStatus_t aclsparseCreateMatDescr(aclsparseMatDescr_t* descr)
{
    if (descr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* d = new (std::nothrow) aclsparseMatDescr;
    if (d == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    *descr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseDestroyMatDescr(aclsparseMatDescr_t descr)
{
    if (descr != nullptr) {
        descr->signature = 0;
        delete descr;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" void aclsparseSetMatType(aclsparseMatDescr_t descr, aclsparseMatrixType_t type)
{
    if (descr != nullptr) {
        descr->type = type;
    }
}
extern "C" void aclsparseSetMatIndexBase(aclsparseMatDescr_t descr, aclsparseIndexBase_t base)
{
    if (descr != nullptr) {
        descr->base = base;
    }
}
extern "C" void aclsparseSetMatDiagType(aclsparseMatDescr_t descr, aclsparseDiagType_t diagType)
{
    if (descr != nullptr) {
        descr->diag = diagType;
    }
}
extern "C" void aclsparseSetMatFillMode(aclsparseMatDescr_t descr, aclsparseFillMode_t fillMode)
{
    if (descr != nullptr) {
        descr->fill = fillMode;
    }
}
extern "C" aclsparseMatrixType_t aclsparseGetMatType(aclsparseMatDescr_t descr)
{
    return descr != nullptr ? descr->type : ACL_SPARSE_MATRIX_TYPE_GENERAL;
}
extern "C" aclsparseIndexBase_t aclsparseGetMatIndexBase(aclsparseMatDescr_t descr)
{
    return descr != nullptr ? descr->base : ACL_SPARSE_INDEX_BASE_ZERO;
}
extern "C" aclsparseDiagType_t aclsparseGetMatDiagType(aclsparseMatDescr_t descr)
{
    return descr != nullptr ? descr->diag : ACL_SPARSE_DIAG_TYPE_NON_UNIT;
}
extern "C" aclsparseFillMode_t aclsparseGetMatFillMode(aclsparseMatDescr_t descr)
{
    return descr != nullptr ? descr->fill : ACL_SPARSE_FILL_MODE_LOWER;
}

/* ------------------------------------------------------------ coo2csr -- */

extern "C" aclsparseStatus_t aclsparseXcoo2csr(aclsparseHandle_t handle, const int* cooRowInd, int nnz, int m,
                                               int* csrRowPtr, aclsparseIndexBase_t idxBase)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (nnz < 0 || (nnz == 0x7fffffff && idxBase == ACL_SPARSE_INDEX_BASE_ONE) || m < 0 || (nnz > 0 && m == 0)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (idxBase != ACL_SPARSE_INDEX_BASE_ZERO && idxBase != ACL_SPARSE_INDEX_BASE_ONE) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if ((nnz > 0 && cooRowInd == nullptr) || csrRowPtr == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (handle->signature != kHandleSignature || handle->stream == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    (void)cudaGetLastError();
    AclspCountLaunches(1);
    Coo2CsrKernel<<<GridFor(static_cast<int64_t>(m) + 1, 256), 256, 0, static_cast<cudaStream_t>(handle->stream)>>>(
        cooRowInd, nnz, m, static_cast<int32_t>(idxBase), csrRowPtr);
    return cudaPeekAtLastError() == cudaSuccess ? ACL_SPARSE_STATUS_SUCCESS : ACL_SPARSE_STATUS_EXECUTION_FAILED;
}

/* ------------------------------------------------------------ csrsort -- */

extern "C" aclsparseStatus_t aclsparseXcsrsort_bufferSizeExt(aclsparseHandle_t handle, int m, int n, int nnz,
                                                             const int* csrRowPtr, const int* csrColInd,
                                                             size_t* pBufferSizeInBytes)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (pBufferSizeInBytes == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const aclsparseStatus_t st = CsrsortCommon(m, n, nnz, csrRowPtr, csrColInd);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    *pBufferSizeInBytes = static_cast<size_t>(nnz) * 2u * sizeof(int32_t);
    return ACL_SPARSE_STATUS_SUCCESS;
}

extern "C" aclsparseStatus_t aclsparseXcsrsort(aclsparseHandle_t handle, int m, int n, int nnz,
                                               const aclsparseMatDescr_t descrA, const int* csrRowPtr,
                                               int* csrColInd, int* P, void* pBuffer)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    const aclsparseStatus_t st = CsrsortCommon(m, n, nnz, csrRowPtr, csrColInd);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (descrA == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const aclsparseIndexBase_t base = descrA->base;
    if (base != ACL_SPARSE_INDEX_BASE_ZERO && base != ACL_SPARSE_INDEX_BASE_ONE) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (nnz == 0) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (P == nullptr || pBuffer == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (handle->signature != kHandleSignature || handle->stream == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto s = static_cast<cudaStream_t>(handle->stream);
    auto* permIn = static_cast<int32_t*>(pBuffer);  // P as it came in
    int32_t* order = permIn + nnz;                   // positions of the entries of very long rows
    (void)cudaGetLastError();
    AclspCountLaunches(3);
    CopyKernel<<<GridFor(nnz, 256), 256, 0, s>>>(P, permIn, nnz);
    SortShortRowsKernel<<<GridFor(m, 8), 256, 0, s>>>(csrRowPtr, m, nnz, static_cast<int32_t>(base), csrColInd, P, permIn);
    SortLongRowsKernel<<<592, 256, 0, s>>>(csrRowPtr, m, nnz, static_cast<int32_t>(base), csrColInd, P, permIn, order);
    return cudaPeekAtLastError() == cudaSuccess ? ACL_SPARSE_STATUS_SUCCESS : ACL_SPARSE_STATUS_EXECUTION_FAILED;
}
