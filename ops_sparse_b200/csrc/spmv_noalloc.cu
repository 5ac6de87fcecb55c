/*
 * aclsparseB200SpMVNoAlloc: CSR SpMV for callers that must not allocate.
 *
 * The regular three-phase API asks the caller for an external buffer that holds
 * the row-partition plan and the per-tile carries.  Some callers cannot supply
 * one: code that runs where device allocation is forbidden or too slow - inside
 * a latency-critical loop whose memory was fixed at start-up, under a framework
 * allocator that owns all of device memory, or in a plug-in that is only handed
 * its operands.  For them this entry point keeps that scratch in a file-scope
 * device array of fixed size, so the call itself allocates nothing: no
 * cudaMalloc / cudaFree, no allocating library routine.
 *
 * The array lives in every CUDA context that loads this library until the
 * process exits, which is why it is kept modest (kScratchBytes).  Its name is
 * a device symbol: host code cannot pass `gScratch` itself to a kernel, it has
 * to ask the runtime for the symbol's device address, once per device, with
 * that device current.  The first call on a device does this
 * (cudaGetSymbolAddress) and caches the answer.  Under lazy module loading
 * that first call is also what loads this library's device code, the array
 * with it: it can take device memory once.  Make it at start-up, outside any
 * stream capture; only the calls after it are allocation-free.
 *
 * All calls on a device share the one array, and it keeps the contents of the
 * previous call.  Nothing in it has to start at zero - every call rewrites the
 * header, the row offsets, the tile table and every tile's carry slots before
 * they are read - but two calls that overlap on the GPU (different streams, or
 * different host threads without ordering) race on it.  Run them in stream
 * order.
 */
#include <cstdint>
#include <cstdio>
#include <mutex>

#include <cuda_runtime.h>

#include "aclsparse_b200_ext.h"
#include "aclsparse_b200_kernels.h"
#include "plan_layout.h"

namespace {

constexpr size_t kScratchBytes = 8u * 1024u * 1024u;  // plan of e.g. 1 M rows with 60 M non-zeros
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char gScratch[kScratchBytes];

std::mutex gSetupMutex;
void* gScratchAddress[kMaxDevices];
bool gScratchReady[kMaxDevices];

// Device address of gScratch on the current device; looked up on the first call per device.
aclsparseStatus_t ScratchAddress(void** out)
{
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_NOT_INITIALIZED;
    }
    std::lock_guard<std::mutex> lock(gSetupMutex);
    if (!gScratchReady[device]) {
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, gScratch);
        if (err != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            std::fprintf(stderr, "[aclsparse] aclsparseB200SpMVNoAlloc: cudaGetSymbolAddress failed: %s\n",
                         cudaGetErrorString(err));
            return ACL_SPARSE_STATUS_INTERNAL_ERROR;
        }
        gScratchAddress[device] = ptr;
        gScratchReady[device] = true;
    }
    *out = gScratchAddress[device];
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

extern "C" aclsparseStatus_t aclsparseB200SpMVNoAlloc(aclrtStream stream, int64_t rows, int64_t cols, int64_t nnz,
                                                      const int32_t* rowOffsets, const int32_t* colInd,
                                                      const float* values, aclsparseIndexBase_t idxBase,
                                                      const float* x, float* y, float alpha, float beta)
{
    if (rows < 0 || cols < 0 || nnz < 0 || (nnz > 0 && (rows == 0 || cols == 0)) ||
        (idxBase != ACL_SPARSE_INDEX_BASE_ZERO && idxBase != ACL_SPARSE_INDEX_BASE_ONE)) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (rows > 0x7FFFFFFF || cols > 0x7FFFFFFF || nnz > 0x7FFFFFFE) {
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (rows == 0) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (rowOffsets == nullptr || y == nullptr || (cols > 0 && x == nullptr) ||
        (nnz > 0 && (colInd == nullptr || values == nullptr))) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    AclspPlanLayout layout;
    aclspSpmvLayout(static_cast<uint64_t>(rows), static_cast<uint64_t>(nnz), &layout);
    if (layout.totalBytes > kScratchBytes) {
        std::fprintf(stderr,
                     "[aclsparse] aclsparseB200SpMVNoAlloc: a matrix with %lld rows and %lld non-zeros needs %llu bytes "
                     "of scratch, the built-in scratch holds %zu; use aclsparseSpMV with an external buffer\n",
                     static_cast<long long>(rows), static_cast<long long>(nnz),
                     static_cast<unsigned long long>(layout.totalBytes), kScratchBytes);
        return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
    }
    void* scratch = nullptr;
    const aclsparseStatus_t st = ScratchAddress(&scratch);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }

    AclspSpmvParams params{};
    params.rows = static_cast<uint32_t>(rows);
    params.cols = static_cast<uint32_t>(cols);
    params.nnz = static_cast<uint32_t>(nnz);
    params.indexBase = static_cast<uint32_t>(idxBase);
    params.colIndStride = 1;
    params.valuesStride = 1;
    params.xStride = 1;
    params.yStride = 1;
    params.alpha = alpha;
    params.beta = beta;
    params.maxRowLenHint = ACLSP_MAX_ROW_LEN_UNKNOWN;  // the plan was built a moment ago: the kernels decide

    (void)cudaGetLastError();
    spmv_b200_preprocess_kernel_do(rowOffsets, scratch, params.rows, params.cols, params.nnz,
                                   static_cast<int32_t>(idxBase), 1, stream);
    spmv_b200_kernel_do(colInd, values, x, y, scratch, &params, stream);
    if (cudaPeekAtLastError() != cudaSuccess) {
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}
