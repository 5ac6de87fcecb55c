/*
 * Preprocessing pass shared by SpMV and SpMM: builds the plan that both keep in
 * the caller's external buffer (layout in plan_layout.h).  Everything runs on
 * the device, asynchronously on the caller's stream, with no host round trip:
 * one-shot callers preprocess on every product, so the pass has to stay a few
 * O(rows) kernels.  The reference's SpMV preprocess normalises the row offsets
 * on a single core (sparse/spmv/arch35/spmv_kernel.cpp:1144-1163) and its SpMM
 * preprocess sorts rows on the host between two synchronous copies
 * (sparse/spmm/arch35/host/spmm_csr_mat.cpp:119-210).
 *
 * All results are integers and are reproduced bit for bit by the CPU twin in
 * the test oracle.
 */
#include <cstdint>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "plan_kernels.h"
#include "plan_layout.h"

namespace {

__device__ __forceinline__ int ClampOffset(int v, int nnz)
{
    return v < 0 ? 0 : (v > nnz ? nnz : v);
}

// dst[i] = src[i * stride] - base for i in [0, rows]; with `longest` non-null also the longest row
// (src[(i + 1) * stride] - src[i * stride], negative counted as 0), one atomicMax per warp.
__global__ void NormalizeRowOffsetsKernel(const int32_t* __restrict__ src, int32_t* __restrict__ dst, uint32_t rows,
                                          int32_t indexBase, int64_t stride, uint32_t* __restrict__ longest)
{
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    int32_t best = 0;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i <= rows; i += step) {
        const int32_t here = src[i * stride];
        dst[i] = here - indexBase;
        if (longest != nullptr && i < rows) {
            const int64_t len = static_cast<int64_t>(src[(i + 1) * stride]) - here;
            const int32_t len32 = len > 0x7fffffff ? 0x7fffffff : static_cast<int32_t>(len);
            best = len32 > best ? len32 : best;
        }
    }
    if (longest != nullptr) {
        for (int o = 16; o > 0; o >>= 1) {
            const int32_t other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if ((threadIdx.x & 31) == 0 && best > 0) {
            atomicMax(longest, static_cast<uint32_t>(best));
        }
    }
}

// Row coordinate where diagonal `diag` crosses the merge path of
// (rowEnd[i] = rowPtr[i + 1], non-zero index j): the number of rows that end
// before the diagonal.  The non-zero coordinate is diag - row.
__device__ __forceinline__ int MergePathRow(const int32_t* __restrict__ rowPtr, int rows, int nnz, int64_t diag)
{
    int64_t lo = diag > nnz ? diag - nnz : 0;
    int64_t hi = diag < rows ? diag : rows;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (ClampOffset(rowPtr[mid + 1], nnz) <= diag - 1 - mid) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    return static_cast<int>(lo);
}

__global__ void TileSplitKernel(void* workspace, uint32_t rows, uint32_t cols, uint32_t nnz, int32_t indexBase,
                                uint32_t tileItems, uint32_t kind, uint32_t denseCols, uint32_t classDiv,
                                AclspPlanLayout layout)
{
    auto* base = static_cast<unsigned char*>(workspace);
    const auto* rowPtr = reinterpret_cast<const int32_t*>(base + layout.rowPtrOff);
    auto* tileRow = reinterpret_cast<int32_t*>(base + layout.tileRowOff);
    auto* tileClass = reinterpret_cast<int32_t*>(base + layout.tileClassOff);
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t == 0) {
        AclspPlanHeader h;
        h.magic = ACLSP_PLAN_MAGIC;
        h.version = ACLSP_PLAN_VERSION;
        h.kind = kind;
        h.tileItems = tileItems;
        h.rows = rows;
        h.cols = cols;
        h.nnz = nnz;
        h.indexBase = static_cast<uint32_t>(indexBase);
        h.numTiles = layout.numTiles;
        h.denseCols = denseCols;
        h.rowPtrOff = layout.rowPtrOff;
        h.tileRowOff = layout.tileRowOff;
        h.tileClassOff = layout.tileClassOff;
        h.carryOff = layout.carryOff;
        h.totalBytes = layout.totalBytes;
        *reinterpret_cast<AclspPlanHeader*>(base) = h;
    }
    if (t >= layout.numTiles) {
        return;
    }
    const int64_t total = static_cast<int64_t>(rows) + nnz;
    int64_t d0 = static_cast<int64_t>(t) * tileItems;
    int64_t d1 = d0 + tileItems;
    d0 = d0 < total ? d0 : total;
    d1 = d1 < total ? d1 : total;
    const int r0 = MergePathRow(rowPtr, static_cast<int>(rows), static_cast<int>(nnz), d0);
    const int r1 = MergePathRow(rowPtr, static_cast<int>(rows), static_cast<int>(nnz), d1);
    tileRow[t] = r0;
    if (t == layout.numTiles - 1) {
        tileRow[t + 1] = r1;
    }
    const int64_t nr = static_cast<int64_t>(r1) - r0;
    const int64_t nt = (d1 - r1) - (d0 - r0);
    tileClass[t] = (nr < 0 || nt < 0) ? 0
                                      : static_cast<int32_t>(aclspTileClass(static_cast<uint32_t>(nr),
                                                                            static_cast<uint32_t>(nt), classDiv));
}

/* ------------------------------------------------------ row-block split -- */

__global__ void RowBlockBoundsKernel(const int32_t* __restrict__ rowPtr, uint32_t rows, uint32_t nnz,
                                     int32_t indexBase, uint32_t parts, int32_t* __restrict__ bounds)
{
    const uint32_t g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g > parts) {
        return;
    }
    // Smallest row r with rowPtr[r] - base >= ceil(g * nnz / parts).
    const int64_t target = (static_cast<int64_t>(g) * nnz + parts - 1) / parts;
    int64_t lo = 0;
    int64_t hi = rows;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(rowPtr[mid]) - indexBase >= target) {
            hi = mid;
        } else {
            lo = mid + 1;
        }
    }
    bounds[g] = g == parts ? static_cast<int32_t>(rows) : static_cast<int32_t>(lo);
}

}  // namespace

void AclspLaunchPlanBuild(const void* rowPtr, void* workspace, uint32_t rows, uint32_t cols, uint32_t nnz,
                          int32_t indexBase, int64_t rowOffsetsStride, uint32_t kind, uint32_t denseCols,
                          cudaStream_t stream)
{
    AclspPlanLayout layout;
    uint32_t tileItems = ACLSP_SPMV_TILE_ITEMS;
    uint32_t classDiv = ACLSP_SPMV_CLASS_DIV;
    if (kind == ACLSP_KIND_SPMM) {
        aclspSpmmLayout(rows, nnz, denseCols, &layout);
        tileItems = ACLSP_SPMM_TILE_ITEMS;
        classDiv = 1u;
    } else {
        aclspSpmvLayout(rows, nnz, &layout);
    }
    auto* bytes = static_cast<unsigned char*>(workspace);
    auto* dst = reinterpret_cast<int32_t*>(bytes + layout.rowPtrOff);
    // The counters behind the header proper (bounded waits that ran out, longest row) start at zero.
    cudaMemsetAsync(bytes + ACLSP_HEADER_WAIT_FAILURES_OFF, 0, ACLSP_HEADER_BYTES - ACLSP_HEADER_WAIT_FAILURES_OFF,
                    stream);
    auto* longest = kind == ACLSP_KIND_SPMV ? reinterpret_cast<uint32_t*>(bytes + ACLSP_HEADER_MAX_ROW_LEN_OFF)
                                            : nullptr;
    const uint64_t entries = static_cast<uint64_t>(rows) + 1u;
    uint64_t blocks = (entries + 255u) / 256u;
    blocks = blocks > 148u * 16u ? 148u * 16u : blocks;
    AclspCountLaunches(1);
    NormalizeRowOffsetsKernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const int32_t*>(rowPtr), dst, rows, indexBase, rowOffsetsStride, longest);
    const uint32_t splitBlocks = (layout.numTiles + 1u + 127u) / 128u;
    AclspCountLaunches(1);
    TileSplitKernel<<<splitBlocks, 128, 0, stream>>>(workspace, rows, cols, nnz, indexBase, tileItems, kind,
                                                     denseCols, classDiv, layout);
}

extern "C" void spmv_b200_preprocess_kernel_do(const void* rowPtr, void* workspace, uint32_t rows, uint32_t cols,
                                               uint32_t nnz, int32_t indexBase, int64_t rowOffsetsStride,
                                               void* stream)
{
    AclspLaunchPlanBuild(rowPtr, workspace, rows, cols, nnz, indexBase, rowOffsetsStride, ACLSP_KIND_SPMV, 1u,
                         static_cast<cudaStream_t>(stream));
}

extern "C" void spmm_b200_preprocess_kernel_do(const void* rowPtr, void* workspace, uint32_t rows, uint32_t cols,
                                               uint32_t nnz, uint32_t denseCols, int32_t indexBase, void* stream)
{
    AclspLaunchPlanBuild(rowPtr, workspace, rows, cols, nnz, indexBase, 1, ACLSP_KIND_SPMM, denseCols,
                         static_cast<cudaStream_t>(stream));
}

extern "C" void aclsp_b200_row_block_bounds_kernel_do(const void* rowPtr, uint32_t rows, uint32_t nnz,
                                                      int32_t indexBase, uint32_t parts, void* bounds, void* stream)
{
    AclspCountLaunches(1);
    RowBlockBoundsKernel<<<(parts + 1u + 63u) / 64u, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int32_t*>(rowPtr), rows, nnz, indexBase, parts, static_cast<int32_t*>(bounds));
}
