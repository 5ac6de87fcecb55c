/*
 * op(A) = transpose for SpMV and SpMM: the transpose of the CSR matrix is built
 * once, by the preprocessing pass, inside the caller's external buffer, as a
 * CSR matrix of its own (row offsets, column indices = the original row
 * numbers, and the permutation that carries the values over), and the
 * non-transposed kernels then run on it.  Only the values are moved per
 * product (one gather through the permutation), so a caller may change them
 * between products (aclsparseSpMatSetValues) without preprocessing again.
 *
 * The reference has three transposed SpMV kernels (atomics, sorted gather, one
 * serial thread: sparse/spmv/arch35/spmv_kernel.cpp:579-879) and builds a CSC
 * copy on the host for SpMM (sparse/spmm/arch35/host/spmm_csr_mat.cpp:212-315,
 * values permuted by kernel/spmm_kernel_transpose.cpp:62).  Here everything
 * stays on the device and nothing is added with atomics: the result is
 * bit-reproducible, as the reference promises for its deterministic variant.
 *
 * Build = a counting sort of the entries by column that keeps entries of one
 * column in their original order:
 *   1. count the entries of every column (integer atomics: the counts do not
 *      depend on the order of arrival) and note the row of every entry;
 *   2. inclusive scan of the counts: the row offsets of the transpose;
 *   3. give every entry a slot of its column (atomic cursor: the order inside
 *      a column is arbitrary at this point);
 *   4. sort the entry numbers inside every column ascending, which is the
 *      original order: a warp ranks up to 32 entries with shuffles, longer
 *      columns are put on a list and sorted by a CTA (bitonic network in
 *      shared memory up to 2048 entries, in global memory beyond);
 *   5. the column index of a transposed entry is the row of the entry it
 *      came from.
 * All of it is integer work and is reproduced bit for bit by the CPU twin in
 * the test oracle.  Entries whose column is out of range are left out, as the
 * kernels skip them; row offsets are clamped to [0, nnz].
 */
#include <cstdint>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "plan_kernels.h"
#include "plan_layout.h"

namespace {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 4;
constexpr int kScanTile = kScanThreads * kScanItems;
constexpr int kSortSmem = 2048;  // longest column sorted in shared memory

__device__ __forceinline__ int ClampOffset(int v, int nnz)
{
    return v < 0 ? 0 : (v > nnz ? nnz : v);
}

// One warp per row: counts[col + 1] += 1 for every entry with a valid column, rowOf[e] = row
// (-1 for entries that are left out).  Entries not covered by any row keep the -1 they start with.
__global__ void CountColumnsKernel(const int32_t* __restrict__ rowPtr, const int32_t* __restrict__ colInd,
                                   uint32_t rows, uint32_t cols, uint32_t nnz, int32_t indexBase, int64_t rowPtrStride,
                                   int64_t colIndStride, int32_t* __restrict__ counts, int32_t* __restrict__ rowOf)
{
    const int lane = threadIdx.x & 31;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x >> 5);
    for (uint64_t r = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const int b = ClampOffset(rowPtr[r * rowPtrStride] - indexBase, static_cast<int>(nnz));
        const int e = ClampOffset(rowPtr[(r + 1) * rowPtrStride] - indexBase, static_cast<int>(nnz));
        for (int q = b + lane; q < e; q += 32) {
            const uint32_t c = static_cast<uint32_t>(colInd[static_cast<int64_t>(q) * colIndStride]) -
                               static_cast<uint32_t>(indexBase);
            if (c < cols) {
                atomicAdd(&counts[c + 1u], 1);
                rowOf[q] = static_cast<int32_t>(r);
            }
        }
    }
}

__global__ void FillKernel(int32_t* __restrict__ dst, uint64_t n, int32_t value)
{
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {
        dst[i] = value;
    }
}

// Inclusive scan of kScanTile items per CTA, in place; the CTA's total goes to sums[blockIdx.x].
__global__ void __launch_bounds__(kScanThreads)
ScanTilesKernel(int32_t* __restrict__ data, uint64_t n, int32_t* __restrict__ sums)
{
    __shared__ int32_t warpTotals[kScanThreads / 32];
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kScanTile + static_cast<uint64_t>(threadIdx.x) * kScanItems;
    int32_t v[kScanItems];
    int32_t run = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        v[i] = base + i < n ? data[base + i] : 0;
        run += v[i];
        v[i] = run;
    }
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    int32_t incl = run;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int32_t up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) {
            incl += up;
        }
    }
    if (lane == 31) {
        warpTotals[warp] = incl;
    }
    __syncthreads();
    int32_t before = incl - run;
    for (int w = 0; w < warp; ++w) {
        before += warpTotals[w];
    }
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
        if (base + i < n) {
            data[base + i] = v[i] + before;
        }
    }
    if (threadIdx.x == kScanThreads - 1) {
        sums[blockIdx.x] = before + run;
    }
}

// data[i] += sums[tile(i) - 1] for every tile but the first (sums already scanned inclusively).
__global__ void AddTileOffsetsKernel(int32_t* __restrict__ data, uint64_t n, const int32_t* __restrict__ sums)
{
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x + kScanTile; i < n; i += step) {
        data[i] += sums[i / kScanTile - 1];
    }
}

// Every kept entry takes the next free slot of its column.
__global__ void PlaceEntriesKernel(const int32_t* __restrict__ colInd, const int32_t* __restrict__ rowOf, uint32_t nnz,
                                   int32_t indexBase, int64_t colIndStride, const int32_t* __restrict__ rowPtrT,
                                   int32_t* __restrict__ cursor, int32_t* __restrict__ perm)
{
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t q = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; q < nnz; q += step) {
        if (rowOf[q] >= 0) {
            const uint32_t c = static_cast<uint32_t>(colInd[static_cast<int64_t>(q) * colIndStride]) -
                               static_cast<uint32_t>(indexBase);
            perm[rowPtrT[c] + atomicAdd(&cursor[c], 1)] = static_cast<int32_t>(q);
        }
    }
}

// One warp per column: up to 32 entry numbers are ranked by counting (they are distinct) and
// written back in ascending order; longer columns go onto the list for SortLongColumnsKernel.
__global__ void SortShortColumnsKernel(const int32_t* __restrict__ rowPtrT, uint32_t cols, int32_t* __restrict__ perm,
                                       int32_t* __restrict__ longList, int32_t* __restrict__ longCount)
{
    const int lane = threadIdx.x & 31;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x >> 5);
    for (uint64_t c = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); c < cols; c += warps) {
        const int b = rowPtrT[c];
        const int len = rowPtrT[c + 1] - b;
        if (len <= 1) {
            continue;
        }
        if (len > 32) {
            if (lane == 0) {
                longList[atomicAdd(longCount, 1)] = static_cast<int32_t>(c);
            }
            continue;
        }
        const int32_t mine = lane < len ? perm[b + lane] : 0x7fffffff;
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            rank += __shfl_sync(0xffffffffu, mine, j) < mine ? 1 : 0;
        }
        __syncwarp();
        if (lane < len) {
            perm[b + rank] = mine;
        }
    }
}

// Sorting network with every comparator ascending (the first step of a merge mirrors, the others
// shift), so that missing elements above `len` behave like +infinity and are simply not touched.
template <typename Get, typename Swap>
__device__ __forceinline__ void BitonicAscending(int len, Get get, Swap swapIfGreater)
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
    (void)get;
}

// Persistent CTAs take the listed columns one by one.
__global__ void __launch_bounds__(256)
SortLongColumnsKernel(const int32_t* __restrict__ rowPtrT, int32_t* __restrict__ perm,
                      const int32_t* __restrict__ longList, const int32_t* __restrict__ longCount)
{
    __shared__ int32_t sKeys[kSortSmem];
    const int count = *longCount;
    for (int w = blockIdx.x; w < count; w += gridDim.x) {
        const int c = longList[w];
        const int b = rowPtrT[c];
        const int len = rowPtrT[c + 1] - b;
        int32_t* seg = perm + b;
        if (len <= kSortSmem) {
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                sKeys[i] = seg[i];
            }
            __syncthreads();
            BitonicAscending(
                len, [&](int i) { return sKeys[i]; },
                [&](int i, int l) {
                    const int32_t a = sKeys[i];
                    const int32_t z = sKeys[l];
                    if (a > z) {
                        sKeys[i] = z;
                        sKeys[l] = a;
                    }
                });
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                seg[i] = sKeys[i];
            }
            __syncthreads();
        } else {
            BitonicAscending(
                len, [&](int i) { return seg[i]; },
                [&](int i, int l) {
                    const int32_t a = seg[i];
                    const int32_t z = seg[l];
                    if (a > z) {
                        seg[i] = z;
                        seg[l] = a;
                    }
                });
        }
    }
}

// colIndT[p] = row of the entry that slot p holds.
__global__ void FillTransposedColumnsKernel(const int32_t* __restrict__ perm, const int32_t* __restrict__ rowOf,
                                            const int32_t* __restrict__ rowPtrT, uint32_t cols,
                                            int32_t* __restrict__ colIndT)
{
    const uint64_t kept = static_cast<uint64_t>(rowPtrT[cols]);
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t p = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < kept; p += step) {
        colIndT[p] = rowOf[perm[p]];
    }
}

// valuesT[p] = values[perm[p]]; slots beyond the kept entries are zeroed so that nothing
// uninitialised is ever multiplied.
// T: an unsigned integer as wide as an element (the bits are moved, not interpreted; zero bits are 0 in
// every element type).
template <typename T>
__global__ void GatherValuesKernel(const T* __restrict__ values, int64_t valuesStride,
                                   const int32_t* __restrict__ perm, const int32_t* __restrict__ rowPtrT, uint32_t cols,
                                   uint32_t nnz, T* __restrict__ valuesT)
{
    const uint64_t kept = static_cast<uint64_t>(rowPtrT[cols]);
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t p = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < nnz; p += step) {
        valuesT[p] = p < kept ? values[static_cast<int64_t>(perm[p]) * valuesStride] : static_cast<T>(0);
    }
}

template <typename T>
void LaunchGatherValues(const void* values, int64_t valuesStride, const int32_t* perm, const int32_t* rowPtrT,
                        uint32_t cols, uint32_t nnz, void* valuesT, unsigned grid, cudaStream_t s)
{
    GatherValuesKernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(values), valuesStride, perm, rowPtrT, cols, nnz,
                                              static_cast<T*>(valuesT));
}

unsigned GridFor(uint64_t items, unsigned perBlock)
{
    uint64_t blocks = (items + perBlock - 1) / perBlock;
    blocks = blocks < 1 ? 1 : (blocks > 148u * 32u ? 148u * 32u : blocks);
    return static_cast<unsigned>(blocks);
}

// Inclusive scan of data[0, n) in place; temp holds the per-tile totals of every level.
void InclusiveScan(int32_t* data, uint64_t n, int32_t* temp, cudaStream_t s)
{
    if (n == 0) {
        return;
    }
    const uint64_t tiles = (n + kScanTile - 1) / kScanTile;
    AclspCountLaunches(1);
    ScanTilesKernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, s>>>(data, n, temp);
    if (tiles > 1) {
        InclusiveScan(temp, tiles, temp + tiles, s);
        AclspCountLaunches(1);
        AddTileOffsetsKernel<<<GridFor(n, 256), 256, 0, s>>>(data, n, temp);
    }
}

}  // namespace

extern "C" void aclsp_b200_transpose_build_kernel_do(const void* rowPtr, const void* colInd, uint32_t rows,
                                                     uint32_t cols, uint32_t nnz, int32_t indexBase,
                                                     int64_t rowPtrStride, int64_t colIndStride, void* workspace,
                                                     const AclspTransposeLayout* layout, void* stream)
{
    auto s = static_cast<cudaStream_t>(stream);
    auto* base = static_cast<unsigned char*>(workspace);
    auto* rowPtrT = reinterpret_cast<int32_t*>(base + layout->rowPtrOff);
    auto* colIndT = reinterpret_cast<int32_t*>(base + layout->colIndOff);
    auto* perm = reinterpret_cast<int32_t*>(base + layout->permOff);
    auto* rowOf = reinterpret_cast<int32_t*>(base + layout->valuesOff);  // free until the first product
    auto* cursor = reinterpret_cast<int32_t*>(base + layout->cursorOff);
    auto* scanTemp = reinterpret_cast<int32_t*>(base + layout->scanOff);
    const auto* rp = static_cast<const int32_t*>(rowPtr);
    const auto* ci = static_cast<const int32_t*>(colInd);

    cudaMemsetAsync(rowPtrT, 0, sizeof(int32_t) * (static_cast<size_t>(cols) + 1u), s);
    cudaMemsetAsync(cursor, 0, sizeof(int32_t) * (static_cast<size_t>(cols) + 2u), s);
    if (nnz > 0) {
        AclspCountLaunches(2);
        FillKernel<<<GridFor(nnz, 256), 256, 0, s>>>(rowOf, nnz, -1);
        CountColumnsKernel<<<GridFor(rows, 8), 256, 0, s>>>(rp, ci, rows, cols, nnz, indexBase, rowPtrStride,
                                                            colIndStride, rowPtrT, rowOf);
    }
    InclusiveScan(rowPtrT + 1, cols, scanTemp, s);
    if (nnz > 0) {
        AclspCountLaunches(4);
        PlaceEntriesKernel<<<GridFor(nnz, 256), 256, 0, s>>>(ci, rowOf, nnz, indexBase, colIndStride, rowPtrT, cursor,
                                                            perm);
        // The cursors are done with: their array now holds the list of long columns, its counter behind it.
        int32_t* longCount = cursor + cols + 1u;
        SortShortColumnsKernel<<<GridFor(cols, 8), 256, 0, s>>>(rowPtrT, cols, perm, cursor, longCount);
        SortLongColumnsKernel<<<592, 256, 0, s>>>(rowPtrT, perm, cursor, longCount);
        FillTransposedColumnsKernel<<<GridFor(nnz, 256), 256, 0, s>>>(perm, rowOf, rowPtrT, cols, colIndT);
    }
}

extern "C" void aclsp_b200_transpose_values_kernel_do(const void* values, int64_t valuesStride, uint32_t cols,
                                                      uint32_t nnz, void* workspace,
                                                      const AclspTransposeLayout* layout, uint32_t elemBytes,
                                                      void* stream)
{
    if (nnz == 0) {
        return;
    }
    auto* base = static_cast<unsigned char*>(workspace);
    const auto* perm = reinterpret_cast<const int32_t*>(base + layout->permOff);
    const auto* rowPtrT = reinterpret_cast<const int32_t*>(base + layout->rowPtrOff);
    void* valuesT = base + layout->valuesOff;
    const unsigned grid = GridFor(nnz, 256);
    auto s = static_cast<cudaStream_t>(stream);
    AclspCountLaunches(1);
    if (elemBytes == 1) {
        LaunchGatherValues<uint8_t>(values, valuesStride, perm, rowPtrT, cols, nnz, valuesT, grid, s);
    } else if (elemBytes == 2) {
        LaunchGatherValues<uint16_t>(values, valuesStride, perm, rowPtrT, cols, nnz, valuesT, grid, s);
    } else {
        LaunchGatherValues<uint32_t>(values, valuesStride, perm, rowPtrT, cols, nnz, valuesT, grid, s);
    }
}
