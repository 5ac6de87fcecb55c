/*
 * CSR SpMM for sm_100a:  C = alpha * A * op(B) + beta * C,  int32 indices, fp32 (and narrow storage types).
 *
 * No tensor cores: at 16-32 non-zeros per row the product is a gather of rows
 * of B, not a dense contraction.
 *
 * Work decomposition.  As for SpMV the matrix is cut along the merge path of
 * (row ends, non-zeros), here into tiles of 1024 items, one CTA per tile, and
 * the CTA cuts its tile once more the same way into equal pieces, one per
 * LANE GROUP.  A group is a warp (eight 128-item pieces) when C has 128
 * columns or more; for narrower C it is as few lanes as cover a row of C in
 * one pass (16 lanes for n <= 64, 8 for n <= 32), so that one warp instruction
 * works on two or four non-zeros.  A group streams at most its piece whatever
 * the row lengths are: a 500 000-entry row is spread over thousands of groups
 * and a run of empty rows costs as much as a run of non-zeros.
 *   1. The CTA stages (column, value) of the tile's non-zeros as one word
 *      pair each in shared memory, from coalesced 128-bit loads (evict-first).
 *   2. Each group walks its non-zeros in order.  For every non-zero the lanes
 *      copy one row of B (G*VW columns of it) into the group's ring of
 *      shared-memory stages with cp.async (.cg for 16-byte pieces: a row is
 *      used once), kStages rows ahead of the FMAs.  A lane reads back only the
 *      bytes it copied itself, so the ring needs no barrier, only
 *      cp.async.wait_group.  Four stages with four columns per lane: the
 *      rings are most of a CTA's shared memory, and resident CTAs matter more
 *      than depth (the kernel is bound on the SM side, not by DRAM).
 *   3. At a row end the accumulators are written as alpha*acc + beta*C.  The
 *      piece of a row that a group shares with its neighbours goes to shared
 *      memory and is combined in group order; the pieces a tile shares with
 *      its neighbours go to the plan's carry area and are combined in tile
 *      order by a second kernel.  All orders are fixed: results are
 *      reproducible.
 *
 * Accuracy.  Products and row sums are fp64 (exact products of fp32 factors,
 * which cannot overflow), alpha * sum + beta * C is evaluated in fp64 and
 * rounded once: a row equals the reference's fp64 test golden (SpmmGolden,
 * test/spmm_op/spmm_op_golden.h:142-205) up to the order of the additions,
 * whatever the data, for every algorithm value.
 *
 * Layouts.  VW in {4, 2, 1} floats per lane is the widest vector the operands
 * allow (unit column stride of op(B) and C, leading dimensions and base
 * addresses aligned to the vector).  VW = 1 addresses both matrices through
 * (row stride, column stride) pairs and so also covers column-major B / C and
 * op(B) = transpose.
 *
 * Element types.  fp16 / bf16 / int8 values and B with C of the same type,
 * fp32 or (int8) saturating int32 run the VW = 1 form without staging on typed
 * loads and stores (element_types.cuh); their products are exact in fp64 too.
 *
 * Out-of-range input never faults: offsets are clamped and entries whose
 * column falls outside [0, k) are skipped (reference:
 * sparse/spmm/arch35/kernel/spmm_kernel_simt.cpp:406-434 clamps alike).
 */
#include <cstdint>
#include <cstdlib>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "element_types.cuh"
#include "node_barrier.cuh"
#include "plan_kernels.h"
#include "plan_layout.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTile = ACLSP_SPMM_TILE_ITEMS;
constexpr int kMaxStages = 8;

using aclsp::kF32;
using aclsp::LoadIn;

struct SpmmPlanView {
    const int32_t* rowPtr;
    int32_t* tileRow;
    double* carry;  // [numTiles][2][n]: tail carry-out, head partial
    uint32_t numTiles;
};

inline SpmmPlanView MakeView(void* workspace, uint32_t rows, uint32_t nnz, uint32_t n)
{
    AclspPlanLayout l;
    aclspSpmmLayout(rows, nnz, n, &l);
    auto* base = static_cast<unsigned char*>(workspace);
    SpmmPlanView v;
    v.rowPtr = reinterpret_cast<const int32_t*>(base + l.rowPtrOff);
    v.tileRow = reinterpret_cast<int32_t*>(base + l.tileRowOff);
    v.carry = reinterpret_cast<double*>(base + l.carryOff);
    v.numTiles = l.numTiles;
    return v;
}

// Element (r, c) of op(B) is B[r * bRow + c * bCol]; the same for C.
struct DenseStrides {
    int64_t bRow;
    int64_t bCol;
    int64_t cRow;
    int64_t cCol;
};

__device__ __forceinline__ int ClampOffset(int v, int nnz)
{
    return v < 0 ? 0 : (v > nnz ? nnz : v);
}

template <int VW>
struct Vec;
template <>
struct Vec<4> {
    using T = float4;
};
template <>
struct Vec<2> {
    using T = float2;
};
template <>
struct Vec<1> {
    using T = float;
};

// Store to an NVLink multicast address: the switch delivers it to every GPU.
__device__ __forceinline__ void MulticastStore(void* addr, const float4& v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(v.x), "f"(v.y),
                 "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void MulticastStore(void* addr, const float2& v)
{
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};\n" ::"l"(addr), "f"(v.x), "f"(v.y) : "memory");
}
__device__ __forceinline__ void MulticastStore(void* addr, const float& v)
{
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;\n" ::"l"(addr), "f"(v) : "memory");
}

template <int BYTES>
__device__ __forceinline__ void CpAsync(void* smem, const void* gmem)
{
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    if constexpr (BYTES == 16) {
        // A gathered row of B is used once by this CTA: keep it out of L1 (the .cg form exists for 16 bytes only).
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem) : "memory");
        return;
    }
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(dst), "l"(gmem), "n"(BYTES) : "memory");
}

__device__ __forceinline__ void CpAsyncCommit()
{
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}

template <int N>
__device__ __forceinline__ void CpAsyncWait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

struct Scalars {
    float alpha;
    float beta;
    bool betaZero;
};

__device__ __forceinline__ Scalars LoadScalars(const AclspSpmmParams& p)
{
    Scalars s;
    s.alpha = p.alphaPtr != nullptr ? *p.alphaPtr : p.alpha;
    s.beta = p.betaPtr != nullptr ? *p.betaPtr : p.beta;
    s.betaZero = s.beta == 0.0f;
    return s;
}

// Merge-path split of a tile held in shared memory: rows of the tile that end
// before local diagonal d.  sOff[k + 1] is the local end offset of row k.
__device__ __forceinline__ int LocalMergeRow(const int* sOff, int nr, int nt, int d)
{
    int lo = d > nt ? d - nt : 0;
    int hi = d < nr ? d : nr;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (sOff[mid + 1] <= d - 1 - mid) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    return lo;
}

// groups: lane groups per CTA (kThreads / G); a group's ring, tail and head hold G * vw columns, so the
// sizes of those arrays do not depend on G.
constexpr size_t SmemBytes(int vw, int groups, int stages)
{
    return sizeof(int) * (kTile + 2)                    // sOff
           + sizeof(int2) * kTile                       // sColVal
           + sizeof(float) * kThreads * stages * vw     // rings
           + sizeof(double) * kThreads * vw * (stages >= 2 ? 1 : 2)  // group heads; tails unless they fit the rings
           + sizeof(int) * (2 * groups + 2);            // group row split, head flags
}

// kIn != kF32 (narrow storage: fp16, bf16 or int8 values and B, C of type p.cType): `values`, `B` and `C`
// address elements of those types; only the one-column-per-lane form without staging exists (VW = 1,
// kStageB = false), which goes through element strides and so covers every layout.
template <int VW, bool kStageB, int kIn = kF32, int G = 32, int kStages = kMaxStages>
// (No minimum of resident CTAs is asked of the compiler: held to 48 registers for five CTAs per SM the
// four-stage instance was slower than with the 57 it takes by itself, c4 1.67 against 1.55 ms.)
__global__ void __launch_bounds__(kThreads)
SpmmTileKernel(const int32_t* __restrict__ colInd, const float* __restrict__ values, const float* __restrict__ B,
               float* __restrict__ C, SpmmPlanView plan, AclspSpmmParams p, DenseStrides ds)
{
    static_assert(kIn == kF32 || (VW == 1 && !kStageB), "narrow storage: one column per lane, no staging");
    static_assert(G == 32 || G == 16 || G == 8, "lane groups of 8, 16 or 32");
    using V = typename Vec<VW>::T;
    // A lane group is G lanes that walk one piece of the tile together, lane l on columns [l VW, (l+1) VW) of
    // the pass.  G = 32 is a warp; with narrower C (n <= 64, n <= 32) a warp holds two or four groups, each on
    // its own piece, so that one warp instruction still serves 32 * VW columns' worth of work.  Below, "warp"
    // in names and comments means such a group.
    constexpr int kGroups = kThreads / G;
    constexpr int kGroupItems = kTile / kGroups;
    constexpr int kPanel = G * VW;

    extern __shared__ __align__(16) unsigned char smemRaw[];
    // With staging, a group's tail (what it hands to the row that continues past it) is written after its walk
    // into the first half of its own ring, which nothing uses any more by then: the rings are most of the
    // CTA's shared memory, and shared memory decides how many CTAs an SM holds.
    constexpr bool kTailInRing = kStageB && kStages >= 2;
    constexpr int kTailStride = kTailInRing ? kStages * kPanel / 2 : kPanel;  // doubles between two groups' tails
    double* sHead = reinterpret_cast<double*>(smemRaw);                // [kGroups][kPanel]
    double* sTailOwn = sHead + kGroups * kPanel;                       // [kGroups][kPanel] unless kTailInRing
    float* sRing = reinterpret_cast<float*>(sTailOwn + (kTailInRing ? 0 : kGroups * kPanel)); // [kGroups][kStages][kPanel]
    double* sTail = kTailInRing ? reinterpret_cast<double*>(sRing) : sTailOwn;
    // [kTile] (column, value bits) of every non-zero, column -1 for a skipped entry: one load serves both.
    // (No rings without staging.)
    int2* sColVal = reinterpret_cast<int2*>(sRing + (kStageB ? kGroups * kStages * kPanel : 0));
    int* sOff = reinterpret_cast<int*>(sColVal + kTile);               // [kTile + 2]
    int* sWarpRow = sOff + kTile + 2;                                 // [kGroups + 1] first local row of each warp
    int* sHasHead = sWarpRow + kGroups + 1;                            // [kGroups]

    const int tid = threadIdx.x;
    const int lane = tid % G;
    const int warp = tid / G;
    const int t = blockIdx.x;
    const int nnz = static_cast<int>(p.nnz);
    const int n = static_cast<int>(p.n);
    const int64_t total = static_cast<int64_t>(p.rows) + nnz;
    int64_t d0 = static_cast<int64_t>(t) * kTile;
    int64_t d1 = d0 + kTile;
    d0 = d0 < total ? d0 : total;
    d1 = d1 < total ? d1 : total;
    const int i0 = plan.tileRow[t];
    const int i1 = plan.tileRow[t + 1];
    const int j0 = static_cast<int>(d0 - i0);
    const int j1 = static_cast<int>(d1 - i1);
    const int nr = i1 - i0;
    const int nt = j1 - j0;
    double* tileTail = plan.carry + static_cast<size_t>(2 * t) * n;
    double* tileHead = tileTail + n;
    if (nr < 0 || nt < 0 || nr + nt > kTile || i0 < 0 || i1 > static_cast<int>(p.rows) || j0 < 0 || j1 > nnz) {
        for (int c = tid; c < 2 * n; c += kThreads) {  // inconsistent row offsets: contribute nothing
            tileTail[c] = 0.0;
        }
        return;
    }

    // Stage the tile: local row offsets, column indices (base 0) and values.
    for (int k = tid; k <= nr; k += kThreads) {
        sOff[k] = ClampOffset(plan.rowPtr[i0 + k], nnz) - j0;
    }
    {
        const bool vector = kIn == kF32 &&
                            (reinterpret_cast<uintptr_t>(colInd) | reinterpret_cast<uintptr_t>(values)) % 16 == 0;
        const int a0 = vector ? (j0 & ~3) : j0;
        const int count = j1 - a0;
        for (int e = 4 * tid; e < count; e += 4 * kThreads) {
            int32_t c[4];
            float w[4];
            const int g = a0 + e;
            if (vector && g + 4 <= nnz) {
                const int4 cv = __ldcs(reinterpret_cast<const int4*>(colInd + g));
                const float4 wv = __ldcs(reinterpret_cast<const float4*>(values + g));
                c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w;
                w[0] = wv.x; w[1] = wv.y; w[2] = wv.z; w[3] = wv.w;
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const bool in = g + q < nnz;
                    c[q] = in ? __ldcs(colInd + g + q) : -1;
                    w[q] = in ? LoadIn<kIn>(values, g + q) : 0.0f;
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int k = g + q - j0;
                if (k >= 0 && k < nt) {
                    const uint32_t col = static_cast<uint32_t>(c[q]) - p.indexBase;
                    sColVal[k] = make_int2(col < p.cols ? static_cast<int>(col) : -1, __float_as_int(w[q]));
                }
            }
        }
    }
    __syncthreads();

    // This warp's piece of the tile: local rows [r0, r1) end in it, local
    // non-zeros [q0, q1) belong to it.
    const int items = nr + nt;
    int da = warp * kGroupItems;
    int db = da + kGroupItems;
    da = da < items ? da : items;
    db = db < items ? db : items;
    const int r0 = LocalMergeRow(sOff, nr, nt, da);
    const int r1 = LocalMergeRow(sOff, nr, nt, db);
    const int q0 = da - r0;
    const int q1 = db - r1;
    const bool headOpen = sOff[r0] < q0;  // row r0 began in an earlier warp or tile
    if (lane == 0) {
        sWarpRow[warp] = r0;
        sHasHead[warp] = (headOpen && r1 > r0) ? 1 : 0;
        if (warp == kGroups - 1) {
            sWarpRow[kGroups] = r1;
        }
    }

    const Scalars sc = LoadScalars(p);
    const uint32_t bRow32 = static_cast<uint32_t>(ds.bRow);  // strides are positive and below 2^31 (host check)
    const aclsp::TypedScalars tsc = aclsp::LoadTypedScalars(p.computeInt, p.alphaPtr, p.betaPtr, p.alpha, p.beta,
                                                            p.alphaInt, p.betaInt);
    (void)tsc;
    float* ring = sRing + warp * kStages * kPanel + lane * VW;
    const bool tileHeadOpen = sOff[0] < 0;

    for (int col0 = 0; col0 < n; col0 += kPanel) {
        const int colL = col0 + lane * VW;
        const bool colOk = colL < n;  // n is a multiple of VW whenever VW > 1
        const float* bLane = B + static_cast<int64_t>(colL) * ds.bCol;
        float* cLane = C + static_cast<int64_t>(colL) * ds.cCol;

        // The running sum of the row piece: an fp64 sum of fp64 products.  Products of fp32 factors are
        // exact in fp64 and cannot overflow, so a row equals the fp64 golden (SpmmGolden,
        // test/spmm_op/spmm_op_golden.h:142-205) up to the order of the additions, Inf and NaN included,
        // whatever the data.  Measured against fp32 FMA row sums on the gather-bound benchmark
        // configurations: 8 to 15 % more kernel time; fp32 sums miss the 1e-5 / 1e-6 tolerance on cancelling rows.
        double acc[VW];
#pragma unroll
        for (int v = 0; v < VW; ++v) {
            acc[v] = 0.0;
        }
        auto issue = [&](int q) {
            const int c = sColVal[q].x;
            if (c >= 0 && colOk) {
                // (a row index and a leading dimension both fit 31 bits: one 32 x 32 -> 64 bit multiply)
                CpAsync<4 * VW>(ring + (static_cast<unsigned>(q) % kStages) * kPanel,
                                bLane + static_cast<uint64_t>(static_cast<uint32_t>(c)) * bRow32);
            }
            CpAsyncCommit();
        };
        // C[row] = alpha * sum + beta * C[row]; beta == 0 never reads C.
        auto storeRow = [&](int localRow, const double (&sum)[VW]) {
            if (!colOk) {
                return;
            }
            if constexpr (kIn != kF32) {
                const int64_t at = static_cast<int64_t>(colL) * ds.cCol + static_cast<int64_t>(i0 + localRow) * ds.cRow;
                aclsp::StoreScaled(p.cType, C, at, C, at, sum[0], tsc);
                return;
            }
            float* dst = cLane + static_cast<int64_t>(i0 + localRow) * ds.cRow;
            V old;
            float* od = reinterpret_cast<float*>(&old);
            if (!sc.betaZero) {
                old = *reinterpret_cast<const V*>(dst);
            }
            V out;
            float* o = reinterpret_cast<float*>(&out);
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                const double r = static_cast<double>(sc.alpha) * sum[v];
                o[v] = static_cast<float>(sc.betaZero ? r : r + static_cast<double>(sc.beta) * od[v]);
            }
            *reinterpret_cast<V*>(dst) = out;
            // Mirrors of C (the other GPUs' result buffers when the matrix is
            // sharded) receive the same 32 * VW contiguous floats per warp.
            if (p.mirrorMulticast != 0) {
                MulticastStore(reinterpret_cast<char*>(dst) + p.mirrorDelta[0], out);
            } else {
                for (uint32_t m = 0; m < p.numMirrors; ++m) {
                    *reinterpret_cast<V*>(reinterpret_cast<char*>(dst) + p.mirrorDelta[m]) = out;
                }
            }
        };
        // A finished row goes to C, unless it is the warp's first row and its
        // beginning lies elsewhere: then it waits in shared memory.
        bool first = true;
        auto flush = [&](int localRow) {
            double sum[VW];
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                sum[v] = acc[v];
            }
            if (first && headOpen) {
                if (colOk) {
#pragma unroll
                    for (int v = 0; v < VW; ++v) {
                        sHead[warp * kPanel + lane * VW + v] = sum[v];
                    }
                }
            } else {
                storeRow(localRow, sum);
            }
            first = false;
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                acc[v] = 0.0;
            }
        };

        int row = r0;
        int rowEnd = row < nr ? sOff[row + 1] : nt + 1;  // the open tail row never ends here
        auto accumulate = [&](float a, const V& b) {
            const float* bv = reinterpret_cast<const float*>(&b);
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                acc[v] = fma(static_cast<double>(a), static_cast<double>(bv[v]), acc[v]);
            }
        };
        if (kStageB) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) {
                if (q0 + s < q1) {
                    issue(q0 + s);
                } else {
                    CpAsyncCommit();
                }
            }
            // One non-zero: wait for its row of B, add it in, start the copy kStages non-zeros ahead.
            auto step = [&](int q) {
                CpAsyncWait<kStages - 1>();
                const int2 cv = sColVal[q];
                if (cv.x >= 0 && colOk) {
                    accumulate(__int_as_float(cv.y),
                               *reinterpret_cast<const V*>(ring + (static_cast<unsigned>(q) % kStages) * kPanel));
                }
                if (q + kStages < q1) {
                    issue(q + kStages);
                } else {
                    CpAsyncCommit();
                }
            };
            if (nt >= 8 * (nr + 1)) {
                // Rows of eight non-zeros and more on average: walk to the next row end without a test per
                // non-zero (measured on c4, rows of 16: 1.47 against 1.60 ms).
                int q = q0;
                while (q < q1) {
                    while (rowEnd <= q && row < r1) {
                        flush(row);
                        ++row;
                        rowEnd = row < nr ? sOff[row + 1] : nt + 1;
                    }
                    const int stop = (row < r1 && rowEnd < q1) ? rowEnd : q1;  // no row ends before it
                    for (; q < stop; ++q) {
                        step(q);
                    }
                }
            } else {
                // Short rows: the inner loop above would be entered and left every few non-zeros (measured on
                // c5: 9.5 against 9.1 ms), so the row end is tested with every non-zero.
                for (int q = q0; q < q1; ++q) {
                    while (rowEnd <= q && row < r1) {
                        flush(row);
                        ++row;
                        rowEnd = row < nr ? sOff[row + 1] : nt + 1;
                    }
                    step(q);
                }
            }
        } else {
            // Rows of B straight into registers, kUnroll gathers in flight per lane.
            constexpr int kUnroll = 4;
            for (int q = q0; q < q1; q += kUnroll) {
                V b[kUnroll];
                float a[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int qq = q + u;
                    const int2 cv = qq < q1 ? sColVal[qq] : make_int2(-1, 0);
                    const int c = cv.x;
                    const bool ok = c >= 0 && colOk;
                    a[u] = ok ? __int_as_float(cv.y) : 0.0f;
                    if constexpr (kIn != kF32) {
                        *reinterpret_cast<float*>(&b[u]) =
                            ok ? LoadIn<kIn>(B, static_cast<int64_t>(colL) * ds.bCol + static_cast<int64_t>(c) * ds.bRow)
                               : 0.0f;
                    } else if (ok) {
                        b[u] = __ldg(reinterpret_cast<const V*>(bLane + static_cast<int64_t>(c) * ds.bRow));
                    } else {
                        float* z = reinterpret_cast<float*>(&b[u]);
#pragma unroll
                        for (int v = 0; v < VW; ++v) {
                            z[v] = 0.0f;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int qq = q + u;
                    if (qq < q1) {
                        while (rowEnd <= qq && row < r1) {
                            flush(row);
                            ++row;
                            rowEnd = row < nr ? sOff[row + 1] : nt + 1;
                        }
                        accumulate(a[u], b[u]);
                    }
                }
            }
        }
        while (row < r1) {
            flush(row);
            ++row;
        }
        CpAsyncWait<0>();  // this lane's copies have landed ...
        __syncwarp();      // ... and every lane of the warp has read what it needed from the rings
        if (colOk) {  // what is left belongs to the row that continues past this warp
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                sTail[warp * kTailStride + lane * VW + v] = acc[v];
            }
        }
        __syncthreads();

        // Rows shared between warps: add the tails of the warps the row
        // crossed, oldest first, then this warp's head piece.
        if (sHasHead[warp] != 0 && colOk) {
            int firstWarp = warp;
            while (firstWarp > 0 && sWarpRow[firstWarp] == r0) {
                --firstWarp;
            }
            double total[VW];
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                double sum = 0.0;
                for (int u = firstWarp; u < warp; ++u) {
                    sum += sTail[u * kTailStride + lane * VW + v];
                }
                total[v] = sum + sHead[warp * kPanel + lane * VW + v];
            }
            // The chain reaches back to the tile's first item exactly when the
            // row is the tile's first row; then an earlier tile holds more of it.
            if (r0 == 0 && tileHeadOpen) {
#pragma unroll
                for (int v = 0; v < VW; ++v) {
                    tileHead[colL + v] = total[v];
                }
            } else {
                storeRow(r0, total);
            }
        }
        if (warp == kGroups - 1 && colOk) {
            int firstWarp = kGroups;
            while (firstWarp > 0 && sWarpRow[firstWarp] == nr) {
                --firstWarp;
            }
#pragma unroll
            for (int v = 0; v < VW; ++v) {
                double sum = 0.0;
                for (int u = firstWarp; u < kGroups; ++u) {
                    sum += sTail[u * kTailStride + lane * VW + v];
                }
                tileTail[colL + v] = sum;
            }
        }
        __syncthreads();
    }
}

// One warp per tile whose first row began in an earlier tile and ends in this
// one: adds the tails of the tiles the row crossed, oldest first, then the head
// piece, and writes the row of C.
template <int kIn = kF32>
__global__ void SpmmCarryFixupKernel(float* __restrict__ C, SpmmPlanView plan, AclspSpmmParams p, DenseStrides ds)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warpsPerGrid = gridDim.x * (blockDim.x >> 5);
    const int nnz = static_cast<int>(p.nnz);
    const int n = static_cast<int>(p.n);
    const int64_t total = static_cast<int64_t>(p.rows) + nnz;
    const Scalars sc = LoadScalars(p);
    for (uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < plan.numTiles; t += warpsPerGrid) {
        const int i0 = plan.tileRow[t];
        const int i1 = plan.tileRow[t + 1];
        if (i1 <= i0 || i0 < 0 || i0 >= static_cast<int>(p.rows)) {
            continue;
        }
        int64_t d0 = static_cast<int64_t>(t) * kTile;
        d0 = d0 < total ? d0 : total;
        if (ClampOffset(plan.rowPtr[i0], nnz) >= d0 - i0) {
            continue;
        }
        uint32_t first = t;
        while (first > 0 && plan.tileRow[first] == i0) {
            --first;
        }
        for (int c = lane; c < n; c += 32) {
            double sum = 0.0;
            for (uint32_t u = first; u < t; ++u) {
                sum += plan.carry[static_cast<size_t>(2 * u) * n + c];
            }
            sum += plan.carry[static_cast<size_t>(2 * t + 1) * n + c];
            if constexpr (kIn != kF32) {
                const int64_t at = static_cast<int64_t>(i0) * ds.cRow + static_cast<int64_t>(c) * ds.cCol;
                aclsp::StoreScaled(p.cType, C, at, C, at, sum,
                                   aclsp::LoadTypedScalars(p.computeInt, p.alphaPtr, p.betaPtr, p.alpha, p.beta,
                                                           p.alphaInt, p.betaInt));
                continue;
            }
            float* dst = C + static_cast<int64_t>(i0) * ds.cRow + static_cast<int64_t>(c) * ds.cCol;
            const double r = static_cast<double>(sc.alpha) * sum;
            const float out = static_cast<float>(sc.betaZero ? r : r + static_cast<double>(sc.beta) * *dst);
            *dst = out;
            if (p.mirrorMulticast != 0) {
                MulticastStore(reinterpret_cast<char*>(dst) + p.mirrorDelta[0], out);
            } else {
                for (uint32_t m = 0; m < p.numMirrors; ++m) {
                    *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.mirrorDelta[m]) = out;
                }
            }
        }
    }
    aclsp::CloseWithNodeBarrier(p.barrier);  // this is the product's last kernel
}

template <int VW, bool kStageB, int G, int kStages = kMaxStages>
void Launch(const void* colInd, const void* values, const void* b, void* c, const SpmmPlanView& plan,
            const AclspSpmmParams& p, const DenseStrides& ds, cudaStream_t s)
{
    constexpr size_t smem = SmemBytes(VW, kThreads / G, kStageB ? kStages : 0);
    // More than 48 KiB of dynamic shared memory has to be requested per kernel
    // and per device; the attribute is cheap to set, so it is set every time.
    cudaFuncSetAttribute(SpmmTileKernel<VW, kStageB, kF32, G, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem));
    AclspCountLaunches(1);
    SpmmTileKernel<VW, kStageB, kF32, G, kStages><<<plan.numTiles, kThreads, smem, s>>>(
        static_cast<const int32_t*>(colInd), static_cast<const float*>(values), static_cast<const float*>(b),
        static_cast<float*>(c), plan, p, ds);
}

template <int VW, int G = 32>
void LaunchByPrecision(const void* colInd, const void* values, const void* b, void* c, const SpmmPlanView& plan,
                       const AclspSpmmParams& p, const DenseStrides& ds, cudaStream_t s)
{
    // Rows of B are staged in shared memory with cp.async by default;
    // ACLSPARSE_SPMM_STAGE_B=0 selects the variant that reads them straight into
    // registers (both run at the same speed on the gather-bound configurations).
    static const bool stage = [] {
        const char* e = std::getenv("ACLSPARSE_SPMM_STAGE_B");
        return e == nullptr || e[0] != '0';
    }();
    // Ring depth (gathers in flight per lane group).  With four columns per lane the rings are the largest
    // part of a CTA's shared memory and decide how many CTAs an SM holds: four stages (5 CTAs per SM) beat
    // eight (3 CTAs) on the benchmark configurations, c4 1.55 against 1.69 ms, c5 8.6 against 10.0 ms; two are
    // no better than four.  ACLSPARSE_SPMM_STAGES=8 / 4 / 2 overrides the choice (read once).
    static const int stagesEnv = [] {
        const char* e = std::getenv("ACLSPARSE_SPMM_STAGES");
        return e == nullptr ? 0 : std::atoi(e);
    }();
    const int stages = stagesEnv != 0 ? stagesEnv : (VW == 4 ? 4 : 8);
    if (stage && stages == 4) {
        Launch<VW, true, G, 4>(colInd, values, b, c, plan, p, ds, s);
    } else if (stage && stages == 2) {
        Launch<VW, true, G, 2>(colInd, values, b, c, plan, p, ds, s);
    } else if (stage) {
        Launch<VW, true, G, 8>(colInd, values, b, c, plan, p, ds, s);
    } else {
        Launch<VW, false, G>(colInd, values, b, c, plan, p, ds, s);
    }
}

template <int kIn>
void LaunchNarrow(const void* colInd, const void* values, const void* b, void* c, const SpmmPlanView& plan,
                  const AclspSpmmParams& p, const DenseStrides& ds, cudaStream_t s)
{
    constexpr size_t smem = SmemBytes(1, kWarps, 0);
    cudaFuncSetAttribute(SpmmTileKernel<1, false, kIn>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem));
    AclspCountLaunches(2);
    SpmmTileKernel<1, false, kIn><<<plan.numTiles, kThreads, smem, s>>>(
        static_cast<const int32_t*>(colInd), static_cast<const float*>(values), static_cast<const float*>(b),
        static_cast<float*>(c), plan, p, ds);
    uint32_t blocks = (plan.numTiles + 7u) / 8u;
    blocks = blocks > 148u * 8u ? 148u * 8u : blocks;
    SpmmCarryFixupKernel<kIn><<<blocks, 256, 0, s>>>(static_cast<float*>(c), plan, p, ds);
}

}  // namespace

extern "C" void spmm_b200_kernel_do(const void* colInd, const void* values, const void* b, void* c,
                                    void* workspace, const AclspSpmmParams* params, void* stream)
{
    auto s = static_cast<cudaStream_t>(stream);
    const AclspSpmmParams p = *params;
    const SpmmPlanView plan = MakeView(workspace, p.rows, p.nnz, p.n);
    if (plan.numTiles == 0 || p.n == 0) {
        return;
    }
    // op(B)[r, c]: B is stored k x n when opB == 0 and n x k otherwise.
    DenseStrides ds;
    const bool bElementRowMajor = (p.opB == 0) == (p.orderB == 0);
    ds.bRow = bElementRowMajor ? p.ldb : 1;
    ds.bCol = bElementRowMajor ? 1 : p.ldb;
    ds.cRow = p.orderC == 0 ? p.ldc : 1;
    ds.cCol = p.orderC == 0 ? 1 : p.ldc;

    if (p.valueType != ACLSP_TYPE_F32) {
        AclspSpmmParams q = p;
        q.numMirrors = 0;
        q.mirrorMulticast = 0;
        q.barrier.world = 0;
        if (p.valueType == ACLSP_TYPE_F16) {
            LaunchNarrow<aclsp::kF16>(colInd, values, b, c, plan, q, ds, s);
        } else if (p.valueType == ACLSP_TYPE_BF16) {
            LaunchNarrow<aclsp::kBF16>(colInd, values, b, c, plan, q, ds, s);
        } else if (p.valueType == ACLSP_TYPE_I8) {
            LaunchNarrow<aclsp::kI8>(colInd, values, b, c, plan, q, ds, s);
        }
        return;
    }
    const bool unit = ds.bCol == 1 && ds.cCol == 1;
    uintptr_t addr = reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
    for (uint32_t m = 0; m < p.numMirrors && m < ACLSP_MAX_MIRRORS; ++m) {
        addr |= static_cast<uintptr_t>(p.mirrorDelta[m]);  // a mirror is as aligned as C and its distance from C
    }
    int vw = 1;
    // ACLSPARSE_SPMM_LANE_GROUPS=0: always whole warps per piece (a debugging aid, read once).
    static const bool groups = [] {
        const char* e = std::getenv("ACLSPARSE_SPMM_LANE_GROUPS");
        return e == nullptr || e[0] != '0';
    }();
    const bool quads = unit && p.n % 4 == 0 && p.ldb % 4 == 0 && p.ldc % 4 == 0 && addr % 16 == 0;
    auto fixup = [&]() {
        uint32_t fixupBlocks = (plan.numTiles + 7u) / 8u;
        fixupBlocks = fixupBlocks > 148u * 8u ? 148u * 8u : fixupBlocks;
        AclspCountLaunches(1);
        SpmmCarryFixupKernel<kF32><<<fixupBlocks, 256, 0, s>>>(static_cast<float*>(c), plan, p, ds);
    };
    if (quads && groups && p.n <= 64) {
        // Narrow C: four columns per lane and as few lanes per piece as cover a row of C in one pass (n <= 32:
        // 8 lanes, n <= 64: 16), so that a warp instruction works on four or two non-zeros at once.  (Eight
        // columns per lane were measured too: slower, c5 12.7 against 10.5 ms, c4 1.95 against 1.83 ms - the
        // doubled rings halve the resident CTAs.)
        if (p.n <= 32) {
            LaunchByPrecision<4, 8>(colInd, values, b, c, plan, p, ds, s);
        } else {
            LaunchByPrecision<4, 16>(colInd, values, b, c, plan, p, ds, s);
        }
        fixup();
        return;
    }
    if (unit && p.n % 4 == 0 && p.n >= 128 && p.ldb % 4 == 0 && p.ldc % 4 == 0 && addr % 16 == 0) {
        vw = 4;
    } else if (unit && p.n % 2 == 0 && p.n >= 64 && p.ldb % 2 == 0 && p.ldc % 2 == 0 && addr % 8 == 0) {
        vw = 2;
    }
    if (vw == 4) {
        LaunchByPrecision<4>(colInd, values, b, c, plan, p, ds, s);
    } else if (vw == 2) {
        LaunchByPrecision<2>(colInd, values, b, c, plan, p, ds, s);
    } else {
        LaunchByPrecision<1>(colInd, values, b, c, plan, p, ds, s);
    }
    uint32_t blocks = (plan.numTiles + 7u) / 8u;
    blocks = blocks > 148u * 8u ? 148u * 8u : blocks;
    AclspCountLaunches(1);
    SpmmCarryFixupKernel<kF32><<<blocks, 256, 0, s>>>(static_cast<float*>(c), plan, p, ds);
}
