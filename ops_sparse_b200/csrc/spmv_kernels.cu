/*
 * CSR SpMV for sm_100a:  y = alpha * A * x + beta * y,  int32 indices, fp32 data (and the narrow storage
 * types of element_types.cuh: typed instances of the same kernels, exact products without the error term).
 *
 * Two kernels.  The preprocessing pass records the longest row of the matrix in
 * the plan header and sends a copy to pinned host memory, asynchronously.  Once
 * that copy has arrived the host launches the kernel that fits; until then (the
 * first product right after a Preprocess call) it launches both, and each looks
 * in the plan header to see whether the product is its to compute.
 *
 * A. Row blocks (SpmvRowBlockKernel), for matrices whose longest row is short
 *    (a stencil, a mesh, a k-regular graph).  A block is 32 consecutive rows;
 *    its non-zeros are one contiguous slice of colInd / values.  Persistent
 *    warps loop over blocks.  No thread issues a global load for the matrix:
 *    lane 0 asks the copy engine (cp.async.bulk, completion counted on an
 *    mbarrier) for the slices and the 33 row offsets of the block kStages
 *    turns ahead, into the warp's own shared-memory stages, so HBM streams
 *    for some warps while the others compute (a stage is sized for the longest
 *    row, so that as many warps as possible are resident: measured on the
 *    27-point stencil, 24 warps with one stage each beat 12 warps with two).
 *    Each lane then walks ONE row out of
 *    shared memory with sixteen gathers of x in flight, adds in registers and
 *    writes y: no shuffle, no barrier, no carry.  The lanes of a warp are on
 *    consecutive rows at the same position, so for banded matrices their
 *    gathers fall into one or two lines of x.  Every wait is bounded; a warp
 *    whose wait runs out stops using the copy engine and finishes its blocks
 *    with plain loads, so the product is still right.  With mirrors (a sharded
 *    product) the 32 results of a block go to the other GPUs straight from
 *    registers, as eight 16-byte vectors when the block is aligned.
 *
 * B. Merge-path tiles (SpmvTileKernel), for everything else.  The matrix is cut
 *    along the merge path of (row ends, non-zeros) into tiles of kTile items, so
 *    a tile holds at most kTile non-zeros plus rows whatever the row-length
 *    distribution.  One CTA owns one tile:
 *   1. the tile's slice of colInd / values is streamed with 128-bit loads
 *      (evict-first: it is read exactly once), x[col] is gathered through the
 *      read-only path, and every product is staged in shared memory as an
 *      exact pair of floats (rounded product, rounding error) with 128-bit,
 *      conflict-free stores;
 *   2. rows that end inside the tile are reduced by groups of 2^class lanes
 *      ("vector per row", class picked per tile by the preprocessing pass from
 *      the tile's mean row length; class 5 is warp per row) with a shuffle
 *      tree; a piece that would keep its lanes busy for kLaneBudget products each
 *      or more is set aside (the lanes of a warp run as long as the longest piece
 *      among them) and gets eight lanes, a whole warp, or, from kLongSegment
 *      products on, the whole CTA;
 *   3. the piece of a row that continues into the next tile becomes the tile's
 *      carry-out, and the piece of a row that began in an earlier tile becomes
 *      its head partial; a second small kernel adds the carries of a split row
 *      in tile order and writes that row.
 *    A tile that lies inside one row (rows longer than a tile) skips staging:
 *    its products are added in registers, the warps joined in warp order.
 * Every sum is taken in a fixed order, so results are bit-reproducible.
 *
 * Accuracy.  Every product is kept exactly (hi + lo, rounded product and its
 * rounding error by FMA); the hi parts are summed in fp64, the lo parts (2^-24
 * of the products) in fp32, alpha * sum + beta * y is evaluated in fp64 and
 * rounded once, so a row is as accurate as the reference's host golden (SpmvCpu
 * with a double accumulator, test/spmv/arch22/spmv_test.cpp:258-279,309-348) up
 * to the order of the additions; the reference's device kernels reach for
 * compensated arithmetic for the same reason
 * (sparse/spmv/arch22/kernels/spmv_kernel.h:19-68).  A row piece whose sum is
 * not finite (an fp32 product overflowed, or the data holds Inf / NaN) is
 * summed again with fp64 products, which cannot overflow, so it again equals
 * the golden; the reference's device code falls back to its uncompensated sum
 * there (sparse/spmv/arch35/spmv_kernel.cpp:459-484).
 *
 * The kernels never read or write out of bounds for any content of the index
 * arrays: offsets are clamped to [0, nnz] and entries whose column falls
 * outside [0, cols) are skipped, as the reference's kernels do
 * (sparse/spmv/arch35/spmv_kernel.cpp:511-521).
 */
#include <cstdint>

#include <cstdlib>
#include <type_traits>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "element_types.cuh"
#include "node_barrier.cuh"
#include "plan_kernels.h"
#include "plan_layout.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTile = ACLSP_SPMV_TILE_ITEMS;
constexpr int kLaneBudget = 16;     // a piece stays with its lanes while each of them adds fewer products than this
constexpr int kOctetMax = 128;      // overflowing pieces shorter than this get eight lanes, longer ones a warp
constexpr int kMaxOctetSeg = kTile / kLaneBudget;
constexpr int kWarpSegment = 64;    // (capacity of the warp list: pieces on it are at least this long)
constexpr int kLongSegment = 1024;  // pieces at least this long get the whole CTA
constexpr int kMaxWarpSeg = kTile / kWarpSegment;
constexpr int kMaxLong = kTile / kLongSegment;

struct SpmvPlanView {
    const int32_t* rowPtr;  // base-0 row offsets, rows + 1 entries
    int32_t* tileRow;       // numTiles + 1
    int32_t* tileClass;     // numTiles
    double* carry;          // 2 * numTiles: [2t] tail carry-out, [2t+1] head partial
    uint32_t numTiles;
};

__host__ __device__ inline SpmvPlanView MakeView(void* workspace, uint32_t rows, uint32_t nnz)
{
    AclspPlanLayout l;
    aclspSpmvLayout(rows, nnz, &l);
    auto* base = static_cast<unsigned char*>(workspace);
    SpmvPlanView v;
    v.rowPtr = reinterpret_cast<const int32_t*>(base + l.rowPtrOff);
    v.tileRow = reinterpret_cast<int32_t*>(base + l.tileRowOff);
    v.tileClass = reinterpret_cast<int32_t*>(base + l.tileClassOff);
    v.carry = reinterpret_cast<double*>(base + l.carryOff);
    v.numTiles = l.numTiles;
    return v;
}

__device__ __forceinline__ int ClampOffset(int v, int nnz)
{
    return v < 0 ? 0 : (v > nnz ? nnz : v);
}

// Type of the matrix values and of x (template parameter kIn of the kernels): fp32 is the fast path
// and the only one with row blocks and mirrors; the narrow types run the tile kernel.  Their products
// are exact in fp32, so they need no error term; only a bf16 product can overflow, and then the sum is
// recomputed in fp64 like any other non-finite sum.
using aclsp::kBF16;
using aclsp::kF16;
using aclsp::kF32;
using aclsp::kI8;
using aclsp::LoadIn;

/* ------------------------------------------------------------ product -- */

using Scalars = aclsp::TypedScalars;

__device__ __forceinline__ Scalars LoadScalars(const AclspSpmvParams& p)
{
    return aclsp::LoadTypedScalars(p.computeInt, p.alphaPtr, p.betaPtr, p.alpha, p.beta, p.alphaInt, p.betaInt);
}

// Row `row` of the result: alpha * sum + beta * (the vector beta scales), written to `at`.  The
// vector beta scales is y itself, or p.betaSource when the product writes a vector of its own
// (the SpMVOp form Z = alpha*A*X + beta*Y).  beta == 0 must not read it: it may hold NaN, be
// uninitialised or be absent.
__device__ __forceinline__ float StoreRow(float* at, int64_t row, double sum, const Scalars& s, const AclspSpmvParams& p)
{
    double r = s.alpha * sum;
    if (!s.betaZero) {
        const float* from = p.betaSource != nullptr ? p.betaSource + row * p.betaSourceStride : at;
        r += s.beta * static_cast<double>(*from);
    }
    const float out = static_cast<float>(r);
    *at = out;
    return out;
}

// The same for an output of any element type (p.yType); y and p.betaSource address elements of that type.
__device__ __forceinline__ void StoreRowTyped(void* y, int64_t row, double sum, const Scalars& s, const AclspSpmvParams& p)
{
    const int64_t at = row * p.yStride;
    const void* from = p.betaSource != nullptr ? static_cast<const void*>(p.betaSource) : y;
    const int64_t fromAt = p.betaSource != nullptr ? row * p.betaSourceStride : at;
    aclsp::StoreScaled(p.yType, y, at, from, fromAt, sum, s);
}

// Mirrors of y (the other GPUs' result buffers when the matrix is sharded)
// receive what y received: plain stores to each mirror, or one multimem.st to
// a multicast address that the switch copies to every GPU.  Never read back.
__device__ __forceinline__ void MirrorStore(float* dst, float v, const AclspSpmvParams& p)
{
    if ((p.mirrorMulticast & 1u) != 0) {
        asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;\n" ::"l"(reinterpret_cast<char*>(dst) +
                                                                                 p.mirrorDelta[0]),
                     "f"(v)
                     : "memory");
        return;
    }
    for (uint32_t m = 0; m < p.numMirrors; ++m) {
        *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.mirrorDelta[m]) = v;
    }
}

__device__ __forceinline__ void MirrorStore(float4* dst, const float4& v, const AclspSpmvParams& p)
{
    if ((p.mirrorMulticast & 1u) != 0) {
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(
                         reinterpret_cast<char*>(dst) + p.mirrorDelta[0]),
                     "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                     : "memory");
        return;
    }
    for (uint32_t m = 0; m < p.numMirrors; ++m) {
        *reinterpret_cast<float4*>(reinterpret_cast<char*>(dst) + p.mirrorDelta[m]) = v;
    }
}

// One product as an unevaluated sum hi + lo of two floats: hi is the rounded
// fp32 product and lo its exact rounding error, so hi + lo == a * x[col]
// exactly.  Entries whose column is out of range contribute nothing.
template <int kIn = kF32>
__device__ __forceinline__ void Product(float a, int32_t rawCol, const void* __restrict__ x, uint32_t base,
                                        uint32_t cols, int64_t xStride, float& hi, float& lo)
{
    const uint32_t c = static_cast<uint32_t>(rawCol) - base;
    if (c >= cols) {
        hi = 0.0f;
        lo = 0.0f;
        return;
    }
    const float xv = LoadIn<kIn>(x, static_cast<int64_t>(c) * xStride);
    hi = __fmul_rn(a, xv);
    lo = kIn == kF32 ? fmaf(a, xv, -hi) : 0.0f;  // products of the narrow types are exact
}

__device__ __forceinline__ bool Finite(double v)
{
    return fabs(v) <= 1.7976931348623157e308;
}

// Non-zeros [e0, e1) of the arrays multiplied and added in fp64, in array order.  Rare (only
// for sums that came out non-finite), so it is kept out of line and takes everything by value.
template <int kIn = kF32>
__device__ __forceinline__ double ExactSum(const int32_t* colInd, const void* values, const void* x, int64_t e0,
                                        int64_t e1, int64_t colIndStride, int64_t valuesStride, int64_t xStride,
                                        uint32_t indexBase, uint32_t cols)
{
    double s = 0.0;
    for (int64_t e = e0; e < e1; ++e) {
        const uint32_t col = static_cast<uint32_t>(colInd[e * colIndStride]) - indexBase;
        if (col < cols) {
            s += static_cast<double>(LoadIn<kIn>(values, e * valuesStride)) *
                 static_cast<double>(LoadIn<kIn>(x, static_cast<int64_t>(col) * xStride));
        }
    }
    return s;
}

/* ------------------------------------------------------------- reduce -- */

// Shared scratch of the reduction, one per CTA.
struct ReduceScratch {
    double warp[kWarps];
    int longSeg[kMaxLong];
    int warpSeg[kMaxWarpSeg];
    int octetSeg[kMaxOctetSeg];
    int numOctetSeg;
    int numLong;
    int numWarpSeg;
};

// The staged tile: nt exact products (hi, lo), the nr + 1 row offsets relative
// to the tile's first product, and nr spare words for the mirrors of y.
struct StagedTile {
    const int32_t* colInd;  // the global arrays, for the exact recomputation of a non-finite piece
    const void* values;
    const void* x;
    int j0;                 // index of the tile's first product in them
    int t;
    int i0;
    int i1;
    int nr;
    int nt;
    int cls;
    const float* hiT;
    const float* loT;
    const int* sOff;
    float* sOut;
};

// Reduces the rows of a staged tile and writes them (y, mirrors, carries).
// Called by all threads of the CTA after the barrier that follows staging and
// after thread 0 has zeroed scratch.numLong / numWarpSeg before that barrier.
template <int kIn>
__device__ __forceinline__ void ReduceTile(const StagedTile& st, float* __restrict__ y, const SpmvPlanView& plan,
                                           const AclspSpmvParams& p, ReduceScratch& scratch)
{
    const int tid = threadIdx.x;
    const int t = st.t;
    const int i0 = st.i0;
    const int i1 = st.i1;
    const int nr = st.nr;
    const int nt = st.nt;
    const float* hiT = st.hiT;
    const float* loT = st.loT;
    const int* sOff = st.sOff;
    float* sOut = st.sOut;
    double* sWarp = scratch.warp;
    int* sLong = scratch.longSeg;
    int* sWarpSeg = scratch.warpSeg;
    int& sNumLong = scratch.numLong;
    int& sNumWarpSeg = scratch.numWarpSeg;
    int* sOctetSeg = scratch.octetSeg;
    int& sNumOctetSeg = scratch.numOctetSeg;
    (void)i1;

    const Scalars sc = LoadScalars(p);
    const bool headOpen = sOff[0] < 0;  // row i0 began in an earlier tile
    const int nseg = nr + 1;            // rows ending here, then the open tail

    const bool batchMirrors = (p.mirrorMulticast & 2u) != 0;
    auto segBegin = [&](int k) { const int b = sOff[k]; return b < 0 ? 0 : (b > nt ? nt : b); };
    auto segEnd = [&](int k) {
        if (k >= nr) {
            return nt;
        }
        const int e = sOff[k + 1];
        return e < 0 ? 0 : (e > nt ? nt : e);
    };
    auto emit = [&](int k, double sum) {
        if (!Finite(sum)) {
            sum = ExactSum<kIn>(st.colInd, st.values, st.x, static_cast<int64_t>(st.j0) + segBegin(k),
                                static_cast<int64_t>(st.j0) + segEnd(k), p.colIndStride, p.valuesStride, p.xStride,
                                p.indexBase, p.cols);
        }
        if (k >= nr) {
            plan.carry[2 * t] = sum;
        } else if (k == 0 && headOpen) {
            plan.carry[2 * t + 1] = sum;
        } else if (kIn != kF32) {
            StoreRowTyped(y, i0 + k, sum, sc, p);  // y addresses elements of p.yType; no mirrors
        } else {
            float* at = y + static_cast<int64_t>(i0 + k) * p.yStride;
            const float out = StoreRow(at, i0 + k, sum, sc, p);
            if (p.numMirrors != 0) {
                if (batchMirrors) {
                    sOut[k] = out;
                } else {
                    MirrorStore(at, out, p);
                }
            }
        }
    };
    // Sum of products [b, e) taken by this thread with the given stride: the hi
    // parts in fp64, the (tiny) lo parts in fp32, joined at the end.
    auto strided = [&](int b, int e, int first, int stride) {
        double h0 = 0.0, h1 = 0.0;
        float l0 = 0.0f, l1 = 0.0f;
        int q = b + first;
        for (; q + stride < e; q += 2 * stride) {  // two independent chains
            h0 += static_cast<double>(hiT[q]);
            l0 += loT[q];
            h1 += static_cast<double>(hiT[q + stride]);
            l1 += loT[q + stride];
        }
        if (q < e) {
            h0 += static_cast<double>(hiT[q]);
            l0 += loT[q];
        }
        return (h0 + h1) + static_cast<double>(l0 + l1);
    };

    // Vector per row: 2^cls lanes share a row piece.
    const int cls = st.cls & 7;
    const int shiftLanes = cls > 5 ? 5 : cls;
    const int lanes = 1 << shiftLanes;
    const int lane = tid & (lanes - 1);
    const int group = tid >> shiftLanes;
    const int ngroups = kThreads >> shiftLanes;
    for (int k0 = 0; k0 < nseg; k0 += ngroups) {
        const int k = k0 + group;
        bool active = k < nseg;
        double sum = 0.0;
        if (active) {
            const int b = segBegin(k);
            const int e = segEnd(k);
            const int len = e - b;
            if (len >= kLaneBudget * lanes) {
                // Too long for its lanes (the lanes of a warp run as long as the longest piece among
                // them, so one long piece would idle the others): queue it for eight lanes, for a
                // warp, or for the whole CTA.  A valid CSR fills no list beyond its capacity; row
                // offsets that overlap could, and the excess is dropped.
                if (lane == 0) {
                    if (len >= kLongSegment) {
                        const int slot = atomicAdd(&sNumLong, 1);
                        if (slot < kMaxLong) {
                            sLong[slot] = k;
                        }
                    } else if (len >= kOctetMax || lanes >= 8) {
                        const int slot = atomicAdd(&sNumWarpSeg, 1);
                        if (slot < kMaxWarpSeg) {
                            sWarpSeg[slot] = k;
                        }
                    } else {
                        const int slot = atomicAdd(&sNumOctetSeg, 1);
                        if (slot < kMaxOctetSeg) {
                            sOctetSeg[slot] = k;
                        }
                    }
                }
                active = false;
            } else {
                sum = strided(b, e, lane, lanes);
            }
        }
        __syncwarp();
        for (int o = lanes >> 1; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (active && lane == 0) {
            emit(k, sum);
        }
    }
    __syncthreads();

    // Pieces a little too long for their lanes: eight lanes per piece.
    const int numOctetSeg = sNumOctetSeg < kMaxOctetSeg ? sNumOctetSeg : kMaxOctetSeg;
    for (int q0 = 0; q0 < numOctetSeg; q0 += kThreads / 8) {
        const int q = q0 + (tid >> 3);
        const bool has = q < numOctetSeg;
        const int k = has ? sOctetSeg[q] : 0;
        double sum = has ? strided(segBegin(k), segEnd(k), tid & 7, 8) : 0.0;
        for (int o = 4; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (has && (tid & 7) == 0) {
            emit(k, sum);
        }
    }

    // Medium pieces: warp per row.
    const int numWarpSeg = sNumWarpSeg < kMaxWarpSeg ? sNumWarpSeg : kMaxWarpSeg;
    for (int q = tid >> 5; q < numWarpSeg; q += kWarps) {
        const int k = sWarpSeg[q];
        double sum = strided(segBegin(k), segEnd(k), tid & 31, 32);
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if ((tid & 31) == 0) {
            emit(k, sum);
        }
    }

    // Long pieces: the whole CTA adds one piece, warps combined in warp order.
    const int numLong = sNumLong < kMaxLong ? sNumLong : kMaxLong;
    for (int q = 0; q < numLong; ++q) {
        const int k = sLong[q];
        double sum = strided(segBegin(k), segEnd(k), tid, kThreads);
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if ((tid & 31) == 0) {
            sWarp[tid >> 5] = sum;
        }
        __syncthreads();
        if (tid == 0) {
            double totalSum = 0.0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                totalSum += sWarp[w];
            }
            emit(k, totalSum);
        }
        __syncthreads();
    }

    // Mirrors, batched: the rows this tile finished are one contiguous run of
    // y.  Their values were kept in shared memory and now go out as whole
    // 16-byte vectors wherever y and the mirrors allow, so that the links carry
    // full lines instead of one packet per row.
    if (p.numMirrors != 0 && batchMirrors) {
        __syncthreads();
        const int skip = headOpen ? 1 : 0;
        const int count = nr - skip;
        const float* vals = sOut + skip;
        if (p.yStride == 1) {
            float* run = y + i0 + skip;
            bool aligned = true;  // a mirror is as aligned as y and its distance from y
            for (uint32_t m = 0; m < p.numMirrors; ++m) {
                aligned = aligned && (p.mirrorDelta[m] & 15) == 0;
            }
            int head = static_cast<int>((16u - (reinterpret_cast<uintptr_t>(run) & 15u)) & 15u) >> 2;
            head = aligned ? (head < count ? head : count) : count;
            head = head < 0 ? 0 : head;
            const int vecs = (count - head) >> 2;
            for (int k = tid; k < head; k += kThreads) {
                MirrorStore(run + k, vals[k], p);
            }
            for (int v = tid; v < vecs; v += kThreads) {
                const int k = head + 4 * v;
                MirrorStore(reinterpret_cast<float4*>(run + k), make_float4(vals[k], vals[k + 1], vals[k + 2], vals[k + 3]),
                            p);
            }
            for (int k = head + 4 * (vecs > 0 ? vecs : 0) + tid; k < count; k += kThreads) {
                MirrorStore(run + k, vals[k], p);
            }
        } else {
            for (int k = tid; k < count; k += kThreads) {
                MirrorStore(y + static_cast<int64_t>(i0 + skip + k) * p.yStride, vals[k], p);
            }
        }
    }
}

/* --------------------------------------------- one CTA per tile -- */

// kIn != kF32: values, x and y address elements of the narrow types (see "element types" above); the
// vector path then takes eight 2-byte values per 128-bit load.
template <bool kVector, int kIn = kF32>
__global__ void __launch_bounds__(kThreads, kVector ? 6 : 1)
SpmvTileKernel(const int32_t* __restrict__ colInd, const float* __restrict__ values, const float* __restrict__ x,
               float* __restrict__ y, SpmvPlanView plan, AclspSpmvParams p, const uint32_t* __restrict__ maxRowLen,
               uint32_t rowBlockCap)
{
    static_assert(!kVector || kIn == kF32 || kIn == kF16 || kIn == kBF16, "vector loads: 4- and 2-byte values");
    if (rowBlockCap != 0 && *maxRowLen <= rowBlockCap) {
        return;  // every row is short: the row-block kernel computes this product
    }
    // One pool of 32-bit words: the hi parts of the tile's products, their lo
    // parts, and the tile's row offsets packed against the end.  A tile has nt
    // products and nr + 1 offsets with nt + nr <= kTile.
    constexpr int kVecElems = kIn == kF32 ? 4 : 8;  // elements of `values` per 128-bit load
    __shared__ __align__(16) float sPool[2 * kTile + 40];
    __shared__ ReduceScratch scratch;

    const int tid = threadIdx.x;
    const int t = blockIdx.x;
    const int nnz = static_cast<int>(p.nnz);
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
    // Row offsets that are not non-decreasing can produce an inconsistent
    // split; such a tile is skipped rather than trusted.
    if (nr < 0 || nt < 0 || nr + nt > kTile || i0 < 0 || i1 > static_cast<int>(p.rows) || j0 < 0 || j1 > nnz) {
        if (tid == 0) {
            plan.carry[2 * t] = 0.0;
            plan.carry[2 * t + 1] = 0.0;
        }
        return;
    }
    // Products are stored at their offset from the 4-aligned array index a0,
    // so that a 128-bit load of the arrays maps onto a 128-bit shared store.
    const int a0 = kVector ? (j0 & ~(kVecElems - 1)) : j0;
    const int shift = j0 - a0;
    const int span = (nt + shift + kVecElems - 1) & ~(kVecElems - 1);
    float* sHi = sPool;
    float* sLo = sPool + span;
    int* sOff = reinterpret_cast<int*>(sPool + 2 * kTile + 40) - (nr + 2);
    // nr more words fit between the products and the offsets (2 * span <= 2 * nt + 28 and
    // nt + nr <= kTile): the finished rows' values, kept for the mirrors of y.
    float* sOut = reinterpret_cast<float*>(sOff) - nr;
    if (tid == 0) {
        scratch.numLong = 0;
        scratch.numWarpSeg = 0;
        scratch.numOctetSeg = 0;
    }
    for (int k = tid; k <= nr; k += kThreads) {
        sOff[k] = ClampOffset(plan.rowPtr[i0 + k], nnz) - j0;
    }

    if constexpr (kVector && kIn == kF32) {
        if (nr == 0) {
            // The tile lies inside one row (a power-law row longer than a tile): no product needs to be
            // staged.  Each thread adds the products of its vectors in registers, in vector order; the
            // warps are joined in warp order: a fixed order, like every other path.
            const int nvec = span >> 2;
            double h = 0.0;
            float l = 0.0f;
            constexpr int kDepth = 2;  // vectors (eight gathers) in flight per thread
            for (int v0 = tid; v0 < nvec; v0 += kDepth * kThreads) {
                int4 c[kDepth];
                float4 w[kDepth];
#pragma unroll
                for (int u = 0; u < kDepth; ++u) {
                    const int v = v0 + u * kThreads;
                    const int e = a0 + 4 * v;
                    if (v < nvec && e + 4 <= nnz) {
                        c[u] = __ldcs(reinterpret_cast<const int4*>(colInd + e));
                        w[u] = __ldcs(reinterpret_cast<const float4*>(values + e));
                    } else {
                        int32_t cc[4];
                        float ww[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const bool in = v < nvec && e + q < nnz;
                            cc[q] = in ? __ldcs(colInd + e + q) : -1;
                            ww[q] = in ? __ldcs(values + e + q) : 0.0f;
                        }
                        c[u] = make_int4(cc[0], cc[1], cc[2], cc[3]);
                        w[u] = make_float4(ww[0], ww[1], ww[2], ww[3]);
                    }
                }
#pragma unroll
                for (int u = 0; u < kDepth; ++u) {
                    const int e = a0 + 4 * (v0 + u * kThreads);
                    const int cc[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
                    const float ww[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
                    float hi[4];
                    float lo[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        // elements of the first and last vector that belong to a neighbouring tile do not count
                        const bool mine = e + q >= j0 && e + q < j1;
                        Product(ww[q], mine ? cc[q] : -1, x, p.indexBase, p.cols, 1, hi[q], lo[q]);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        h += static_cast<double>(hi[q]);
                        l += lo[q];
                    }
                }
            }
            double sum = h + static_cast<double>(l);
            for (int o = 16; o > 0; o >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            if ((tid & 31) == 0) {
                scratch.warp[tid >> 5] = sum;
            }
            __syncthreads();
            if (tid == 0) {
                double total = 0.0;
#pragma unroll
                for (int wq = 0; wq < kWarps; ++wq) {
                    total += scratch.warp[wq];
                }
                if (!Finite(total)) {
                    total = ExactSum<kIn>(colInd, values, x, j0, j1, 1, 1, 1, p.indexBase, p.cols);
                }
                plan.carry[2 * t] = total;  // the tile's open tail; there is no head piece (no row ends here)
            }
            return;
        }
    }
    if constexpr (kVector && kIn != kF32) {
        // Eight 2-byte values and eight column indices per step: one 128-bit load of the values, two
        // of the indices; elements of the first and last vector that belong to a neighbouring tile
        // are multiplied too, nothing reads their slots.
        const int nvec = span >> 3;
        for (int v = tid; v < nvec; v += kThreads) {
            const int e = a0 + 8 * v;
            int32_t c[8];
            float w[8];
            if (e + 8 <= nnz) {
                const int4 c0 = __ldcs(reinterpret_cast<const int4*>(colInd + e));
                const int4 c1 = __ldcs(reinterpret_cast<const int4*>(colInd + e + 4));
                const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(values) + e));
                c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w;
                c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if constexpr (kIn == kF16) {
                        const __half2 h = *reinterpret_cast<const __half2*>(&words[q]);
                        w[2 * q] = __low2float(h);
                        w[2 * q + 1] = __high2float(h);
                    } else {  // bf16: the upper half of an fp32
                        w[2 * q] = __uint_as_float(words[q] << 16);
                        w[2 * q + 1] = __uint_as_float(words[q] & 0xffff0000u);
                    }
                }
            } else {  // the last vector of the arrays may be partial
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const bool in = e + q < nnz;
                    c[q] = in ? __ldcs(colInd + e + q) : -1;
                    w[q] = in ? LoadIn<kIn>(values, e + q) : 0.0f;
                }
            }
            float hi[8];
            float lo[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                Product<kIn>(w[q], c[q], x, p.indexBase, p.cols, 1, hi[q], lo[q]);
            }
            *reinterpret_cast<float4*>(sHi + 8 * v) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<float4*>(sHi + 8 * v + 4) = make_float4(hi[4], hi[5], hi[6], hi[7]);
            *reinterpret_cast<float4*>(sLo + 8 * v) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            *reinterpret_cast<float4*>(sLo + 8 * v + 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    } else if constexpr (kVector) {
        const int nvec = span >> 2;
        struct Vec4 {
            int4 c;
            float4 w;
        };
        auto loadVec = [&](int v, Vec4& o) {
            const int e = a0 + 4 * v;
            if (e + 4 <= nnz) {
                o.c = __ldcs(reinterpret_cast<const int4*>(colInd + e));
                o.w = __ldcs(reinterpret_cast<const float4*>(values + e));
            } else {  // the last vector of the arrays may be partial
                int32_t c[4];
                float w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const bool in = e + q < nnz;
                    c[q] = in ? __ldcs(colInd + e + q) : -1;
                    w[q] = in ? __ldcs(values + e + q) : 0.0f;
                }
                o.c = make_int4(c[0], c[1], c[2], c[3]);
                o.w = make_float4(w[0], w[1], w[2], w[3]);
            }
        };
        // Elements of the first and last vector that belong to a neighbouring
        // tile are multiplied too; nothing reads their slots.
        auto useVec = [&](int v, const Vec4& o) {
            float4 hi, lo;
            Product(o.w.x, o.c.x, x, p.indexBase, p.cols, 1, hi.x, lo.x);
            Product(o.w.y, o.c.y, x, p.indexBase, p.cols, 1, hi.y, lo.y);
            Product(o.w.z, o.c.z, x, p.indexBase, p.cols, 1, hi.z, lo.z);
            Product(o.w.w, o.c.w, x, p.indexBase, p.cols, 1, hi.w, lo.w);
            *reinterpret_cast<float4*>(sHi + 4 * v) = hi;
            *reinterpret_cast<float4*>(sLo + 4 * v) = lo;
        };
        // A tile spans at most kTile / 4 + 1 vectors: kVecsPerThread per thread,
        // all of them loaded before the first is used, plus a one-vector remainder.
        constexpr int kVecsPerThread = kTile / 4 / kThreads;
        Vec4 vv[kVecsPerThread];
#pragma unroll
        for (int u = 0; u < kVecsPerThread; ++u) {
            if (tid + u * kThreads < nvec) {
                loadVec(tid + u * kThreads, vv[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kVecsPerThread; ++u) {
            if (tid + u * kThreads < nvec) {
                useVec(tid + u * kThreads, vv[u]);
            }
        }
        for (int v = tid + kVecsPerThread * kThreads; v < nvec; v += kThreads) {
            Vec4 vc;
            loadVec(v, vc);
            useVec(v, vc);
        }
    } else {
        for (int k = tid; k < nt; k += kThreads) {
            const int64_t e = static_cast<int64_t>(j0) + k;
            Product<kIn>(LoadIn<kIn>(values, e * p.valuesStride), colInd[e * p.colIndStride], x, p.indexBase, p.cols,
                         p.xStride, sHi[k], sLo[k]);
        }
    }
    __syncthreads();

    StagedTile st;
    st.colInd = colInd;
    st.values = values;
    st.x = x;
    st.j0 = j0;
    st.t = t;
    st.i0 = i0;
    st.i1 = i1;
    st.nr = nr;
    st.nt = nt;
    st.cls = plan.tileClass[t];
    st.hiT = sHi + shift;  // product k of the tile
    st.loT = sLo + shift;
    st.sOff = sOff;
    st.sOut = sOut;
    ReduceTile<kIn>(st, y, plan, p, scratch);
}

/* ------------------------------------------------ row blocks (A) -- */

constexpr int kBlockRows = 32;             // rows per block: one per lane
constexpr int kOffsetWords = 36;           // 33 row offsets, rounded up to whole 16-byte vectors
constexpr uint32_t kSpinLimit = 1u << 18;  // polls of about a microsecond before a wait is given up

// Elements of one stage slice for rows of at most `cap` non-zeros, and the words of a stage: the
// offsets, then the slice of values and the slice of colInd, each from the aligned array index below
// the block's first non-zero to the aligned index above its last.  `align` is the number of elements
// of `values` in 16 bytes (4 for fp32, 8 for the 2-byte types): slices start and end on multiples of it,
// so that both bulk copies start on a 16-byte boundary and have a multiple of 16 bytes.
__host__ __device__ constexpr int RowBlockSpanCap(int cap, int align) { return kBlockRows * cap + 2 * align; }
__host__ __device__ constexpr int RowBlockStageWords(int cap, int align)
{
    return kOffsetWords + RowBlockSpanCap(cap, align) + RowBlockSpanCap(cap, align) * 4 / align;
}
constexpr int kRowBlockMaxLen = 40;  // longest row the row-block kernel is used for

__device__ __forceinline__ uint32_t SharedAddress(const void* ptr)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}

// The matrix is read once per product: its lines are marked evict-first in L2 so
// that they do not push x (which every block gathers from) out of it.
__device__ __forceinline__ uint64_t EvictFirstPolicy()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}

// Bulk copy into this CTA's shared memory; the source is this GPU's own memory; no multicast.
__device__ __forceinline__ void BulkLoad(void* smemDst, const void* gmemSrc, uint32_t bytes, uint64_t* bar,
                                         uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::
            "r"(SharedAddress(smemDst)),
        "l"(gmemSrc), "r"(bytes), "r"(SharedAddress(bar)), "l"(policy)
        : "memory");
}

// Bounded wait for a stage: false when the copies have not landed after kSpinLimit polls.
__device__ __forceinline__ bool WaitStage(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = SharedAddress(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done != 0) {
            return true;
        }
    }
    return false;
}

struct RowBlockGeom {
    int r0;         // first row
    int nrows;      // rows in the block (32 except at the end of the matrix)
    int a0;         // aligned array index the staged slices start at
    int span;       // words staged per slice
    int copyElems;  // leading part of the span that is whole vectors inside the arrays: bulk-copied
    int offWords;   // row offsets copied, whole vectors
    bool valid;     // false: offsets inconsistent with the recorded longest row; nothing is copied
};

// j0 / j1: offsets of the block's first row and of the row after its last one, as loaded from the plan.
__device__ __forceinline__ RowBlockGeom BlockGeometry(uint32_t block, int j0, int j1, const AclspSpmvParams& p,
                                                      int spanCap, int align)
{
    RowBlockGeom g;
    const int nnz = static_cast<int>(p.nnz);
    g.r0 = static_cast<int>(block) * kBlockRows;
    const int left = static_cast<int>(p.rows) - g.r0;
    g.nrows = left < kBlockRows ? left : kBlockRows;
    j0 = ClampOffset(j0, nnz);
    j1 = ClampOffset(j1, nnz);
    g.a0 = j0 & ~(align - 1);
    g.span = (j1 - g.a0 + align - 1) & ~(align - 1);
    g.valid = j1 >= j0 && g.span <= spanCap;
    const int whole = (nnz & ~(align - 1)) - g.a0;
    g.copyElems = whole < 0 ? 0 : (whole < g.span ? whole : g.span);
    g.offWords = (g.nrows + 1 + 3) & ~3;
    return g;
}

// Lane 0: announce the bytes of a block to the stage's barrier and start its copies.
// valueBytes: size of an element of `values` (4 or 2).
__device__ __forceinline__ void IssueBlock(const RowBlockGeom& g, float* stage, int spanCap, uint64_t* bar,
                                           const int32_t* colInd, const void* values, const int32_t* rowPtr,
                                           uint64_t policy, uint32_t valueBytes)
{
    const uint32_t colBytes = g.valid ? 4u * static_cast<uint32_t>(g.copyElems) : 0u;
    const uint32_t valBytes = g.valid ? valueBytes * static_cast<uint32_t>(g.copyElems) : 0u;
    const uint32_t offBytes = 4u * static_cast<uint32_t>(g.offWords);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(SharedAddress(bar)),
                 "r"(colBytes + valBytes + offBytes)
                 : "memory");
    BulkLoad(stage, rowPtr + g.r0, offBytes, bar, policy);
    if (colBytes != 0) {
        BulkLoad(stage + kOffsetWords, static_cast<const unsigned char*>(values) + static_cast<size_t>(g.a0) * valueBytes,
                 valBytes, bar, policy);
        BulkLoad(stage + kOffsetWords + spanCap * valueBytes / 4u, colInd + g.a0, colBytes, bar, policy);
    }
}

// cap: longest row a stage can hold (the launcher sized shared memory for it).  kWarpsPerCta warps
// per CTA, each with its own kStages stages; the launcher sizes the grid so that the stages of the
// resident CTAs fill shared memory.  checkPlan != 0: return at once unless the plan header says that
// no row is longer than cap (the host did not know yet which kernel the matrix needs).
// kIn: fp32, or one of the 2-byte types (values, x and y then address elements of those types).
template <int kStages, int kWarpsPerCta, int kUnroll, int kIn = kF32>
__global__ void __launch_bounds__(32 * kWarpsPerCta)
SpmvRowBlockKernel(const int32_t* __restrict__ colInd, const float* __restrict__ values, const float* __restrict__ x,
                   float* __restrict__ y, SpmvPlanView plan, AclspSpmvParams p, const uint32_t* __restrict__ maxRowLen,
                   uint32_t* __restrict__ waitFailures, int cap, int checkPlan)
{
    static_assert(kIn == kF32 || kIn == kF16 || kIn == kBF16, "bulk-copied slices: 4- and 2-byte values");
    constexpr int kAlign = kIn == kF32 ? 4 : 8;         // elements of `values` in 16 bytes
    constexpr uint32_t kValueBytes = kIn == kF32 ? 4u : 2u;
    using StagedValue = typename std::conditional<kIn == kF32, float, uint16_t>::type;
    if (checkPlan != 0 && *maxRowLen > static_cast<uint32_t>(cap)) {
        return;  // some row is too long for a stage: the merge-path tiles compute this product
    }
    const int kSpanCap = RowBlockSpanCap(cap, kAlign);
    const int kWords = RowBlockStageWords(cap, kAlign);
    extern __shared__ __align__(128) unsigned char smemRaw[];
    const int lane = threadIdx.x & 31;
    const int warpInCta = threadIdx.x >> 5;
    float* ring = reinterpret_cast<float*>(smemRaw) + static_cast<size_t>(warpInCta) * kStages * kWords;
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<float*>(smemRaw) +
                                                 static_cast<size_t>(kWarpsPerCta) * kStages * kWords) +
                     warpInCta * kStages;

    const int nnz = static_cast<int>(p.nnz);
    const uint32_t numBlocks = (p.rows + kBlockRows - 1u) / kBlockRows;
    const uint32_t totalWarps = gridDim.x * kWarpsPerCta;
    const uint32_t firstBlock = blockIdx.x * kWarpsPerCta + warpInCta;
    const uint64_t policy = EvictFirstPolicy();
    const Scalars sc = LoadScalars(p);
    const int32_t* rowPtr = plan.rowPtr;

    auto lastRowOf = [&](uint32_t block) {
        const uint32_t end = (block + 1u) * kBlockRows;
        return end < p.rows ? end : p.rows;
    };
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(SharedAddress(full + s)) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        uint32_t b = firstBlock;
        for (int s = 0; s < kStages && b < numBlocks; ++s, b += totalWarps) {
            const RowBlockGeom g = BlockGeometry(b, rowPtr[b * kBlockRows], rowPtr[lastRowOf(b)], p, kSpanCap, kAlign);
            IssueBlock(g, ring + s * kWords, kSpanCap, full + s, colInd, values, rowPtr, policy, kValueBytes);
        }
    }
    __syncwarp();

    // A row straight from global memory with fp64 products: the path of a warp whose wait ran
    // out, and of blocks that do not fit a stage (row offsets that contradict the longest row the
    // stages were sized for): slow, but right whatever the offsets and the hint are.
    auto slowRow = [&](int row) {
        const int b = ClampOffset(rowPtr[row], nnz);
        const int e = ClampOffset(rowPtr[row + 1], nnz);
        return ExactSum<kIn>(colInd, values, x, b, e, 1, 1, 1, p.indexBase, p.cols);
    };
    auto writeRow = [&](int row, double sum) {
        if (kIn != kF32) {
            StoreRowTyped(y, row, sum, sc, p);  // y addresses elements of p.yType; no mirrors
            return;
        }
        float* at = y + static_cast<int64_t>(row) * p.yStride;
        const float out = StoreRow(at, row, sum, sc, p);
        if (p.numMirrors != 0) {
            MirrorStore(at, out, p);  // 32 consecutive rows per warp: whole lines on the links
        }
    };

    bool waitedOut = false;
    uint32_t gaveUpAt = 0;
    uint32_t it = 0;
    // Extent of the block that refills the stage in use, loaded a turn ahead of its use.
    int refillJ0 = 0, refillJ1 = 0;
    for (uint32_t block = firstBlock; block < numBlocks; block += totalWarps, ++it) {
        const int s = static_cast<int>(it % kStages);
        const uint32_t parity = (it / kStages) & 1u;
        float* stage = ring + s * kWords;
        const uint32_t refill = block + kStages * totalWarps;
        if (lane == 0 && refill < numBlocks && !waitedOut) {
            refillJ0 = rowPtr[refill * kBlockRows];
            refillJ1 = rowPtr[lastRowOf(refill)];
        }
        const int r0 = static_cast<int>(block) * kBlockRows;
        const int row = r0 + lane;
        const bool rowOk = row < static_cast<int>(p.rows);
        if (!waitedOut) {
            const bool landed = WaitStage(full + s, parity);
            if (__any_sync(0xffffffffu, !landed)) {
                waitedOut = true;
                gaveUpAt = it;
            }
        }
        if (waitedOut) {
            if (rowOk) {
                writeRow(row, slowRow(row));
            }
            continue;
        }
        const int* off = reinterpret_cast<const int*>(stage);
        const RowBlockGeom g = BlockGeometry(block, off[0], off[lastRowOf(block) - r0], p, kSpanCap, kAlign);
        if (!g.valid) {
            if (rowOk) {
                writeRow(row, slowRow(row));
            }
        } else {
            StagedValue* sVal = reinterpret_cast<StagedValue*>(stage + kOffsetWords);
            int* sCol = reinterpret_cast<int*>(stage + kOffsetWords + kSpanCap * static_cast<int>(kValueBytes) / 4);
            if (g.copyElems < g.span) {
                // The arrays end inside this span with a partial vector: plain loads fill it.
                for (int k = g.copyElems + lane; k < g.span; k += 32) {
                    const int e = g.a0 + k;
                    sCol[k] = e < nnz ? __ldcs(colInd + e) : -1;
                    sVal[k] = e < nnz ? __ldcs(reinterpret_cast<const StagedValue*>(values) + e) : StagedValue(0);
                }
                __syncwarp();
            }
            // A staged value as fp32 (exact).
            auto widen = [](StagedValue v) {
                if constexpr (kIn == kF16) {
                    return __half2float(__ushort_as_half(v));
                } else if constexpr (kIn == kBF16) {
                    return __uint_as_float(static_cast<uint32_t>(v) << 16);
                } else {
                    return v;
                }
            };
            int b = 0, e = 0;
            if (rowOk) {
                b = ClampOffset(off[lane], nnz) - g.a0;
                e = ClampOffset(off[lane + 1], nnz) - g.a0;
                b = b < 0 ? 0 : (b > g.span ? g.span : b);
                e = e < b ? b : (e > g.span ? g.span : e);
            }
            double h = 0.0;
            float l = 0.0f;
            int q = b;
            // kUnroll products per lane and turn, all their gathers in flight together.
            while (__any_sync(0xffffffffu, q < e)) {
                int cc[kUnroll];
                float vv[kUnroll];
                float xx[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const bool ok = q + u < e;
                    cc[u] = ok ? sCol[q + u] : -1;
                    vv[u] = ok ? widen(sVal[q + u]) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const uint32_t col = static_cast<uint32_t>(cc[u]) - p.indexBase;
                    const bool in = col < p.cols;
                    xx[u] = in ? LoadIn<kIn>(x, col) : 0.0f;
                    vv[u] = in ? vv[u] : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const float hi = __fmul_rn(vv[u], xx[u]);
                    if (kIn == kF32) {  // products of the narrow types are exact
                        l += fmaf(vv[u], xx[u], -hi);
                    }
                    h += static_cast<double>(hi);
                }
                q += kUnroll;
            }
            double sum = h + static_cast<double>(l);
            if (rowOk && !Finite(sum)) {
                sum = ExactSum<kIn>(colInd, values, x, static_cast<int64_t>(g.a0) + b, static_cast<int64_t>(g.a0) + e,
                                    1, 1, 1, p.indexBase, p.cols);
            }
            // With mirrors, a full block whose 32 results start on a 16-byte boundary everywhere goes out as
            // eight 16-byte vectors (lanes 0 - 7, four neighbours' results each) instead of 32 words: the links
            // carry packets four times as large.
            bool vectorMirrors = false;
            if (kIn == kF32 && p.numMirrors != 0) {
                vectorMirrors = g.nrows == kBlockRows && p.yStride == 1 &&
                                (reinterpret_cast<uintptr_t>(y + r0) & 15u) == 0;
                for (uint32_t m = 0; m < p.numMirrors; ++m) {
                    vectorMirrors = vectorMirrors && (p.mirrorDelta[m] & 15) == 0;
                }
            }
            if (vectorMirrors) {
                float* at = y + row;
                const float out = StoreRow(at, row, sum, sc, p);
                float4 v;
                v.x = __shfl_sync(0xffffffffu, out, 4 * (lane & 7));
                v.y = __shfl_sync(0xffffffffu, out, 4 * (lane & 7) + 1);
                v.z = __shfl_sync(0xffffffffu, out, 4 * (lane & 7) + 2);
                v.w = __shfl_sync(0xffffffffu, out, 4 * (lane & 7) + 3);
                if (lane < 8) {
                    MirrorStore(reinterpret_cast<float4*>(y + r0 + 4 * lane), v, p);
                }
            } else if (rowOk) {
                writeRow(row, sum);
            }
        }
        __syncwarp();  // every lane is done with the stage
        if (lane == 0 && refill < numBlocks) {
            // Shared-memory reads of the block above come before the copy engine's writes.
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            const RowBlockGeom r = BlockGeometry(refill, refillJ0, refillJ1, p, kSpanCap, kAlign);
            IssueBlock(r, stage, kSpanCap, full + s, colInd, values, rowPtr, policy, kValueBytes);
        }
    }
    if (waitedOut) {
        // Copies started before the warp gave up may still land in its stages: each of them gets
        // one more bounded wait before the warp, and with it perhaps the CTA, leaves.
        for (uint32_t j = gaveUpAt; j < gaveUpAt + kStages; ++j) {
            if (static_cast<uint64_t>(firstBlock) + static_cast<uint64_t>(j) * totalWarps < numBlocks) {
                (void)WaitStage(full + j % kStages, (j / kStages) & 1u);
            }
        }
        if (lane == 0) {
            atomicAdd(waitFailures, 1u);
        }
    }
    // p.barrier is set for this kernel only when it is the product's last one (checkPlan == 0).
    aclsp::CloseWithNodeBarrier(p.barrier);
}

/* ----------------------------------------------------- carry fix-up -- */

// Rows that span tiles.  A warp looks at 32 tiles, one per lane: tile t needs a fix-up when its
// first row began in an earlier tile and ends in t.  Almost always the row began in tile t - 1:
// the lane adds that tile's carry-out and its own head partial and writes the row.  Rows that
// crossed several tiles are then taken one by one by the whole warp: the lanes add the carry-outs
// of the tiles the row crossed (lane-strided, then a shuffle tree: a fixed order), lane 0 adds the
// head partial and writes the row.
template <int kIn>
__device__ __forceinline__ void JoinCarries(float* __restrict__ y, const SpmvPlanView& plan, const AclspSpmvParams& p)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t t = warp * 32u + lane;
    const int nnz = static_cast<int>(p.nnz);
    const int64_t total = static_cast<int64_t>(p.rows) + nnz;
    const Scalars sc = LoadScalars(p);
    auto writeRow = [&](int row, double sum) {
        if (kIn != kF32) {
            StoreRowTyped(y, row, sum, sc, p);
            return;
        }
        float* at = y + static_cast<int64_t>(row) * p.yStride;
        const float out = StoreRow(at, row, sum, sc, p);
        if (p.numMirrors != 0) {
            MirrorStore(at, out, p);
        }
    };
    bool longRow = false;
    int i0 = 0;
    if (t < plan.numTiles) {
        i0 = plan.tileRow[t];
        const int i1 = plan.tileRow[t + 1];
        if (i1 > i0 && i0 >= 0 && i0 < static_cast<int>(p.rows)) {
            int64_t d0 = static_cast<int64_t>(t) * kTile;
            d0 = d0 < total ? d0 : total;
            if (ClampOffset(plan.rowPtr[i0], nnz) < d0 - i0) {
                // t > 0 here: tile 0 starts at item 0, before which no row can begin.
                longRow = t >= 2 && plan.tileRow[t - 1] == i0;
                if (!longRow) {
                    writeRow(i0, plan.carry[2 * (t - 1)] + plan.carry[2 * t + 1]);
                }
            }
        }
    }
    uint32_t todo = __ballot_sync(0xffffffffu, longRow);
    while (todo != 0) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const uint32_t tt = warp * 32u + src;
        const int row = __shfl_sync(0xffffffffu, i0, src);
        // Tiles first .. tt-1 hold the earlier pieces of the row: `first` is the last tile that
        // starts at a row before it (tileRow is non-decreasing), or tile 0.
        uint32_t lo = 0;
        uint32_t hi = tt;
        while (lo < hi) {
            const uint32_t mid = (lo + hi) >> 1;
            if (plan.tileRow[mid] < row) {
                lo = mid + 1;
            } else {
                hi = mid;
            }
        }
        const uint32_t first = lo > 0 ? lo - 1 : 0;
        double sum = 0.0;
        for (uint32_t u = first + lane; u < tt; u += 32) {
            sum += plan.carry[2 * u];
        }
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (lane == 0) {
            writeRow(row, sum + plan.carry[2 * tt + 1]);
        }
    }
}

template <int kIn = kF32>
__global__ void __launch_bounds__(kThreads)
SpmvCarryFixupKernel(float* __restrict__ y, SpmvPlanView plan, AclspSpmvParams p, const uint32_t* __restrict__ maxRowLen,
                     uint32_t rowBlockCap)
{
    // rowBlockCap != 0 and no longer row: the row-block kernel computed this product, there are no carries;
    // the closing barrier (this is the product's last kernel) is still this kernel's to run.
    if (!(rowBlockCap != 0 && *maxRowLen <= rowBlockCap)) {
        JoinCarries<kIn>(y, plan, p);
    }
    aclsp::CloseWithNodeBarrier(p.barrier);
}

int EnvInt(const char* name, int fallback)
{
    const char* e = std::getenv(name);
    return e == nullptr ? fallback : std::atoi(e);
}

template <int kIn>
void LaunchRowBlocks(const void* colInd, const void* values, const void* x, void* y, const SpmvPlanView& plan,
                     const AclspSpmvParams& p, const uint32_t* maxRowLen, uint32_t* waitFailures, int cap, bool checkPlan,
                     cudaStream_t s)
{
    constexpr int kAlign = kIn == kF32 ? 4 : 8;
    constexpr int kStages = 1;
    constexpr int kWarpsPerCta = 2;
    constexpr int kUnroll = 16;
    int device = 0;
    int sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
        sms = 148;
    }
    const size_t smem = sizeof(float) * kWarpsPerCta * kStages * RowBlockStageWords(cap, kAlign) +
                        sizeof(uint64_t) * kWarpsPerCta * kStages;
    auto kernel = SpmvRowBlockKernel<kStages, kWarpsPerCta, kUnroll, kIn>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    // Resident CTAs per SM: what shared memory holds (a CTA also takes 1 KiB of system shared memory),
    // at most 32 CTAs and 32 warps of this register footprint.
    uint32_t ctasPerSm = static_cast<uint32_t>((220u * 1024u) / (smem + 1024u));
    ctasPerSm = ctasPerSm > 32u / kWarpsPerCta ? 32u / kWarpsPerCta : (ctasPerSm > 0 ? ctasPerSm : 1u);
    const uint32_t numBlocks = (p.rows + kBlockRows - 1u) / kBlockRows;
    uint32_t grid = static_cast<uint32_t>(sms) * ctasPerSm;
    const uint32_t needed = (numBlocks + kWarpsPerCta - 1u) / kWarpsPerCta;
    grid = grid < needed ? grid : needed;
    AclspCountLaunches(1);
    kernel<<<grid > 0 ? grid : 1u, 32 * kWarpsPerCta, smem, s>>>(
        static_cast<const int32_t*>(colInd), static_cast<const float*>(values), static_cast<const float*>(x),
        static_cast<float*>(y), plan, p, maxRowLen, waitFailures, cap, checkPlan ? 1 : 0);
}

// One product of element type kIn: picks the kernel (see spmv_b200_kernel_do) and launches it.
template <int kIn>
void LaunchProduct(const void* colInd, const void* values, const void* x, void* y, void* workspace,
                   const SpmvPlanView& plan, const AclspSpmvParams& p, cudaStream_t s)
{
    // 128-bit loads and bulk copies: 4- or 2-byte values, unit strides, 16-byte aligned arrays.
    constexpr bool kCanVector = kIn == kF32 || kIn == kF16 || kIn == kBF16;
    const bool vector = kCanVector && p.colIndStride == 1 && p.valuesStride == 1 && p.xStride == 1 &&
                        reinterpret_cast<uintptr_t>(colInd) % 16 == 0 && reinterpret_cast<uintptr_t>(values) % 16 == 0;
    auto* header = static_cast<unsigned char*>(workspace);
    const auto* maxRowLen = reinterpret_cast<const uint32_t*>(header + ACLSP_HEADER_MAX_ROW_LEN_OFF);
    auto* waitFailures = reinterpret_cast<uint32_t*>(header + ACLSP_HEADER_WAIT_FAILURES_OFF);
    // The row-block kernel needs unit strides and 16-byte aligned sources for its bulk copies (the CSR
    // arrays and the row offsets inside the plan), and a stage that holds the longest row.  It pays when
    // rows are short and of similar length, i.e. when the longest row is not much longer than the mean.
    // ACLSPARSE_SPMV_ROW_BLOCKS=0 switches the row-block kernel off (a debugging aid, read once).
    static const int rowBlocksEnv = EnvInt("ACLSPARSE_SPMV_ROW_BLOCKS", 1);
    const bool eligible = vector && rowBlocksEnv != 0 && reinterpret_cast<uintptr_t>(plan.rowPtr) % 16 == 0 &&
                          p.rows > 0 && p.nnz > 0;
    uint32_t cap = 0;         // != 0: launch the row-block kernel with stages for rows of this length
    bool checkPlan = false;   // the kernels decide by the plan header which of them computes
    if (eligible && p.maxRowLenHint != ACLSP_MAX_ROW_LEN_UNKNOWN) {
        // The longest row is known: exactly one kernel is launched.
        const uint64_t longest = p.maxRowLenHint;
        if (longest <= static_cast<uint64_t>(kRowBlockMaxLen) && longest * p.rows <= 3ull * p.nnz + p.rows) {
            cap = static_cast<uint32_t>(longest > 0 ? longest : 1u);
        }
    } else if (eligible) {
        // Not known yet: guess from the mean row length, launch both, let the plan header decide.
        const uint64_t mean8 = (8ull * p.nnz + p.rows - 1u) / p.rows;  // mean row length, in eighths, rounded up
        cap = mean8 <= 8u * 14u ? 16u : (mean8 <= 8u * 28u ? 32u : 0u);
        checkPlan = cap != 0;
    }
    // The closing barrier of a sharded product belongs to the last kernel launched: the row-block kernel
    // when it is the only one, else the carry fix-up.
    AclspSpmvParams inner = p;
    inner.barrier.world = 0;
    if constexpr (kCanVector) {
        if (cap != 0) {
            LaunchRowBlocks<kIn>(colInd, values, x, y, plan, checkPlan ? inner : p, maxRowLen, waitFailures,
                                 static_cast<int>(cap), checkPlan, s);
            if (!checkPlan) {
                return;
            }
        }
    }
    const uint32_t tileCap = checkPlan ? cap : 0u;
    const auto* ci = static_cast<const int32_t*>(colInd);
    const auto* va = static_cast<const float*>(values);  // typed by kIn inside the kernels
    const auto* xv = static_cast<const float*>(x);
    auto* yv = static_cast<float*>(y);
    AclspCountLaunches(2);
    bool launched = false;
    if constexpr (kCanVector) {
        if (vector) {
            SpmvTileKernel<true, kIn><<<plan.numTiles, kThreads, 0, s>>>(ci, va, xv, yv, plan, inner, maxRowLen, tileCap);
            launched = true;
        }
    }
    if (!launched) {
        SpmvTileKernel<false, kIn><<<plan.numTiles, kThreads, 0, s>>>(ci, va, xv, yv, plan, inner, maxRowLen, tileCap);
    }
    const uint32_t fixupWarps = (plan.numTiles + 31u) / 32u;
    SpmvCarryFixupKernel<kIn><<<(fixupWarps + kWarps - 1u) / kWarps, kThreads, 0, s>>>(yv, plan, p, maxRowLen, tileCap);
}

}  // namespace

extern "C" void spmv_b200_kernel_do(const void* colInd, const void* values, const void* x, void* y,
                                    void* workspace, const AclspSpmvParams* params, void* stream)
{
    auto s = static_cast<cudaStream_t>(stream);
    AclspSpmvParams p = *params;
    // Bit 1 of mirrorMulticast (internal): send a tile's finished rows to the mirrors as one contiguous
    // run of 16-byte vectors after the tile, instead of row by row as they are produced.  Row by row costs
    // the kernel nothing but arrives as 32- to 64-byte packets (about 185 GB/s into a B200, measured), enough
    // for one or two peers; batching costs a barrier per tile (+10 % kernel time) and is what keeps 8 GPUs
    // fed.  ACLSPARSE_SPMV_MIRROR_BATCH=0 / 1 overrides the choice.
    static const int batchEnv = [] {
        const char* e = std::getenv("ACLSPARSE_SPMV_MIRROR_BATCH");
        return e == nullptr ? -1 : (e[0] == '1' ? 1 : 0);
    }();
    const bool multicast = (p.mirrorMulticast & 1u) != 0;
    const bool batch = batchEnv >= 0 ? batchEnv == 1 : (multicast || p.numMirrors >= 3);
    p.mirrorMulticast = (multicast ? 1u : 0u) | (batch ? 2u : 0u);
    const SpmvPlanView plan = MakeView(workspace, p.rows, p.nnz);
    if (plan.numTiles == 0) {
        return;
    }
    if (p.valueType == ACLSP_TYPE_F32) {
        LaunchProduct<kF32>(colInd, values, x, y, workspace, plan, p, s);
        return;
    }
    p.numMirrors = 0;  // mirrors of y and the closing barrier are for fp32 products
    p.barrier.world = 0;
    if (p.valueType == ACLSP_TYPE_F16) {
        LaunchProduct<kF16>(colInd, values, x, y, workspace, plan, p, s);
    } else if (p.valueType == ACLSP_TYPE_BF16) {
        LaunchProduct<kBF16>(colInd, values, x, y, workspace, plan, p, s);
    } else if (p.valueType == ACLSP_TYPE_I8) {
        LaunchProduct<kI8>(colInd, values, x, y, workspace, plan, p, s);
    }
}
