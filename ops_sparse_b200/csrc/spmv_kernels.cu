/*
 * CSR SpMV for sm_100a:  y = alpha * A * x + beta * y,  fp32 data, int32 indices.
 *
 * Work decomposition.  The matrix is cut along the merge path of (row ends,
 * non-zeros) into tiles of kTile items, so a tile holds at most kTile
 * non-zeros plus rows whatever the row-length distribution: short rows, empty
 * rows and 200 000-entry rows all cost the same per item.  One CTA owns one
 * tile:
 *   1. the tile's slice of colInd / values is streamed with 128-bit loads
 *      (evict-first: it is read exactly once), x[col] is gathered through the
 *      read-only path, and every product is staged in shared memory as an
 *      exact pair of floats (rounded product, rounding error) with 128-bit,
 *      conflict-free stores;
 *   2. rows that end inside the tile are reduced by groups of 2^class lanes
 *      ("vector per row", class picked per tile by the preprocessing pass from
 *      the tile's mean row length; class 5 is warp per row) with a shuffle
 *      tree; pieces of kWarpSegment products or more that are too long for their
 *      lanes get a whole warp each (warp per row), pieces of kLongSegment or
 *      more the whole CTA;
 *   3. the piece of a row that continues into the next tile becomes the tile's
 *      carry-out, and the piece of a row that began in an earlier tile becomes
 *      its head partial; a second small kernel adds the carries of a split row
 *      in tile order and writes that row.
 * Every sum is taken in a fixed order, so results are bit-reproducible.
 *
 * Accuracy.  Every product is kept exactly (hi + lo) and the hi parts are summed
 * in fp64 (the lo parts, 2^-24 of the products, in fp32), so
 * a row is as accurate as the reference's host golden (SpmvCpu with a double
 * accumulator, test/spmv/arch22/spmv_test.cpp:258-279,309-348) up to the order
 * of the additions; the reference's device kernels reach for compensated
 * arithmetic for the same reason (sparse/spmv/arch22/kernels/spmv_kernel.h:19-68).
 *
 * The kernels never read or write out of bounds for any content of the index
 * arrays: offsets are clamped to [0, nnz] and entries whose column falls
 * outside [0, cols) are skipped, as the reference's kernels do
 * (sparse/spmv/arch35/spmv_kernel.cpp:511-521).
 */
#include <cstdint>

#include <cstdlib>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "plan_layout.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTile = ACLSP_SPMV_TILE_ITEMS;
constexpr int kWarpSegment = 64;    // pieces at least this long get a whole warp
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

/* ------------------------------------------------------------ product -- */

struct Scalars {
    double alpha;
    double beta;
    bool betaZero;
};

__device__ __forceinline__ Scalars LoadScalars(const AclspSpmvParams& p)
{
    const float a = p.alphaPtr != nullptr ? *p.alphaPtr : p.alpha;
    const float b = p.betaPtr != nullptr ? *p.betaPtr : p.beta;
    Scalars s;
    s.alpha = static_cast<double>(a);
    s.beta = static_cast<double>(b);
    s.betaZero = b == 0.0f;
    return s;
}

// beta == 0 must not read y: it may hold NaN or be uninitialised.
__device__ __forceinline__ float StoreRow(float* __restrict__ y, int64_t index, double sum, const Scalars& s)
{
    const double r = s.betaZero ? s.alpha * sum : s.alpha * sum + s.beta * static_cast<double>(y[index]);
    const float out = static_cast<float>(r);
    y[index] = out;
    return out;
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
__device__ __forceinline__ void Product(float a, int32_t rawCol, const float* __restrict__ x, uint32_t base,
                                        uint32_t cols, int64_t xStride, float& hi, float& lo)
{
    const uint32_t c = static_cast<uint32_t>(rawCol) - base;
    if (c >= cols) {
        hi = 0.0f;
        lo = 0.0f;
        return;
    }
    const float xv = __ldg(x + static_cast<int64_t>(c) * xStride);
    hi = __fmul_rn(a, xv);
    lo = fmaf(a, xv, -hi);
}

/* ------------------------------------------------------------- reduce -- */

// Shared scratch of the reduction, one per CTA.
struct ReduceScratch {
    double warp[kWarps];
    int longSeg[kMaxLong];
    int warpSeg[kMaxWarpSeg];
    int numLong;
    int numWarpSeg;
};

// The staged tile: nt exact products (hi, lo), the nr + 1 row offsets relative
// to the tile's first product, and nr spare words for the mirrors of y.
struct StagedTile {
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
        if (k >= nr) {
            plan.carry[2 * t] = sum;
        } else if (k == 0 && headOpen) {
            plan.carry[2 * t + 1] = sum;
        } else {
            float* at = y + static_cast<int64_t>(i0 + k) * p.yStride;
            const float out = StoreRow(at, 0, sum, sc);
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
            if (len >= kWarpSegment && len >= 32 * lanes) {
                // Too long for its lanes: queue it for a warp, or for the whole CTA.
                // A valid CSR fills neither list beyond its capacity; row offsets
                // that overlap could, and the excess is dropped.
                if (lane == 0) {
                    if (len >= kLongSegment) {
                        const int slot = atomicAdd(&sNumLong, 1);
                        if (slot < kMaxLong) {
                            sLong[slot] = k;
                        }
                    } else {
                        const int slot = atomicAdd(&sNumWarpSeg, 1);
                        if (slot < kMaxWarpSeg) {
                            sWarpSeg[slot] = k;
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

template <bool kVector>
__global__ void __launch_bounds__(kThreads)
SpmvTileKernel(const int32_t* __restrict__ colInd, const float* __restrict__ values, const float* __restrict__ x,
               float* __restrict__ y, SpmvPlanView plan, AclspSpmvParams p)
{
    // One pool of 32-bit words: the hi parts of the tile's products, their lo
    // parts, and the tile's row offsets packed against the end.  A tile has nt
    // products and nr + 1 offsets with nt + nr <= kTile.
    __shared__ __align__(16) float sPool[2 * kTile + 24];
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
    const int a0 = kVector ? (j0 & ~3) : j0;
    const int shift = j0 - a0;
    const int span = (nt + shift + 3) & ~3;
    float* sHi = sPool;
    float* sLo = sPool + span;
    int* sOff = reinterpret_cast<int*>(sPool + 2 * kTile + 24) - (nr + 2);
    // nr more words fit between the products and the offsets (2 * span <= 2 * nt + 12 and
    // nt + nr <= kTile): the finished rows' values, kept for the mirrors of y.
    float* sOut = reinterpret_cast<float*>(sOff) - nr;
    if (tid == 0) {
        scratch.numLong = 0;
        scratch.numWarpSeg = 0;
    }
    for (int k = tid; k <= nr; k += kThreads) {
        sOff[k] = ClampOffset(plan.rowPtr[i0 + k], nnz) - j0;
    }

    if (kVector) {
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
            Product(values[e * p.valuesStride], colInd[e * p.colIndStride], x, p.indexBase, p.cols, p.xStride,
                    sHi[k], sLo[k]);
        }
    }
    __syncthreads();

    StagedTile st;
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
    ReduceTile(st, y, plan, p, scratch);
}

/* ------------------------------------- persistent, bulk-copy fed -- */

// The same tile work inside a persistent CTA that never issues a global load
// for the matrix: thread 0 asks the copy engine (cp.async.bulk, completion on an
// mbarrier) for the tile's slice of values, colInd and row offsets kStreamStages
// tiles ahead, straight into the shared-memory words where the products will
// replace them.  Measured on B200 (27-point stencil, 4.1 M rows): the copies
// alone stream at 6.7 TB/s, but a CTA needs about 3.6 us of dependent latency per
// tile (x gather, barriers, reduction) whatever runs beside it, and the stages
// leave room for only 4 CTAs per SM, so the whole product takes 0.33 ms against
// 0.26 ms for the one-CTA-per-tile kernel with its 6 CTAs per SM.  It is
// therefore opt-in (ACLSPARSE_SPMV_STREAM=1) and kept bit-identical to the
// default kernel by the tests.
constexpr int kStreamStages = 3;
constexpr int kStageWords = 2 * kTile + 24;
constexpr int kStreamCtasPerSm = 4;
constexpr uint32_t kSpinLimit = 1u << 18;  // polls of about a microsecond before a wait is given up

struct TileGeom {
    int i0, i1, j0, nr, nt;
    int a0, shift, span;     // first 4-aligned array index, distance of the tile's first product from it, words staged
    int copyElems;           // leading part of the span that is whole vectors inside the arrays: bulk-copied
    int offFirst, offShift;  // first 4-aligned row offset copied, distance of row i0 from it
    int offWords;
    bool valid;
};

__device__ __forceinline__ TileGeom Geometry(uint32_t t, int i0, int i1, const AclspSpmvParams& p)
{
    TileGeom g;
    const int nnz = static_cast<int>(p.nnz);
    const int64_t total = static_cast<int64_t>(p.rows) + nnz;
    int64_t d0 = static_cast<int64_t>(t) * kTile;
    int64_t d1 = d0 + kTile;
    d0 = d0 < total ? d0 : total;
    d1 = d1 < total ? d1 : total;
    g.i0 = i0;
    g.i1 = i1;
    g.j0 = static_cast<int>(d0 - i0);
    const int j1 = static_cast<int>(d1 - i1);
    g.nr = i1 - i0;
    g.nt = j1 - g.j0;
    g.valid = !(g.nr < 0 || g.nt < 0 || g.nr + g.nt > kTile || i0 < 0 || i1 > static_cast<int>(p.rows) || g.j0 < 0 ||
                j1 > nnz);
    g.a0 = g.j0 & ~3;
    g.shift = g.j0 - g.a0;
    g.span = (g.nt + g.shift + 3) & ~3;
    const int whole = (nnz & ~3) - g.a0;
    g.copyElems = whole < 0 ? 0 : (whole < g.span ? whole : g.span);
    g.offFirst = i0 & ~3;
    g.offShift = i0 - g.offFirst;
    g.offWords = (g.nr + 1 + g.offShift + 3) & ~3;
    return g;
}

__device__ __forceinline__ uint32_t SharedAddress(const void* ptr)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}

// The matrix is read once per product: its lines are marked evict-first in L2 so
// that they do not push x (which every tile gathers from) out of it.
__device__ __forceinline__ uint64_t EvictFirstPolicy()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void BulkLoad(void* smemDst, const void* gmemSrc, uint32_t bytes, uint64_t* bar,
                                         uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::
            "r"(SharedAddress(smemDst)),
        "l"(gmemSrc), "r"(bytes), "r"(SharedAddress(bar)), "l"(policy)
        : "memory");
}

// Thread 0: announce the bytes of a tile to the stage's barrier and start its copies.
__device__ __forceinline__ void IssueTile(const TileGeom& g, float* stage, uint64_t* bar, const int32_t* colInd,
                                          const float* values, const int32_t* rowPtr, uint64_t policy)
{
    const uint32_t arrayBytes = g.valid ? 4u * static_cast<uint32_t>(g.copyElems) : 0u;
    const uint32_t offBytes = g.valid ? 4u * static_cast<uint32_t>(g.offWords) : 0u;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(SharedAddress(bar)),
                 "r"(2u * arrayBytes + offBytes)
                 : "memory");
    if (arrayBytes != 0) {
        BulkLoad(stage, values + g.a0, arrayBytes, bar, policy);
        BulkLoad(stage + g.span, colInd + g.a0, arrayBytes, bar, policy);
    }
    if (offBytes != 0) {
        BulkLoad(stage + 2 * g.span, rowPtr + g.offFirst, offBytes, bar, policy);
    }
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

template <int kStages, int kCtas>
__global__ void __launch_bounds__(kThreads, kCtas)
SpmvStreamKernel(const int32_t* __restrict__ colInd, const float* __restrict__ values, const float* __restrict__ x,
                 float* __restrict__ y, SpmvPlanView plan, AclspSpmvParams p, uint32_t* __restrict__ waitFailures)
{
    extern __shared__ __align__(128) unsigned char smemRaw[];
    float* stages = reinterpret_cast<float*>(smemRaw);                                   // kStages * kStageWords
    uint64_t* full = reinterpret_cast<uint64_t*>(stages + kStages * kStageWords);  // kStages barriers
    ReduceScratch& scratch = *reinterpret_cast<ReduceScratch*>(full + kStages);

    const int tid = threadIdx.x;
    const int nnz = static_cast<int>(p.nnz);
    const uint32_t numTiles = plan.numTiles;
    const uint32_t stride = gridDim.x;
    const uint64_t policy = EvictFirstPolicy();

    if (tid == 0) {
        for (int sIdx = 0; sIdx < kStages; ++sIdx) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(SharedAddress(full + sIdx)) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        uint32_t t = blockIdx.x;
        for (int sIdx = 0; sIdx < kStages && t < numTiles; ++sIdx, t += stride) {
            const TileGeom g = Geometry(t, plan.tileRow[t], plan.tileRow[t + 1], p);
            IssueTile(g, stages + sIdx * kStageWords, full + sIdx, colInd, values, plan.rowPtr, policy);
        }
    }
    __syncthreads();

    // Split points and row bin of the tile after this one, fetched a tile ahead.
    uint32_t t = blockIdx.x;
    int nextI0 = 0, nextI1 = 0, nextCls = 0;
    if (t < numTiles) {
        nextI0 = plan.tileRow[t];
        nextI1 = plan.tileRow[t + 1];
        nextCls = plan.tileClass[t];
    }
    bool waitedOut = false;
    for (uint32_t it = 0; t < numTiles; ++it, t += stride) {
        const int sIdx = static_cast<int>(it % kStages);
        const uint32_t parity = (it / kStages) & 1u;
        float* stage = stages + sIdx * kStageWords;
        const TileGeom g = Geometry(t, nextI0, nextI1, p);
        const int cls = nextCls;
        const uint32_t tNext = t + stride;
        if (tNext < numTiles) {
            nextI0 = plan.tileRow[tNext];
            nextI1 = plan.tileRow[tNext + 1];
            nextCls = plan.tileClass[tNext];
        }
        // Thread 0 refills this stage after the tile: its split points are fetched now.
        const uint32_t tRefill = t + kStages * stride;
        int refillI0 = 0, refillI1 = 0;
        if (tid == 0 && tRefill < numTiles) {
            refillI0 = plan.tileRow[tRefill];
            refillI1 = plan.tileRow[tRefill + 1];
        }
        if (tid == 0) {
            scratch.numLong = 0;
            scratch.numWarpSeg = 0;
        }
        // A wait that runs out is recorded and the tile goes on with whatever the
        // stage holds: indices are range-checked, so the worst outcome is a wrong
        // value, and every thread keeps reaching the barriers below.
        if (!waitedOut && !WaitStage(full + sIdx, parity)) {
            waitedOut = true;  // and no further wait of this CTA is attempted
        }

        if (!g.valid) {
            if (tid == 0) {
                plan.carry[2 * t] = 0.0;
                plan.carry[2 * t + 1] = 0.0;
            }
        } else {
            float* sHi = stage;            // values, then the hi parts
            float* sLo = stage + g.span;   // colInd, then the lo parts
            int* sOff = reinterpret_cast<int*>(stage + 2 * g.span) + g.offShift;
            float* sOut = stage + 2 * g.span + g.offWords;
            for (int k = tid; k <= g.nr; k += kThreads) {
                sOff[k] = ClampOffset(sOff[k], nnz) - g.j0;
            }
            const int nvec = g.span >> 2;
            const int copied = g.copyElems >> 2;
            struct Vec4 {
                int4 c;
                float4 w;
            };
            auto loadVec = [&](int v, Vec4& o) {
                if (v < copied) {
                    o.w = *reinterpret_cast<const float4*>(sHi + 4 * v);
                    o.c = *reinterpret_cast<const int4*>(sLo + 4 * v);
                } else {  // the last, partial vector of the arrays: plain loads
                    const int e = g.a0 + 4 * v;
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
            auto useVec = [&](int v, const Vec4& o) {
                float4 hi, lo;
                Product(o.w.x, o.c.x, x, p.indexBase, p.cols, 1, hi.x, lo.x);
                Product(o.w.y, o.c.y, x, p.indexBase, p.cols, 1, hi.y, lo.y);
                Product(o.w.z, o.c.z, x, p.indexBase, p.cols, 1, hi.z, lo.z);
                Product(o.w.w, o.c.w, x, p.indexBase, p.cols, 1, hi.w, lo.w);
                *reinterpret_cast<float4*>(sHi + 4 * v) = hi;
                *reinterpret_cast<float4*>(sLo + 4 * v) = lo;
            };
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
            __syncthreads();

            StagedTile st;
            st.t = static_cast<int>(t);
            st.i0 = g.i0;
            st.i1 = g.i1;
            st.nr = g.nr;
            st.nt = g.nt;
            st.cls = cls;
            st.hiT = sHi + g.shift;
            st.loT = sLo + g.shift;
            st.sOff = sOff;
            st.sOut = sOut;
            ReduceTile(st, y, plan, p, scratch);
        }
        __syncthreads();  // the stage and the scratch are free
        if (tid == 0 && tRefill < numTiles) {
            // Shared-memory writes of the tile above come before the copy engine's writes.
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            const TileGeom r = Geometry(tRefill, refillI0, refillI1, p);
            IssueTile(r, stage, full + sIdx, colInd, values, plan.rowPtr, policy);
        }
    }
    if (waitedOut) {
        atomicAdd(waitFailures, 1u);
    }
}

// One thread per tile whose first row began in an earlier tile and ends in
// this one: adds the carry-outs of the tiles the row crossed, oldest first,
// then the head partial, and writes the row.
__global__ void SpmvCarryFixupKernel(float* __restrict__ y, SpmvPlanView plan, AclspSpmvParams p)
{
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= plan.numTiles) {
        return;
    }
    const int nnz = static_cast<int>(p.nnz);
    const int i0 = plan.tileRow[t];
    const int i1 = plan.tileRow[t + 1];
    if (i1 <= i0 || i0 < 0 || i0 >= static_cast<int>(p.rows)) {
        return;
    }
    const int64_t total = static_cast<int64_t>(p.rows) + nnz;
    int64_t d0 = static_cast<int64_t>(t) * kTile;
    d0 = d0 < total ? d0 : total;
    const int64_t j0 = d0 - i0;
    if (ClampOffset(plan.rowPtr[i0], nnz) >= j0) {
        return;
    }
    uint32_t first = t;
    while (first > 0 && plan.tileRow[first] == i0) {
        --first;
    }
    double sum = 0.0;
    for (uint32_t u = first; u < t; ++u) {
        sum += plan.carry[2 * u];
    }
    sum += plan.carry[2 * t + 1];
    float* at = y + static_cast<int64_t>(i0) * p.yStride;
    const float out = StoreRow(at, 0, sum, LoadScalars(p));
    if (p.numMirrors != 0) {
        MirrorStore(at, out, p);
    }
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
    const bool vector = p.colIndStride == 1 && p.valuesStride == 1 && p.xStride == 1 &&
                        reinterpret_cast<uintptr_t>(colInd) % 16 == 0 && reinterpret_cast<uintptr_t>(values) % 16 == 0;
    // ACLSPARSE_SPMV_STREAM=1 selects the persistent bulk-copy kernel.  It needs 16-byte aligned sources
    // for its copies: the CSR arrays (as the vector path does) and the row offsets inside the plan.
    static const bool streamEnv = [] {
        const char* e = std::getenv("ACLSPARSE_SPMV_STREAM");
        return e != nullptr && e[0] == '1';
    }();
    const bool streamed = vector && streamEnv && reinterpret_cast<uintptr_t>(plan.rowPtr) % 16 == 0;
    if (streamed) {
        int device = 0;
        int sms = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
            sms = 148;
        }
        auto* waitFailures =
            reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(workspace) + ACLSP_HEADER_WAIT_FAILURES_OFF);
        auto launch = [&](auto kernel, int stages, int ctas) {
            const size_t smem = sizeof(float) * stages * kStageWords + sizeof(uint64_t) * stages + sizeof(ReduceScratch);
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            const uint32_t resident = static_cast<uint32_t>(sms) * ctas;
            const uint32_t grid = plan.numTiles < resident ? plan.numTiles : resident;
            kernel<<<grid, kThreads, smem, s>>>(static_cast<const int32_t*>(colInd), static_cast<const float*>(values),
                                                static_cast<const float*>(x), static_cast<float*>(y), plan, p,
                                                waitFailures);
        };
        // Also measured: 2 stages with 5 / 6 CTAs per SM (48 / 40 registers): 0.344 / 0.381 ms on the stencil.
        launch(SpmvStreamKernel<kStreamStages, kStreamCtasPerSm>, kStreamStages, kStreamCtasPerSm);
    } else if (vector) {
        SpmvTileKernel<true><<<plan.numTiles, kThreads, 0, s>>>(
            static_cast<const int32_t*>(colInd), static_cast<const float*>(values), static_cast<const float*>(x),
            static_cast<float*>(y), plan, p);
    } else {
        SpmvTileKernel<false><<<plan.numTiles, kThreads, 0, s>>>(
            static_cast<const int32_t*>(colInd), static_cast<const float*>(values), static_cast<const float*>(x),
            static_cast<float*>(y), plan, p);
    }
    SpmvCarryFixupKernel<<<(plan.numTiles + 255u) / 256u, 256, 0, s>>>(static_cast<float*>(y), plan, p);
}
