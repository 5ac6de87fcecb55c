/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the ops-sparse host goldens
 * and of the preprocessing metadata for the CSR SpMV / SpMM path.  Nothing in
 * the shipped library calls into this file; it is the checker that the tests,
 * the smoke run and the benchmark's CPU baseline use.
 *
 * Each function names the reference file:line whose arithmetic it follows.
 * The oracle is pinned by the reference's own known-answer tests (see
 * tests/golden/reference_kats.json and tests/test_oracle.py).
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off so that no product/sum
 * pair is fused: the reference goldens round every product).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ SpMV -- */

/* fp64-accumulated truth of y = alpha*A*x + beta*y for fp32 data.
 * reference: SpmvCpu<double,float,double> as instantiated by BuildSpmvGolden,
 * test/spmv/arch22/spmv_test.cpp:258-279 and :309-348 — per row a sequential
 * sum of (double)val * (double)x[col], then alpha*sum + beta*y in double. */
ORACLE_API void oracle_spmv_f64(int64_t rows, const int32_t* rowPtr, const int32_t* colInd, const float* values,
                                const float* x, const float* yIn, double* out, float alpha, float beta,
                                int32_t indexBase, int threads)
{
    const double a = (double)alpha;
    const double b = (double)beta;
    (void)threads;
#pragma omp parallel for schedule(dynamic, 4096) num_threads(threads > 0 ? threads : 1)
    for (int64_t i = 0; i < rows; ++i) {
        double sum = 0.0;
        for (int64_t j = (int64_t)rowPtr[i] - indexBase; j < (int64_t)rowPtr[i + 1] - indexBase; ++j) {
            sum += (double)values[j] * (double)x[colInd[j] - indexBase];
        }
        out[i] = a * sum + b * (double)yIn[i];
    }
}

/* The same product with every operation in fp32.
 * reference: SpmvCpu<float,float,float>, test/spmv/arch22/spmv_test.cpp:258-279. */
ORACLE_API void oracle_spmv_f32(int64_t rows, const int32_t* rowPtr, const int32_t* colInd, const float* values,
                                const float* x, const float* yIn, float* out, float alpha, float beta,
                                int32_t indexBase)
{
    for (int64_t i = 0; i < rows; ++i) {
        float sum = 0.0f;
        for (int64_t j = (int64_t)rowPtr[i] - indexBase; j < (int64_t)rowPtr[i + 1] - indexBase; ++j) {
            const float prod = values[j] * x[colInd[j] - indexBase];
            sum += prod;
        }
        out[i] = alpha * sum + beta * yIn[i];
    }
}

/* reference: SpmvTransCpu<double,...>, test/spmv/arch22/spmv_test.cpp:283-307. */
ORACLE_API void oracle_spmv_transpose_f64(int64_t rows, int64_t cols, const int32_t* rowPtr, const int32_t* colInd,
                                          const float* values, const float* x, const float* yIn, double* out,
                                          float alpha, float beta, int32_t indexBase)
{
    for (int64_t j = 0; j < cols; ++j) {
        out[j] = (double)beta * (double)yIn[j];
    }
    for (int64_t i = 0; i < rows; ++i) {
        const double xv = (double)alpha * (double)x[i];
        if (xv == 0.0) {
            continue;
        }
        for (int64_t k = (int64_t)rowPtr[i] - indexBase; k < (int64_t)rowPtr[i + 1] - indexBase; ++k) {
            const int64_t c = colInd[k] - indexBase;
            out[c] = out[c] + xv * (double)values[k];
        }
    }
}

/* ------------------------------------------------------------------ SpMM -- */

static inline int64_t DenseIndex(int64_t r, int64_t c, int64_t ld, int rowMajor)
{
    return rowMajor ? r * ld + c : c * ld + r;
}

/* fp32 golden of C = alpha*A*op(B) + beta*C, layout / opB / index base aware.
 * reference: SpmmCpuFp32, test/spmm/arch35/spmm_test.cpp:247-283 — for every
 * (row, column) a sequential fp32 `acc += val * b` over the row's entries,
 * then alpha*acc + beta*cOld.  The loops here run (row, entry, column) with
 * one accumulator per column, which performs the same operations on every
 * accumulator in the same order.  With ld == n, row-major and opB = N this is
 * also spmm_csr_cpu of test/spmm/arch22/spmm_test.cpp:135-149. */
ORACLE_API void oracle_spmm_f32(int64_t m, int64_t n, const int32_t* rowPtr, const int32_t* colInd,
                                const float* values, const float* B, int64_t ldb, int bRowMajor, int opBTranspose,
                                float* C, int64_t ldc, int cRowMajor, float alpha, float beta, int32_t indexBase,
                                int threads)
{
    (void)threads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        float* acc = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
#pragma omp for schedule(dynamic, 256)
        for (int64_t r = 0; r < m; ++r) {
            for (int64_t j = 0; j < n; ++j) {
                acc[j] = 0.0f;
            }
            for (int64_t p = (int64_t)rowPtr[r] - indexBase; p < (int64_t)rowPtr[r + 1] - indexBase; ++p) {
                const int64_t c = colInd[p] - indexBase;
                const float v = values[p];
                /* op(B)[c, j]: B stored k x n (opB = N) or n x k (opB = T). */
                const int elementRowMajor = opBTranspose ? !bRowMajor : bRowMajor;
                for (int64_t j = 0; j < n; ++j) {
                    const float prod = v * B[DenseIndex(c, j, ldb, elementRowMajor)];
                    acc[j] += prod;
                }
            }
            for (int64_t j = 0; j < n; ++j) {
                const int64_t ci = DenseIndex(r, j, ldc, cRowMajor);
                C[ci] = alpha * acc[j] + beta * C[ci];
            }
        }
        free(acc);
    }
}

/* fp64 truth of the same product; out is canonical row-major m x n.
 * reference: SpmmGolden / SpmmGoldenDotProduct, test/spmm_op/spmm_op_golden.h:142-205
 * (entries whose column falls outside [0, k) are skipped there as well). */
ORACLE_API void oracle_spmm_f64(int64_t m, int64_t n, int64_t k, const int32_t* rowPtr, const int32_t* colInd,
                                const float* values, const float* B, int64_t ldb, int bRowMajor, int opBTranspose,
                                const float* Cin, int64_t ldc, int cRowMajor, double* out, float alpha, float beta,
                                int32_t indexBase, int64_t rowBegin, int64_t rowEnd, int threads)
{
    (void)threads;
    (void)m;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        double* acc = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
#pragma omp for schedule(dynamic, 256)
        for (int64_t r = rowBegin; r < rowEnd; ++r) {
            for (int64_t j = 0; j < n; ++j) {
                acc[j] = 0.0;
            }
            for (int64_t p = (int64_t)rowPtr[r] - indexBase; p < (int64_t)rowPtr[r + 1] - indexBase; ++p) {
                const int64_t c = colInd[p] - indexBase;
                if (c < 0 || c >= k) {
                    continue;
                }
                const double v = (double)values[p];
                const int elementRowMajor = opBTranspose ? !bRowMajor : bRowMajor;
                for (int64_t j = 0; j < n; ++j) {
                    acc[j] += v * (double)B[DenseIndex(c, j, ldb, elementRowMajor)];
                }
            }
            for (int64_t j = 0; j < n; ++j) {
                const double cOld = beta == 0.0f ? 0.0 : (double)Cin[DenseIndex(r, j, ldc, cRowMajor)];
                out[(r - rowBegin) * n + j] = (double)alpha * acc[j] + (double)beta * cOld;
            }
        }
        free(acc);
    }
}

/* ------------------------------------------------- reference metadata -- */

/* reference: SpmvArch35PreprocessKernel, sparse/spmv/arch35/spmv_kernel.cpp:1155-1158. */
ORACLE_API void oracle_normalize_row_offsets(const int32_t* rowPtr, int64_t rows, int32_t indexBase, int64_t stride,
                                             int32_t* out)
{
    for (int64_t i = 0; i <= rows; ++i) {
        out[i] = rowPtr[i * stride] - indexBase;
    }
}

/* reference: SpmvArch35WorkspaceBytes (non-transposed),
 * sparse/spmv/arch35/spmv_tiling_data.h:96-127: align64(192 + 4*(rows+1)). */
ORACLE_API uint64_t oracle_ref_spmv_workspace_bytes(uint64_t rows)
{
    return (192u + 4u * (rows + 1u) + 63u) & ~(uint64_t)63u;
}

/* reference: InitializeWsOffsets / ComputeWsOffsets without the tensor-unit
 * areas, sparse/spmm/arch35/host/spmm_host.cpp:685-705,928-950, with
 * sizeof(SpmmTilingWireV1) == 240 (sparse/spmm/arch35/spmm_tiling_wire.h:119). */
ORACLE_API uint64_t oracle_ref_spmm_workspace_bytes(uint64_t m, uint64_t bins)
{
    const uint64_t tilingOff = 64u;
    const uint64_t reorderOff = (tilingOff + 240u + 63u) & ~(uint64_t)63u;
    const uint64_t binEdgeOff = (reorderOff + 4u * m + 63u) & ~(uint64_t)63u;
    return (binEdgeOff + 4u * (bins + 1u) + 63u) & ~(uint64_t)63u;
}

typedef struct {
    int32_t nnz;
    int32_t row;
} RowKey;

static int CompareRowKey(const void* pa, const void* pb)
{
    const RowKey* a = (const RowKey*)pa;
    const RowKey* b = (const RowKey*)pb;
    if (a->nnz != b->nnz) {
        return a->nnz > b->nnz ? -1 : 1; /* longer rows first */
    }
    return a->row < b->row ? -1 : (a->row > b->row ? 1 : 0);
}

/* Binary min-heap of (load, bin), ordered like std::pair<int64_t,int32_t>
 * under std::greater: smallest load first, ties by smallest bin. */
typedef struct {
    int64_t load;
    int32_t bin;
} BinLoad;

static int BinLess(const BinLoad* a, const BinLoad* b)
{
    return a->load < b->load || (a->load == b->load && a->bin < b->bin);
}

static void HeapSiftDown(BinLoad* h, int32_t n, int32_t i)
{
    for (;;) {
        int32_t s = i;
        const int32_t l = 2 * i + 1;
        const int32_t r = l + 1;
        if (l < n && BinLess(&h[l], &h[s])) {
            s = l;
        }
        if (r < n && BinLess(&h[r], &h[s])) {
            s = r;
        }
        if (s == i) {
            return;
        }
        const BinLoad tmp = h[i];
        h[i] = h[s];
        h[s] = tmp;
        i = s;
    }
}

/* Row reorder and bin edges of the reference's SpMM preprocessing.
 * reference: GreedyRowBinPack and BuildIdentityRowReorder,
 * sparse/spmm/arch35/host/spmm_csr_mat.cpp:37-117 — near-uniform rows
 * (max - min <= 1) keep their order and are split evenly; otherwise rows
 * sorted by (nnz descending, index ascending) go one by one to the least
 * loaded bin, a row costing nnz + 1.
 * reorder[m], binEdges[bins+1]; returns identityReorder, *uniformDegree as there. */
ORACLE_API int oracle_greedy_row_bin_pack(const int32_t* rowNnz, int32_t m, int32_t bins, int32_t* reorder,
                                          int32_t* binEdges, int32_t* uniformDegree)
{
    int32_t mn = 0;
    int32_t mx = 0;
    for (int32_t i = 0; i < m; ++i) {
        if (i == 0 || rowNnz[i] < mn) {
            mn = rowNnz[i];
        }
        if (i == 0 || rowNnz[i] > mx) {
            mx = rowNnz[i];
        }
    }
    *uniformDegree = m == 0 ? 0 : (mn == mx ? mn : -1);
    if (m == 0 || mx - mn <= 1) {
        for (int32_t i = 0; i < m; ++i) {
            reorder[i] = i;
        }
        const int64_t perBin = ((int64_t)m + bins - 1) / bins;
        for (int32_t b = 0; b <= bins; ++b) {
            const int64_t edge = (int64_t)b * perBin;
            binEdges[b] = (int32_t)(edge < m ? edge : m);
        }
        return 1;
    }
    RowKey* order = (RowKey*)malloc(sizeof(RowKey) * (size_t)m);
    int32_t* binOf = (int32_t*)malloc(sizeof(int32_t) * (size_t)m);
    int32_t* count = (int32_t*)calloc((size_t)bins + 1, sizeof(int32_t));
    BinLoad* heap = (BinLoad*)malloc(sizeof(BinLoad) * (size_t)bins);
    for (int32_t i = 0; i < m; ++i) {
        order[i].nnz = rowNnz[i];
        order[i].row = i;
    }
    qsort(order, (size_t)m, sizeof(RowKey), CompareRowKey);
    for (int32_t b = 0; b < bins; ++b) {
        heap[b].load = 0;
        heap[b].bin = b; /* already a valid heap: equal loads, ascending bins */
    }
    for (int32_t i = 0; i < m; ++i) {
        const int32_t pick = heap[0].bin;
        binOf[i] = pick;
        ++count[pick + 1];
        heap[0].load += (int64_t)order[i].nnz + 1;
        HeapSiftDown(heap, bins, 0);
    }
    binEdges[0] = 0;
    for (int32_t b = 0; b < bins; ++b) {
        binEdges[b + 1] = binEdges[b] + count[b + 1];
    }
    /* Rows keep their visiting order inside a bin. */
    int32_t* cursor = (int32_t*)malloc(sizeof(int32_t) * (size_t)bins);
    for (int32_t b = 0; b < bins; ++b) {
        cursor[b] = binEdges[b];
    }
    for (int32_t i = 0; i < m; ++i) {
        reorder[cursor[binOf[i]]++] = order[i].row;
    }
    free(cursor);
    free(heap);
    free(count);
    free(binOf);
    free(order);
    return 0;
}

/* ---------------------------------------------------- B200 plan twin -- */

static inline int32_t ClampOffset(int32_t v, int32_t nnz)
{
    return v < 0 ? 0 : (v > nnz ? nnz : v);
}

static int32_t MergePathRow(const int32_t* rowPtr, int64_t rows, int64_t nnz, int64_t diag)
{
    int64_t lo = diag > nnz ? diag - nnz : 0;
    int64_t hi = diag < rows ? diag : rows;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if ((int64_t)ClampOffset(rowPtr[mid + 1], (int32_t)nnz) <= diag - 1 - mid) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    return (int32_t)lo;
}

/* CPU twin of the device preprocessing pass (no reference counterpart: the
 * merge-path tile split and the per-tile row bins are this library's own
 * metadata).  rowPtrN is base 0.  tileRow[numTiles+1], tileClass[numTiles]. */
ORACLE_API void oracle_plan_tiles(const int32_t* rowPtrN, int64_t rows, int64_t nnz, uint32_t tileItems,
                                  uint32_t classDiv, int32_t* tileRow, int32_t* tileClass)
{
    const int64_t total = rows + nnz;
    const int64_t numTiles = (total + tileItems - 1) / tileItems;
    for (int64_t t = 0; t <= numTiles; ++t) {
        int64_t d = t * (int64_t)tileItems;
        d = d < total ? d : total;
        tileRow[t] = MergePathRow(rowPtrN, rows, nnz, d);
    }
    for (int64_t t = 0; t < numTiles; ++t) {
        int64_t d0 = t * (int64_t)tileItems;
        int64_t d1 = d0 + tileItems;
        d0 = d0 < total ? d0 : total;
        d1 = d1 < total ? d1 : total;
        const int64_t nr = (int64_t)tileRow[t + 1] - tileRow[t];
        const int64_t nt = (d1 - tileRow[t + 1]) - (d0 - tileRow[t]);
        uint32_t cls = 0;
        if (nr >= 0 && nt >= 0) {
            const uint32_t avg = (uint32_t)nt / ((uint32_t)nr + 1u);
            const uint32_t want = (avg + classDiv - 1u) / classDiv;
            while (cls < 5u && (1u << cls) < want) {
                ++cls;
            }
        }
        tileClass[t] = (int32_t)cls;
    }
}

/* CPU twin of the nnz-balanced row-block split over `parts` devices. */
ORACLE_API void oracle_row_block_bounds(const int32_t* rowPtr, int64_t rows, int64_t nnz, int32_t indexBase,
                                        int32_t parts, int32_t* bounds)
{
    for (int32_t g = 0; g <= parts; ++g) {
        const int64_t target = ((int64_t)g * nnz + parts - 1) / parts;
        int64_t lo = 0;
        int64_t hi = rows;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if ((int64_t)rowPtr[mid] - indexBase >= target) {
                hi = mid;
            } else {
                lo = mid + 1;
            }
        }
        bounds[g] = g == parts ? (int32_t)rows : (int32_t)lo;
    }
}

/* ------------------------------------------------------------ verifier -- */

/* Counts elements with |got - truth| > atol + rtol*|truth| (or non-finite),
 * and reports the largest absolute and relative error.
 * reference: AccumulateSpmvVerification, test/spmv/arch22/spmv_test_verification.h:32-56. */
ORACLE_API int64_t oracle_check_tolerance(const float* got, const double* truth, int64_t count, double rtol,
                                          double atol, double* maxAbs, double* maxRel)
{
    int64_t bad = 0;
    double worstAbs = 0.0;
    double worstRel = 0.0;
    for (int64_t i = 0; i < count; ++i) {
        const double g = (double)got[i];
        const double t = truth[i];
        if (!isfinite(g) || !isfinite(t)) {
            ++bad;
            worstAbs = INFINITY;
            continue;
        }
        const double err = fabs(g - t);
        if (err > atol + rtol * fabs(t)) {
            ++bad;
        }
        if (err > worstAbs) {
            worstAbs = err;
        }
        if (t != 0.0 && err / fabs(t) > worstRel) {
            worstRel = err / fabs(t);
        }
    }
    if (maxAbs != NULL) {
        *maxAbs = worstAbs;
    }
    if (maxRel != NULL) {
        *maxRel = worstRel;
    }
    return bad;
}

ORACLE_API int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
