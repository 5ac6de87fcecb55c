/*
 * TEST INFRASTRUCTURE ONLY.  Thin C entry points around a few of the
 * reference's own host-side sources, compiled where they lie (the include
 * paths point into the reference checkout; see oracle/Makefile, target `ref`).
 * The resulting oracle/_ref/libref_host.so is used to check the oracle's
 * restatement against the reference's real code and to generate the golden
 * fixtures under tests/golden/.  No reference source is copied here.
 *
 * What is wrapped:
 *   - SpmmGolden, the fp64 triple-loop golden (test/spmm_op/spmm_op_golden.h:177-205);
 *   - SparseFillGenerator, the test CSR generator (test/frame/fill.h:55-195);
 *   - SpmvArch35WorkspaceBytes (sparse/spmv/arch35/spmv_tiling_data.h:96-127);
 *   - SpmmCsrMat::DoPreProcess, i.e. GreedyRowBinPack / BuildIdentityRowReorder
 *     (sparse/spmm/arch35/host/spmm_csr_mat.cpp:37-210), run with host memory
 *     standing in for device memory.
 */
#include <cstdint>
#include <cstring>
#include <vector>

#include "cann_ops_sparse.h"
#include "spmm_op_golden.h"
#include "fill.h"
#include "spmv_tiling_data.h"
#include "spmm_csr_mat.cpp"

extern "C" {

void ref_spmm_golden_f64(int64_t m, int64_t n, int64_t k, const int32_t* rowPtr, const int32_t* colInd,
                         const float* values, int64_t nnz, const float* B, const float* cInit, double alpha,
                         double beta, int opBTranspose, int32_t indexBase, double* out)
{
    sparse_test::SpmmCsr csr;
    csr.rowOffsets.assign(rowPtr, rowPtr + m + 1);
    csr.colIndices.assign(colInd, colInd + nnz);
    csr.values.assign(values, values + nnz);
    csr.m = m;
    csr.k = k;
    csr.nnz = nnz;
    csr.indexBase = indexBase;
    const std::vector<double> b(B, B + k * n);
    const std::vector<double> c(cInit, cInit + m * n);
    const auto res = sparse_test::SpmmGolden(m, n, k, csr, b, c, alpha, beta,
                                             opBTranspose ? ACL_SPARSE_OP_TRANSPOSE : ACL_SPARSE_OP_NON_TRANSPOSE);
    std::memcpy(out, res.data(), sizeof(double) * res.size());
}

/* Returns nnz; fills the arrays when they are large enough (capacity in elements). */
int64_t ref_fill_csr(int64_t rows, int64_t cols, double sparsity, double emptyRowProb, double lo, double hi,
                     uint32_t seed, int32_t* rowOffsets, int32_t* colIndices, float* values, int64_t capacity)
{
    sparse_test::SparseFillGenerator gen(seed);
    gen.setSparsity(sparsity);
    gen.setEmptyRowProb(emptyRowProb);
    gen.setValueRange(lo, hi);
    const sparse_test::CsrMatrix csr = gen.generateCsr(rows, cols);
    if (csr.nnz <= capacity) {
        std::memcpy(rowOffsets, csr.rowOffsets.data(), sizeof(int32_t) * (rows + 1));
        std::memcpy(colIndices, csr.colIndices.data(), sizeof(int32_t) * csr.nnz);
        std::memcpy(values, csr.values.data(), sizeof(float) * csr.nnz);
    }
    return csr.nnz;
}

void ref_fill_dense(int64_t size, double lo, double hi, uint32_t seed, float* out)
{
    sparse_test::SparseFillGenerator gen(seed);
    gen.setValueRange(lo, hi);
    const auto v = gen.generateDenseFloat(size);
    std::memcpy(out, v.data(), sizeof(float) * size);
}

uint64_t ref_spmv_workspace_bytes(uint64_t rows, uint64_t cols, int transpose)
{
    size_t bytes = 0;
    if (!SpmvArch35WorkspaceBytes(rows, cols, SPMV35_COMPUTE_F32, transpose != 0, &bytes)) {
        return 0;
    }
    return bytes;
}

/* reorder[m], binEdges[bins+1].  Returns the reference's status code. */
uint32_t ref_spmm_row_reorder(const int32_t* rowPtr, int64_t m, int64_t k, int64_t nnz, int32_t bins,
                              int32_t* reorder, int32_t* binEdges, int* identityReorder, int32_t* uniformDegree)
{
    aclsparseSpMatDescr descr;
    descr.format = ACL_SPARSE_FORMAT_CSR;
    descr.rows = static_cast<uint64_t>(m);
    descr.cols = static_cast<uint64_t>(k);
    descr.nnz = static_cast<uint64_t>(nnz);
    descr.ptrs = const_cast<int32_t*>(rowPtr);
    descr.ptrType = ACL_SPARSE_INDEX_32I;
    descr.IdxType = ACL_SPARSE_INDEX_32I;
    const int64_t reorderOff = 0;
    const int64_t binEdgeOff = static_cast<int64_t>(sizeof(int32_t)) * (m > 0 ? m : 1);
    std::vector<uint8_t> workspace(static_cast<size_t>(binEdgeOff) + sizeof(int32_t) * (bins + 1));
    SpmmCsrMat csr(&descr, bins);
    const uint32_t st = csr.DoPreProcess(workspace.data(), reorderOff, binEdgeOff, false);
    if (st == 0) {
        std::memcpy(reorder, workspace.data() + reorderOff, sizeof(int32_t) * m);
        std::memcpy(binEdges, workspace.data() + binEdgeOff, sizeof(int32_t) * (bins + 1));
        *identityReorder = csr.IsIdentityReorder() ? 1 : 0;
        *uniformDegree = csr.GetUniformDegree();
    }
    return st;
}

}  // extern "C"
