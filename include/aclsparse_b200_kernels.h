/*
 * Inner boundary: the C-ABI launch shim between the C++ host layer and the
 * sm_100a CUDA kernels.  The reference isolates its device code the same way,
 * behind `extern "C" void ..._kernel_do(raw pointers, POD tiling, stream)`
 * launchers that never synchronise and report nothing; the host detects an
 * enqueue failure by clearing and then peeking the runtime's last error
 * (reference: sparse/spmv/arch35/spmv_host.cpp:564-575,617-629).
 *
 * Every pointer below is a CUDA device pointer unless it is marked "host";
 * `stream` is a cudaStream_t.
 */
#ifndef ACLSPARSE_B200_KERNELS_H_
#define ACLSPARSE_B200_KERNELS_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility: only what this header declares is exported. */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Mirrors of an output: besides the result buffer itself a kernel can store every element it writes at the
 * same element position of up to ACLSP_MAX_MIRRORS further buffers - the result buffers of the other GPUs
 * of the node, mapped into this device's address space - so that the product and the reassembly of the
 * sharded result over NVLink are one kernel.  mirrorDelta[m] is the BYTE distance from the output base to
 * mirror m's base.  Plain stores only; the caller's barrier follows the launch.  With mirrorMulticast != 0
 * there is exactly one mirror and it is an NVLink multicast address bound to the result buffers of all GPUs:
 * the kernels write it with multimem.st and the switch delivers one copy to every GPU, so each device sends
 * its row block once instead of once per peer.  The reference library is single-device and has nothing of
 * the kind. */
#define ACLSP_MAX_MIRRORS 7

/* Closing barrier of a sharded product: with world > 1 the last kernel of the product ends with one node
 * barrier (see aclsp_b200_node_barrier_kernel_do below for the protocol and the state), run by the CTA that
 * finishes last, so that a step is the product kernels alone.  local: this rank's AclspNodeBarrierState;
 * peers[r]: rank r's state as this device addresses it (entry `rank` unused); spinLimit: polls per peer
 * before the wait is given up and local->status is set.  Zero-filled: no barrier. */
#define ACLSP_BARRIER_MAX_RANKS 16
typedef struct AclspBarrierLink {
    void* local;
    void* peers[ACLSP_BARRIER_MAX_RANKS];
    uint32_t world;
    uint32_t rank;
    uint32_t spinLimit;
    uint32_t reserved;
} AclspBarrierLink;

/* Per-launch parameters of the SpMV kernels.  Counterpart of the reference's
 * SpmvArch35TilingData (sparse/spmv/arch35/spmv_tiling_data.h:38-68), passed
 * by value as a kernel argument instead of being published to the workspace. */
typedef struct AclspSpmvParams {
    uint32_t rows;
    uint32_t cols;
    uint32_t nnz;
    uint32_t indexBase;      /* subtracted from every column index */
    int64_t colIndStride;    /* element strides of the CSR arrays and vectors */
    int64_t valuesStride;
    int64_t xStride;
    int64_t yStride;
    float alpha;             /* used when alphaPtr == NULL (host pointer mode) */
    float beta;
    const float* alphaPtr;   /* device pointer mode: scalars are read on the device */
    const float* betaPtr;
    uint32_t numMirrors;     /* 0: y only */
    uint32_t mirrorMulticast;
    int64_t mirrorDelta[ACLSP_MAX_MIRRORS];
    /* Longest row of the matrix as the preprocessing pass recorded it in the plan header, when the host
     * has learnt it (an asynchronous copy to pinned memory), else ACLSP_MAX_ROW_LEN_UNKNOWN: then both
     * SpMV kernels are launched and decide by the plan header which of them computes. */
    uint32_t maxRowLenHint;
    /* The vector that beta scales when it is not y itself (Z = alpha*A*X + beta*Y, the SpMVOp form):
     * element i at betaSource[i * betaSourceStride].  NULL: y is updated in place. */
    const float* betaSource;
    int64_t betaSourceStride;
    /* Element types (ACLSP_TYPE_*).  valueType is the type of the matrix values and of x (the reference
     * requires them equal, sparse/spmv/arch35/spmv_host.cpp:44-66), yType that of y and of betaSource.
     * Zero-filled parameters mean fp32 throughout.  With valueType != ACLSP_TYPE_F32 the pointer
     * arguments of the launcher address elements of these types, there are no mirrors, and
     * - computeInt == 0: alpha / beta are the floats above, sums are fp64, y is rounded once, to nearest even;
     * - computeInt == 1 (int8 values, int32 y): alphaInt / betaInt (device pointer mode: alphaPtr / betaPtr
     *   address int32), the sum is exact and y = alpha*sum + beta*y saturates to the int32 range
     *   (sparse/spmv/arch35/spmv_kernel.cpp:333-375). */
    uint32_t valueType;
    uint32_t yType;
    uint32_t computeInt;
    int32_t alphaInt;
    int32_t betaInt;
    AclspBarrierLink barrier; /* closing barrier of a sharded product (fp32 only); world == 0: none */
} AclspSpmvParams;

#define ACLSP_MAX_ROW_LEN_UNKNOWN 0xFFFFFFFFu

#define ACLSP_TYPE_F32 0u
#define ACLSP_TYPE_F16 1u
#define ACLSP_TYPE_BF16 2u
#define ACLSP_TYPE_I8 3u
#define ACLSP_TYPE_I32 4u

/* Per-launch parameters of the SpMM kernels.  Counterpart of the reference's
 * SpmmTilingWireV1 (sparse/spmm/arch35/spmm_tiling_wire.h:23-74). */
typedef struct AclspSpmmParams {
    uint32_t rows;           /* m: rows of A and C */
    uint32_t cols;           /* k: columns of A, rows of op(B) */
    uint32_t nnz;
    uint32_t indexBase;
    uint32_t n;              /* columns of C */
    uint32_t opB;            /* 0: B is k x n, 1: B is n x k and read transposed */
    uint32_t orderB;         /* 0 row-major, 1 column-major */
    uint32_t orderC;
    uint32_t highPrecision;  /* 1: the caller asked for FP32_HIGH_PRECISION; every algorithm sums in fp64, so unused */
    uint32_t reserved;
    int64_t ldb;
    int64_t ldc;
    float alpha;
    float beta;
    const float* alphaPtr;
    const float* betaPtr;
    uint32_t numMirrors;     /* 0: C only */
    uint32_t mirrorMulticast;
    int64_t mirrorDelta[ACLSP_MAX_MIRRORS];
    /* Element types (ACLSP_TYPE_*): valueType of the matrix values and of B (equal in every supported
     * combination, sparse/spmm/arch35/host/spmm_host.cpp:379-387), cType of C; computeInt, alphaInt and
     * betaInt as in AclspSpmvParams.  Zero-filled: fp32 throughout.  Narrow types: no mirrors. */
    uint32_t valueType;
    uint32_t cType;
    uint32_t computeInt;
    int32_t alphaInt;
    int32_t betaInt;
    AclspBarrierLink barrier; /* closing barrier of a sharded product (fp32 only); world == 0: none */
} AclspSpmmParams;

/* Builds the SpMV plan in `workspace`: header, base-0 row offsets, merge-path
 * tile splits and per-tile row bins.  Replaces spmv_arch35_preprocess_kernel_do
 * (reference: sparse/spmv/arch35/spmv_kernel.h:10-17, spmv_kernel.cpp:1165-1171),
 * which only normalises the row offsets on one core. */
void spmv_b200_preprocess_kernel_do(const void* rowPtr, void* workspace, uint32_t rows, uint32_t cols,
                                    uint32_t nnz, int32_t indexBase, int64_t rowOffsetsStride, void* stream);

/* y = alpha * A * x + beta * y over the plan in `workspace`.  Replaces
 * spmv_arch35_kernel_do (reference: sparse/spmv/arch35/spmv_kernel.cpp:1173-1184). */
void spmv_b200_kernel_do(const void* colInd, const void* values, const void* x, void* y, void* workspace,
                         const AclspSpmvParams* params, void* stream);

/* Builds the SpMM plan in `workspace`.  Replaces the host-side row reorder of
 * the reference (sparse/spmm/arch35/host/spmm_csr_mat.cpp:180-210), which
 * copies the row offsets to the host, sorts and copies a permutation back. */
void spmm_b200_preprocess_kernel_do(const void* rowPtr, void* workspace, uint32_t rows, uint32_t cols,
                                    uint32_t nnz, uint32_t denseCols, int32_t indexBase, void* stream);

/* C = alpha * A * op(B) + beta * C over the plan in `workspace`.  Replaces
 * spmm_kernel_launch (reference: sparse/spmm/arch35/kernel/spmm_kernel.h:18-31,
 * spmm_kernel.cpp:265-309). */
void spmm_b200_kernel_do(const void* colInd, const void* values, const void* b, void* c, void* workspace,
                         const AclspSpmmParams* params, void* stream);

/* Row-block boundaries that split the non-zeros evenly over `parts` devices:
 * bounds[g] = min{ r : rowPtr[r] - base >= ceil(g * nnz / parts) }, g = 0..parts.
 * `bounds` is a device array of parts+1 int32.  No counterpart in the
 * reference, which is single-device. */
void aclsp_b200_row_block_bounds_kernel_do(const void* rowPtr, uint32_t rows, uint32_t nnz, int32_t indexBase,
                                           uint32_t parts, void* bounds, void* stream);

/* Copies `countElems` floats at element `offsetElems` of `src` to the same place in each of the
 * `numPeers` buffers (16 per launch; a peer buffer aligned differently from `src` gets 4-byte stores) of the host array `peers` - peer-mapped device pointers of the other
 * ranks' result buffers - with plain stores, all peers in one launch.  The caller supplies the barrier
 * that follows.  No counterpart in the reference, which is single-device. */
void aclsp_b200_push_slice_kernel_do(const void* src, void* const* peers, uint32_t numPeers, int64_t offsetElems,
                                     int64_t countElems, void* stream);

/* op(A) = transpose.  Builds the transpose of the CSR matrix in `workspace` as a CSR matrix of its own:
 * row offsets at the place where a plan keeps them (so that the preprocess launcher above can then be run
 * on them in place), column indices (the original row numbers, ascending inside a row), and the
 * permutation perm[p] = original index of transposed entry p; entries of one column keep their original
 * order (a stable counting sort), so the result does not depend on scheduling.  `layout` is a host
 * pointer to the offsets (AclspTransposeLayout, csrc/plan_layout.h).  Replaces the reference's host-built
 * CSC copy (sparse/spmm/arch35/host/spmm_csr_mat.cpp:212-315) and stands in for its transposed SpMV
 * kernels (sparse/spmv/arch35/spmv_kernel.cpp:579-879). */
struct AclspTransposeLayout;
void aclsp_b200_transpose_build_kernel_do(const void* rowPtr, const void* colInd, uint32_t rows, uint32_t cols,
                                          uint32_t nnz, int32_t indexBase, int64_t rowPtrStride,
                                          int64_t colIndStride, void* workspace,
                                          const struct AclspTransposeLayout* layout, void* stream);

/* valuesT[p] = values[perm[p] * valuesStride] into the workspace of a transpose built by the call above
 * (the per-product part of op(A) = transpose); elements of elemBytes (1, 2 or 4) bytes.  Replaces
 * spmm_transpose_values_launch (reference: sparse/spmm/arch35/kernel/spmm_kernel_transpose.cpp:62). */
void aclsp_b200_transpose_values_kernel_do(const void* values, int64_t valuesStride, uint32_t cols, uint32_t nnz,
                                           void* workspace, const struct AclspTransposeLayout* layout,
                                           uint32_t elemBytes, void* stream);

/* Number of kernels this library has launched in this process so far (all entry points, all streams;
 * launches recorded into a CUDA graph count once, at capture).  A diagnostic for benchmarks. */
uint64_t aclsp_b200_kernel_launches(void);

/* State of the node barrier, one per rank, in memory that every rank of the node can address (peer-mapped /
 * symmetric memory), zero-filled before the first barrier.  epoch: barriers this rank has entered.
 * status: 0, or 1 + the rank that did not arrive within the limit of some barrier since the host last
 * looked.  flag[r]: the epoch rank r has announced to this rank. */
typedef struct AclspNodeBarrierState {
    uint32_t epoch;
    uint32_t status;
    uint32_t reserved[2];    /* [0]: CTA tickets of a closing barrier, zero between kernels */
    uint32_t flag[ACLSP_BARRIER_MAX_RANKS];
} AclspNodeBarrierState;

/* One barrier across `world` (2..16) ranks: announces this rank's next epoch in every peer's state, then
 * waits, at most `spinLimit` polls per peer (a poll is a fraction of a microsecond), until every peer has
 * announced it too; a wait that runs out sets localState->status and the kernel returns.  peerStates is a
 * host array of `world` device pointers, entry r being rank r's state as this device addresses it (entry
 * `rank` is unused).  One warp, one launch.  No counterpart in the reference, which is single-device. */
void aclsp_b200_node_barrier_kernel_do(void* localState, void* const* peerStates, uint32_t world, uint32_t rank,
                                       uint32_t spinLimit, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif

#endif /* ACLSPARSE_B200_KERNELS_H_ */
