/*
 * B200 additions to the aclsparse API.  The reference library drives one
 * device through one stream and has no multi-device code, so the entry points
 * in this header have no counterpart there; they carry the one piece of the
 * multi-GPU path that has to run where the matrix lives.
 */
#ifndef ACLSPARSE_B200_EXT_H_
#define ACLSPARSE_B200_EXT_H_

#include "cann_ops_sparse.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility: only what this header declares is exported. */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Row-block boundaries that balance the non-zeros of a CSR matrix over `parts`
 * devices.  Writes parts+1 int32 values to the DEVICE array `bounds`
 * (asynchronously, on the handle's stream):
 *     bounds[g] = min{ r : rowOffsets[r] - base >= ceil(g * nnz / parts) },  bounds[parts] = rows.
 * Device g then owns rows [bounds[g], bounds[g+1]); x (or B) is replicated and
 * y (or C) is reassembled by an all-gather.  Needs int32 row offsets with unit
 * stride.  No counterpart in the reference. */
aclsparseStatus_t aclsparseB200RowBlockBounds(aclsparseHandle_t handle, aclsparseConstSpMatDescr_t matA, int parts,
                                              void* bounds);

/* y = alpha * A * x + beta * y for a CSR matrix (int32 indices, fp32 data, unit strides, host scalars)
 * WITHOUT an external buffer and without allocating anything: the plan and the per-tile carries that
 * aclsparseSpMV keeps in the caller's buffer live in an 8 MiB device array built into the library.
 * For callers that cannot allocate device memory when they need the product - a latency-critical loop
 * whose memory was fixed at start-up, a host framework whose allocator owns the device, a plug-in that
 * is only handed its operands.  Asynchronous on `stream`.
 *   - Matrices whose plan exceeds the built-in scratch (roughly rows * 4 + (rows + nnz) * 0.012 bytes
 *     > 8 MiB) are refused with ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES and a message on stderr.
 *   - The first call on a device loads the library's device code (with it the scratch array) and looks up
 *     the scratch's device address: that call can take device memory once and must be made at start-up,
 *     outside any stream capture.  Every later call on that device allocates nothing.
 *   - All calls on a device share the scratch: calls that overlap on the GPU race; keep them in stream order.
 * This entry point has no counterpart in the reference. */
aclsparseStatus_t aclsparseB200SpMVNoAlloc(aclrtStream stream, int64_t rows, int64_t cols, int64_t nnz,
                                           const int32_t* rowOffsets, const int32_t* colInd, const float* values,
                                           aclsparseIndexBase_t idxBase, const float* x, float* y, float alpha,
                                           float beta);

/* Mirrors of an output vector / matrix: after this call every element that aclsparseSpMV (aclsparseSpMM)
 * writes to `vec` (`mat`) is also stored at the same element position of each of the `count` (at most 7)
 * buffers `mirrors[0..count)`, by the product kernels themselves.  With the result buffers of the other
 * GPUs of the node as mirrors (peer-mapped pointers, each advanced to this device's row block) the product
 * and the reassembly of a row-block-sharded y / C over NVLink become one kernel; the caller follows it with
 * a barrier across the devices.  A mirror has the layout (stride, leading dimension, order) of the vector
 * or matrix itself.  count == 0 clears the list.  The host array `mirrors` is copied.  beta scales the
 * values of `vec` / `mat` only; mirrors are never read.  No counterpart in the reference. */
aclsparseStatus_t aclsparseB200DnVecSetMirrors(aclsparseDnVecDescr_t vec, int count, void* const* mirrors);
aclsparseStatus_t aclsparseB200DnMatSetMirrors(aclsparseDnMatDescr_t mat, int count, void* const* mirrors);

/* The same with ONE mirror that is an NVLink multicast address (a cuMulticast / symmetric-memory mapping
 * bound to the result buffers of all GPUs of the node, advanced to this device's row block): the kernels
 * store to it with multimem.st, NVSwitch replicates each store to every GPU, and a device sends its block
 * once instead of once per peer.  Replaces any mirror list; SetMirrors(.., 0, NULL) clears it.  Only on
 * devices and buffers for which such a mapping exists.  No counterpart in the reference. */
aclsparseStatus_t aclsparseB200DnVecSetMulticastMirror(aclsparseDnVecDescr_t vec, void* multicast);
aclsparseStatus_t aclsparseB200DnMatSetMulticastMirror(aclsparseDnMatDescr_t mat, void* multicast);

/* Barrier across the GPUs of a node that share a row-block-sharded result: enqueues, on `stream`, one
 * small kernel that tells every peer "my row block is in your buffer" and waits until every peer has said
 * the same.  `localState` is this rank's AclspNodeBarrierState (aclsparse_b200_kernels.h; 128 bytes of
 * zero-filled memory that all ranks can address), `peerStates[r]` rank r's as this device addresses it.
 * The wait is bounded by `spinLimit` polls per peer (0 picks the default, about a second): a peer that
 * never arrives makes the kernel give up and record it, nothing hangs and nothing traps.
 * aclsparseB200NodeBarrierStatus synchronises `stream`, reads that record and clears it: it returns
 * ACL_SPARSE_STATUS_EXECUTION_FAILED when a barrier since the last call gave up (and, if `missingRank` is
 * non-null, stores the rank that was missing), ACL_SPARSE_STATUS_SUCCESS otherwise.
 * No counterpart in the reference, which is single-device. */
aclsparseStatus_t aclsparseB200NodeBarrier(aclrtStream stream, void* localState, void* const* peerStates, int world,
                                           int rank, unsigned spinLimit);
aclsparseStatus_t aclsparseB200NodeBarrierStatus(aclrtStream stream, void* localState, int* missingRank);

/* How many warps of SpMV products over the plan in `externalBuffer` gave up waiting for a bulk copy since the
 * plan was built (the SpMV row-block kernel waits for its copies at most about a quarter of a second each; a
 * warp whose wait runs out computes its remaining rows with plain loads, so the results are right either way,
 * and counts itself here).  Synchronises `stream` and reads the counter from the plan header.  A diagnostic:
 * anything but 0 means the copy engine did not deliver in time.  No counterpart in the reference. */
aclsparseStatus_t aclsparseB200SpMVWaitFailures(aclrtStream stream, const void* externalBuffer, unsigned* count);

/* The same barrier as the END of every product written into `vec` / `mat`, instead of a kernel of its own:
 * the last kernel of aclsparseSpMV / aclsparseSpMM (fp32) runs it in the CTA that finishes last, after
 * that CTA has seen all others fence their stores, so a sharded step is the product kernels alone.  The
 * arguments are those of aclsparseB200NodeBarrier; world <= 1 or localState == NULL removes it.  A product
 * that has nothing to launch (no rows) runs no barrier: such a rank calls aclsparseB200NodeBarrier.  The
 * wait is bounded as above and reported through aclsparseB200NodeBarrierStatus. */
aclsparseStatus_t aclsparseB200DnVecSetClosingBarrier(aclsparseDnVecDescr_t vec, void* localState,
                                                      void* const* peerStates, int world, int rank,
                                                      unsigned spinLimit);
aclsparseStatus_t aclsparseB200DnMatSetClosingBarrier(aclsparseDnMatDescr_t mat, void* localState,
                                                      void* const* peerStates, int world, int rank,
                                                      unsigned spinLimit);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif

#endif /* ACLSPARSE_B200_EXT_H_ */
