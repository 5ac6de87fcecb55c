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

/* Row-block boundaries that balance the non-zeros of a CSR matrix over `parts`
 * devices.  Writes parts+1 int32 values to the DEVICE array `bounds`
 * (asynchronously, on the handle's stream):
 *     bounds[g] = min{ r : rowOffsets[r] - base >= ceil(g * nnz / parts) },  bounds[parts] = rows.
 * Device g then owns rows [bounds[g], bounds[g+1]); x (or B) is replicated and
 * y (or C) is reassembled by an all-gather.  Needs int32 row offsets with unit
 * stride.  No counterpart in the reference. */
aclsparseStatus_t aclsparseB200RowBlockBounds(aclsparseHandle_t handle, aclsparseConstSpMatDescr_t matA, int parts,
                                              void* bounds);

#ifdef __cplusplus
}
#endif

#endif /* ACLSPARSE_B200_EXT_H_ */
