/* Internal: launcher of the plan-building kernels (plan_kernels.cu). */
#ifndef ACLSPARSE_B200_PLAN_KERNELS_H_
#define ACLSPARSE_B200_PLAN_KERNELS_H_

#include <cstdint>

#include <cuda_runtime.h>

// kind: ACLSP_KIND_SPMV or ACLSP_KIND_SPMM (plan_layout.h); denseCols is the
// width of C for SpMM and 1 for SpMV.
void AclspLaunchPlanBuild(const void* rowPtr, void* workspace, uint32_t rows, uint32_t cols, uint32_t nnz,
                          int32_t indexBase, int64_t rowOffsetsStride, uint32_t kind, uint32_t denseCols,
                          cudaStream_t stream);

// Every kernel launch of this library is counted (aclsp_b200_kernel_launches reads the total): the
// benchmark reports how many of the library's kernels make up a step.
void AclspCountLaunches(unsigned n);

#endif  // ACLSPARSE_B200_PLAN_KERNELS_H_
