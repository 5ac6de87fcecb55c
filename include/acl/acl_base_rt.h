/*
 * Stand-in for the two CANN runtime headers the aclsparse API pulls in
 * (<acl/acl_base_rt.h> and <acl/acl.h>), reduced to what the CSR SpMV / SpMM
 * path needs and re-targeted at the CUDA runtime.
 *
 * The sparse library only uses three things from the platform header set:
 * the element-type enum `aclDataType`, the opaque stream type `aclrtStream`
 * and the error code type `aclError`.  On B200 a stream is a `cudaStream_t`;
 * both are pointer-sized opaque handles, so the typedef below keeps every
 * prototype of the public header source compatible.
 *
 * The numeric values of `aclDataType` follow the public CANN enumeration.
 * The sparse host code never depends on the numbers (it switches on the
 * enumerator names), so a caller that is recompiled against this header is
 * unaffected by the exact values.
 */
#ifndef ACLSPARSE_B200_ACL_BASE_RT_H_
#define ACLSPARSE_B200_ACL_BASE_RT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int aclError;
#define ACL_SUCCESS 0
#define ACL_ERROR_NONE 0

/* A CUDA stream (cudaStream_t) passed through the ACL-shaped API. */
typedef void* aclrtStream;

typedef enum {
    ACL_DT_UNDEFINED = -1,
    ACL_FLOAT = 0,
    ACL_FLOAT16 = 1,
    ACL_INT8 = 2,
    ACL_INT32 = 3,
    ACL_UINT8 = 4,
    ACL_INT16 = 6,
    ACL_UINT16 = 7,
    ACL_UINT32 = 8,
    ACL_INT64 = 9,
    ACL_UINT64 = 10,
    ACL_DOUBLE = 11,
    ACL_BOOL = 12,
    ACL_STRING = 13,
    ACL_COMPLEX64 = 16,
    ACL_COMPLEX128 = 17,
    ACL_BF16 = 27,
    ACL_INT4 = 29,
    ACL_UINT1 = 30,
    ACL_COMPLEX32 = 33,
    ACL_HIFLOAT8 = 34,
    ACL_FLOAT8_E5M2 = 35,
    ACL_FLOAT8_E4M3FN = 36,
    ACL_FLOAT8_E8M0 = 37,
    ACL_FLOAT6_E3M2 = 38,
    ACL_FLOAT6_E2M3 = 39,
    ACL_FLOAT4_E2M1 = 40,
    ACL_FLOAT4_E1M2 = 41
} aclDataType;

#ifdef __cplusplus
}
#endif

#endif /* ACLSPARSE_B200_ACL_BASE_RT_H_ */
