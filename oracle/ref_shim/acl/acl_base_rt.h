/* TEST INFRASTRUCTURE ONLY.  Minimal stand-in for CANN's <acl/acl_base_rt.h>,
 * used solely to compile a few of the reference's host-side source files on a
 * CPU so that the oracle can be checked against the reference's own code.
 * "Device" memory is host memory here: aclrtMemcpy is memcpy. */
#ifndef ORACLE_REF_SHIM_ACL_BASE_RT_H_
#define ORACLE_REF_SHIM_ACL_BASE_RT_H_
#include "../../../include/acl/acl_base_rt.h"
#include <string.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef enum {
    ACL_MEMCPY_HOST_TO_HOST = 0,
    ACL_MEMCPY_HOST_TO_DEVICE = 1,
    ACL_MEMCPY_DEVICE_TO_HOST = 2,
    ACL_MEMCPY_DEVICE_TO_DEVICE = 3
} aclrtMemcpyKind;
static inline aclError aclrtMemcpy(void* dst, size_t destMax, const void* src, size_t count, aclrtMemcpyKind kind)
{
    (void)kind;
    if (count > destMax) {
        return 1;
    }
    memcpy(dst, src, count);
    return ACL_SUCCESS;
}
static inline aclError aclrtSynchronizeStream(aclrtStream stream)
{
    (void)stream;
    return ACL_SUCCESS;
}
static inline aclError aclrtFree(void* ptr)
{
    (void)ptr;
    return ACL_SUCCESS;
}
#ifdef __cplusplus
}
#endif
#endif
