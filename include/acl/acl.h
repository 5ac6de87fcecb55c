/* Callers written against CANN include <acl/acl.h>; on B200 everything the
 * sparse path needs from it lives in acl_base_rt.h. */
#ifndef ACLSPARSE_B200_ACL_H_
#define ACLSPARSE_B200_ACL_H_
#include "acl_base_rt.h"
#endif
