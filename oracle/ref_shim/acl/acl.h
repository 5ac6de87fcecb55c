/* TEST INFRASTRUCTURE ONLY.  See acl_base_rt.h in this directory. */
#ifndef ORACLE_REF_SHIM_ACL_H_
#define ORACLE_REF_SHIM_ACL_H_
#include "acl_base_rt.h"
#endif
