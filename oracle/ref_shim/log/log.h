/* TEST INFRASTRUCTURE ONLY.  The reference logs through CANN's dlog macros;
 * on the CPU build they expand to nothing. */
#ifndef ORACLE_REF_SHIM_LOG_H_
#define ORACLE_REF_SHIM_LOG_H_
#define OP_LOGE(...) ((void)0)
#define OP_LOGW(...) ((void)0)
#define OP_LOGI(...) ((void)0)
#define OP_LOGD(...) ((void)0)
#endif
