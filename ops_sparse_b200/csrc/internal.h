/*
 * Private definitions behind the opaque aclsparse handle and descriptors.
 * Follows the reference's host runtime (sparse/common/aclsparse_handle_internal.h:65-86,
 * sparse/common/aclsparse_descr_internal.h:242-311,437-468) for the fields the
 * CSR SpMV / SpMM path uses; nothing here is visible to callers.
 */
#ifndef ACLSPARSE_B200_INTERNAL_H_
#define ACLSPARSE_B200_INTERNAL_H_

#include <cstddef>
#include <cstdint>

#include "aclsparse_b200_kernels.h"
#include "cann_ops_sparse.h"

// Every opaque object starts with a signature word that is checked before any
// other field is read and cleared before the object is freed, so that stale or
// foreign pointers fail with a status instead of being dereferenced further.
constexpr uint32_t kHandleSignature = 0xAC1F9501u;
constexpr uint32_t kSpMatSignature = 0x53504D54u;
constexpr uint32_t kDnVecSignature = 0xD0D2D4D6u;
constexpr uint32_t kDnMatSignature = 0xD0D2D4D8u;

constexpr int kAclsparseVersion = 1 * 10000 + 0 * 100 + 0;
constexpr size_t kDefaultWorkspaceBytes = 4u * 1024u * 1024u;
constexpr int kMaxStridedBatchCount = 65535;

struct aclsparseContext {
    uint32_t signature = kHandleSignature;
    aclrtStream stream = nullptr;
    // Bumped whenever the stream changes: preprocessing is enqueued on a
    // stream, so metadata built under an older epoch is not reused.
    uint64_t streamEpoch = 0;
    aclsparsePointerMode_t pointerMode = ACL_SPARSE_POINTER_MODE_HOST;
    int device = -1;  // device of the lazily allocated default workspace
    void* defaultWorkspace = nullptr;
    size_t defaultWorkspaceSize = 0;
    void* userWorkspace = nullptr;
    size_t userWorkspaceSize = 0;
    bool useUserWorkspace = false;
};

// A word of pinned host memory that a value from the device arrives in (host_flags.cpp).
struct AclspHostSlot {
    uint32_t* word = nullptr;
    uint32_t index = 0;
    uint64_t generation = 0;
};
AclspHostSlot AclspAcquireHostSlot();
// True, and the value, once the device's copy has arrived and the slot still belongs to its holder.
bool AclspHostSlotValue(const AclspHostSlot& slot, uint32_t* value);

// What the most recent SpMV preprocessing of a matrix was built from.  The
// buffer is reused by aclsparseSpMV only while every field still matches
// (reference: sparse/spmv/arch35/spmv.h:47-107).
struct SpmvPlanRecord {
    const void* buffer = nullptr;
    const void* rowOffsets = nullptr;
    const void* colIndices = nullptr;
    const void* values = nullptr;
    int64_t rowOffsetsStride = 1;
    int64_t colIndStride = 1;
    int64_t valuesStride = 1;
    int64_t xStride = 1;
    int64_t yStride = 1;
    uint64_t rows = 0;
    uint64_t cols = 0;
    uint64_t nnz = 0;
    aclsparseIndexBase_t base = ACL_SPARSE_INDEX_BASE_ZERO;
    aclDataType valueType = ACL_FLOAT;
    aclDataType xType = ACL_FLOAT;
    aclDataType yType = ACL_FLOAT;
    aclDataType computeType = ACL_FLOAT;
    aclsparseOperation_t op = ACL_SPARSE_OP_NON_TRANSPOSE;
    int32_t alg = -1;
    const void* stream = nullptr;
    uint64_t streamEpoch = 0;
    uint64_t serial = 0;          // AclspPublishPlan's answer for this build; 0: no plan
    bool fromPreprocess = false;  // built by an explicit Preprocess call: only such a plan is reused
    AclspHostSlot longestRow;     // where the plan's longest row arrives on the host
};

// SpMM preprocessing depends on the structure of A and on the width of C only.
// B, C, alpha and beta are per-launch kernel arguments, so rebinding them does
// not invalidate the plan (the reference keys its cache on them as well,
// sparse/spmm/arch35/host/spmm_host.cpp:63-97, and pays a host rebuild).
struct SpmmPlanRecord {
    const void* buffer = nullptr;
    bool transposed = false;            // the buffer holds the plan of the transpose, and the transpose
    const void* colIndices = nullptr;   // what that transpose was built from
    const void* rowOffsets = nullptr;
    uint64_t rows = 0;
    uint64_t cols = 0;
    uint64_t nnz = 0;
    uint64_t denseCols = 0;
    aclsparseIndexBase_t base = ACL_SPARSE_INDEX_BASE_ZERO;
    const void* stream = nullptr;
    uint64_t streamEpoch = 0;
    uint64_t ownerId = 0;
    uint64_t serial = 0;
    bool fromPreprocess = false;
};

struct aclsparseSpMatDescr {
    uint32_t signature = kSpMatSignature;
    aclsparseFormat_t format = ACL_SPARSE_FORMAT_CSR;
    uint64_t rows = 0;
    uint64_t cols = 0;
    uint64_t nnz = 0;
    void* ptrs = nullptr;    // CSR row offsets
    void* idxs = nullptr;    // CSR column indices
    void* values = nullptr;
    int64_t ptrStride = 1;
    int64_t idxStride = 1;
    int64_t valueStride = 1;
    aclsparseIndexBase_t baseType = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseIndexType_t ptrType = ACL_SPARSE_INDEX_32I;
    aclsparseIndexType_t idxType = ACL_SPARSE_INDEX_32I;
    aclDataType valueType = ACL_FLOAT;
    // Identity that tells two descriptors at a recycled address apart when
    // they share one workspace (reference: aclsparse_descr.cpp:31-35).
    uint64_t workspaceOwnerId = 0;
    uint64_t structureGeneration = 1;
    // `activeBuffer` is the buffer that currently holds SpMM metadata of this
    // matrix, `spmv.buffer` the one that holds SpMV metadata; the two
    // operators use different layouts and invalidate each other when they are
    // handed the same allocation.
    const void* activeBuffer = nullptr;
    SpmvPlanRecord spmv;
    SpmmPlanRecord spmm;
};

struct aclsparseDnVecDescr {
    uint32_t signature = 0;
    uint64_t nums = 0;
    void* values = nullptr;
    int64_t stride = 1;
    aclDataType valueType = ACL_FLOAT;
    // aclsparseB200DnVecSetMirrors: further buffers that receive every element SpMV writes.
    int numMirrors = 0;
    bool mirrorMulticast = false;
    void* mirrors[7] = {};
    // aclsparseB200DnVecSetClosingBarrier: the node barrier that ends a product into this vector.
    AclspBarrierLink barrier = {};
};

struct aclsparseDnMatDescr {
    uint32_t signature = 0;
    int64_t rows = 0;
    int64_t cols = 0;
    int64_t ld = 0;
    aclsparseOrder_t order = ACL_SPARSE_ORDER_ROW;
    void* values = nullptr;
    aclDataType valueType = ACL_FLOAT;
    int32_t batchCount = 1;
    int64_t batchStride = 0;
    // aclsparseB200DnMatSetMirrors: further buffers that receive every element SpMM writes.
    int numMirrors = 0;
    bool mirrorMulticast = false;
    void* mirrors[7] = {};
    // aclsparseB200DnMatSetClosingBarrier: the node barrier that ends a product into this matrix.
    AclspBarrierLink barrier = {};
};

uint64_t AclspNextWorkspaceOwnerId();

// Plan ownership of workspace buffers (plan_registry.cpp).  AclspPublishPlan records that `buffer` now
// holds a freshly built plan and returns its serial number; AclspPlanIsCurrent says whether the plan
// with that serial is still the last one built in `buffer`.
uint64_t AclspPublishPlan(const void* buffer);
bool AclspPlanIsCurrent(const void* buffer, uint64_t serial);
void AclspResetSpmvPlan(aclsparseSpMatDescr* descr);

// Logging: ACLSPARSE_LOG_LEVEL=0 (off, default) / 1 (errors) / 2 (info) / 3 (debug) -> stderr.
int AclspLogLevel();
void AclspLog(int level, const char* api, const char* fmt, ...) __attribute__((format(printf, 3, 4)));
#define ACLSP_LOGE(api, ...) do { if (AclspLogLevel() >= 1) AclspLog(1, api, __VA_ARGS__); } while (0)
#define ACLSP_LOGI(api, ...) do { if (AclspLogLevel() >= 2) AclspLog(2, api, __VA_ARGS__); } while (0)
#define ACLSP_LOGD(api, ...) do { if (AclspLogLevel() >= 3) AclspLog(3, api, __VA_ARGS__); } while (0)

// Number of streaming multiprocessors of the current device (0 when no device
// can be queried).  Takes the place of the reference's AIV core count.
uint32_t AclspSmCount();

#endif  // ACLSPARSE_B200_INTERNAL_H_
