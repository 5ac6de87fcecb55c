/*
 * Library handle: stream, scalar pointer mode and the library / user workspace.
 * Behaviour follows the reference's sparse/common/aclsparse_auxiliary.cpp:103-330.
 */
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <new>

#include <cuda_runtime.h>

#include "internal.h"

namespace {

// NULL -> HANDLE_IS_NULLPTR, wrong signature -> INVALID_VALUE
// (reference: aclsparse_auxiliary.cpp:37-48).
aclsparseStatus_t CheckedHandle(aclsparseHandle_t handle, aclsparseContext** out)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (handle->signature != kHandleSignature) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *out = handle;
    return ACL_SPARSE_STATUS_SUCCESS;
}

void FreeDefaultWorkspace(aclsparseContext* h)
{
    if (h->defaultWorkspace == nullptr) {
        return;
    }
    int current = -1;
    const bool switched = cudaGetDevice(&current) == cudaSuccess && h->device >= 0 && current != h->device;
    if (switched) {
        cudaSetDevice(h->device);
    }
    cudaFree(h->defaultWorkspace);
    if (switched) {
        cudaSetDevice(current);
    }
    h->defaultWorkspace = nullptr;
    h->defaultWorkspaceSize = 0;
}

}  // namespace

int AclspLogLevel()
{
    static const int level = [] {
        const char* env = std::getenv("ACLSPARSE_LOG_LEVEL");
        return env == nullptr ? 0 : std::atoi(env);
    }();
    return level;
}

void AclspLog(int level, const char* api, const char* fmt, ...)
{
    static const char* const kNames[] = {"", "ERROR", "INFO", "DEBUG"};
    std::fprintf(stderr, "[aclsparse][%s][%s] ", kNames[level < 1 ? 1 : (level > 3 ? 3 : level)], api);
    va_list args;
    va_start(args, fmt);
    std::vfprintf(stderr, fmt, args);
    va_end(args);
    std::fputc('\n', stderr);
}

uint32_t AclspSmCount()
{
    int device = 0;
    int count = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return count > 0 ? static_cast<uint32_t>(count) : 0u;
}

extern "C" {

aclsparseStatus_t aclsparseCreate(aclsparseHandle_t* handle)
{
    if (handle == nullptr) {
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    // A non-NULL *handle is taken for a live handle: overwriting it would leak.
    if (*handle != nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    auto* h = new (std::nothrow) aclsparseContext();
    if (h == nullptr) {
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    *handle = h;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDestroy(aclsparseHandle_t handle)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    // Work enqueued through this handle may still reference its workspace.
    if (h->stream != nullptr) {
        cudaStreamSynchronize(static_cast<cudaStream_t>(h->stream));
    }
    FreeDefaultWorkspace(h);
    h->userWorkspace = nullptr;
    h->userWorkspaceSize = 0;
    h->useUserWorkspace = false;
    h->stream = nullptr;
    h->signature = 0;
    delete h;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSetStream(aclsparseHandle_t handle, aclrtStream stream)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (h->stream != stream) {
        ++h->streamEpoch;
        if (h->streamEpoch == 0) {
            h->streamEpoch = 1;  // never wrap back onto the initial epoch
        }
    }
    h->stream = stream;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetStream(aclsparseHandle_t handle, aclrtStream* stream)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (stream == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *stream = h->stream;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSetWorkspace(aclsparseHandle_t handle, void* workspace, size_t workspaceSize)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (workspace == nullptr) {  // back to the library-owned workspace
        h->userWorkspace = nullptr;
        h->userWorkspaceSize = 0;
        h->useUserWorkspace = false;
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (workspaceSize == 0) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    // Grow-only: a buffer no larger than the current user workspace is ignored.
    if (h->useUserWorkspace && workspaceSize <= h->userWorkspaceSize) {
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    h->userWorkspace = workspace;
    h->userWorkspaceSize = workspaceSize;
    h->useUserWorkspace = true;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetWorkspace(aclsparseHandle_t handle, void** workspace, size_t* workspaceSize)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (workspace == nullptr || workspaceSize == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (h->useUserWorkspace) {
        *workspace = h->userWorkspace;
        *workspaceSize = h->userWorkspaceSize;
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (h->defaultWorkspace == nullptr) {
        void* ptr = nullptr;
        if (cudaMalloc(&ptr, kDefaultWorkspaceBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return ACL_SPARSE_STATUS_ALLOC_FAILED;
        }
        h->defaultWorkspace = ptr;
        h->defaultWorkspaceSize = kDefaultWorkspaceBytes;
        (void)cudaGetDevice(&h->device);
    }
    *workspace = h->defaultWorkspace;
    *workspaceSize = h->defaultWorkspaceSize;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetVersion(aclsparseHandle_t handle, int* version)
{
    (void)handle;  // may be NULL
    if (version == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *version = kAclsparseVersion;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t mode)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (mode != ACL_SPARSE_POINTER_MODE_HOST && mode != ACL_SPARSE_POINTER_MODE_DEVICE) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    h->pointerMode = mode;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t* mode)
{
    aclsparseContext* h = nullptr;
    const aclsparseStatus_t st = CheckedHandle(handle, &h);
    if (st != ACL_SPARSE_STATUS_SUCCESS) {
        return st;
    }
    if (mode == nullptr) {
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    *mode = h->pointerMode;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
