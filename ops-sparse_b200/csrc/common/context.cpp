// aclsparse handle: stream, pointer mode and workspace management.
// Behaviour follows sparse/common/aclsparse_auxiliary.cpp:64-198, 253-279 of the reference;
// device memory comes from the CUDA runtime instead of aclrtMalloc.
#include <atomic>
#include <mutex>
#include <new>
#include <unordered_map>

#include "internal.h"

namespace b200sp {

int LogLevel()
{
    static const int level = [] {
        const char *s = std::getenv("B200SP_LOG_LEVEL");
        return s ? std::atoi(s) : 1;
    }();
    return level;
}


namespace {
std::mutex gGenerationMutex;
std::unordered_map<const void *, uint64_t> gGenerations;
uint64_t gNextGeneration = 0;
}  // namespace

uint64_t NoteBufferWrite(const void *buffer)
{
    if (buffer == nullptr) return 0;
    std::lock_guard<std::mutex> lock(gGenerationMutex);
    return gGenerations[buffer] = ++gNextGeneration;
}

uint64_t BufferGeneration(const void *buffer)
{
    if (buffer == nullptr) return 0;
    std::lock_guard<std::mutex> lock(gGenerationMutex);
    const auto it = gGenerations.find(buffer);
    return it == gGenerations.end() ? 0 : it->second;
}

}  // namespace b200sp

namespace {
std::atomic<unsigned long long> gKernelLaunches{0};
}

extern "C" {

unsigned long long b200sp_kernel_launches(void) { return gKernelLaunches.load(std::memory_order_relaxed); }
void b200sp_note_launches(int n) { gKernelLaunches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

aclsparseStatus_t aclsparseCreate(aclsparseHandle_t *handle)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    // An already-populated slot would leak the previous handle (aclsparse_auxiliary.cpp:71-73).
    if (*handle != nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;

    auto *ctx = new (std::nothrow) aclsparseContext();
    if (ctx == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;

    if (cudaGetDevice(&ctx->device) != cudaSuccess) {
        B200SP_LOGE("aclsparseCreate: no usable CUDA device (%s)", cudaGetErrorString(cudaGetLastError()));
        delete ctx;
        return ACL_SPARSE_STATUS_NOT_INITIALIZED;
    }
    if (cudaMalloc(&ctx->ownedWorkspace, b200sp::kDefaultWorkspaceBytes) != cudaSuccess) {
        (void)cudaGetLastError();
        delete ctx;
        return ACL_SPARSE_STATUS_ALLOC_FAILED;
    }
    ctx->ownedWorkspaceBytes = b200sp::kDefaultWorkspaceBytes;
    *handle = ctx;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDestroy(aclsparseHandle_t handle)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    // Kernels enqueued through this handle may still use its workspace: drain first
    // (aclsparse_auxiliary.cpp:101-104 does the same when a stream is set).
    (void)cudaStreamSynchronize(handle->stream);
    if (handle->ownedWorkspace != nullptr) (void)cudaFree(handle->ownedWorkspace);
    delete handle;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSetStream(aclsparseHandle_t handle, aclrtStream stream)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    handle->stream = reinterpret_cast<cudaStream_t>(stream);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetStream(aclsparseHandle_t handle, aclrtStream *stream)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (stream == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    *stream = reinterpret_cast<aclrtStream>(handle->stream);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSetWorkspace(aclsparseHandle_t handle, void *workspace, size_t workspaceSize)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (workspace == nullptr) {  // back to the built-in workspace; the user pointer is remembered
        handle->userWorkspaceActive = false;
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    if (workspaceSize == 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    // Grow-only: a request no larger than the active user workspace changes nothing
    // (aclsparse_auxiliary.cpp:164-167).
    if (handle->userWorkspaceActive && workspaceSize <= handle->userWorkspaceBytes) return ACL_SPARSE_STATUS_SUCCESS;
    handle->userWorkspace = workspace;
    handle->userWorkspaceBytes = workspaceSize;
    handle->userWorkspaceActive = true;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetWorkspace(aclsparseHandle_t handle, void **workspace, size_t *workspaceSize)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (workspace == nullptr || workspaceSize == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    *workspace = handle->Workspace();
    *workspaceSize = handle->WorkspaceBytes();
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetVersion(aclsparseHandle_t handle, int *version)
{
    (void)handle;  // not inspected by the reference either (aclsparse_auxiliary.cpp:188-196)
    if (version == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    *version = b200sp::kLibraryVersion;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t mode)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (mode != ACL_SPARSE_POINTER_MODE_HOST && mode != ACL_SPARSE_POINTER_MODE_DEVICE)
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    handle->pointerMode = mode;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseGetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t *mode)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (mode == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    *mode = handle->pointerMode;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
