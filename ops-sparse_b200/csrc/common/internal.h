// Host-side object model behind the opaque aclsparse handles.
//
// Role of each struct matches the reference's internal headers
// (sparse/common/aclsparse_handle_internal.h:56-100, aclsparse_descr_internal.h:32-56,
// 102-128); field sets are trimmed to what the CSR SpMV / SpMM path uses and extended
// with the analysis-plan bookkeeping the B200 kernels need.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include <cuda_runtime_api.h>

#include "cann_ops_sparse.h"
#include "b200sp_kernels.h"

namespace b200sp {

constexpr size_t kDefaultWorkspaceBytes = 4u << 20;  // reference: ACLSPARSE_DEFAULT_WORKSPACE_SIZE, 4 MiB
constexpr int kLibraryVersion = 10000;               // reference: ACLSPARSE_VERSION
constexpr uint32_t kDnVecMagic = 0xD0D2D4D6u;        // reference: kDnVecSignature, aclsparse_descr.cpp:29

// Log level from the environment (B200SP_LOG_LEVEL = 0 silent, 1 errors [default], 2 info).
int LogLevel();

#define B200SP_LOGE(...)                                   \
    do {                                                   \
        if (::b200sp::LogLevel() >= 1) {                   \
            std::fprintf(stderr, "[aclsparse][E] ");       \
            std::fprintf(stderr, __VA_ARGS__);             \
            std::fprintf(stderr, "\n");                    \
        }                                                  \
    } while (0)

#define B200SP_LOGI(...)                                   \
    do {                                                   \
        if (::b200sp::LogLevel() >= 2) {                   \
            std::fprintf(stderr, "[aclsparse][I] ");       \
            std::fprintf(stderr, __VA_ARGS__);             \
            std::fprintf(stderr, "\n");                    \
        }                                                  \
    } while (0)

// Which analysis currently lives in a caller-provided buffer.
enum class PlanKind : int32_t { kNone = 0, kSpmv = 1, kSpmm = 2 };

// Host mirror of "this buffer holds a valid analysis of this matrix".  The reference keeps
// only the buffer pointer (activeBuffer); the extra fields let a compute call detect that
// the matrix was re-pointed or resized after Preprocess and fall back to a fresh analysis.
struct ActivePlan {
    const void *buffer = nullptr;
    PlanKind kind = PlanKind::kNone;
    const void *rowPtr = nullptr;
    int64_t rows = 0;
    int64_t nnz = 0;
    int64_t n = 0;         // SpMM only: dense column count the partial-sum area was sized for
    int32_t segments = 0;  // SpMM only: long-row segments found by the analysis
    int32_t blockUnits = 0;  // SpMM only: units of the column-block path for the long rows (0 = summed by segments)
    int32_t longRows = 0;   // SpMM only: rows listed as long
    const void *colInd = nullptr;  // SpMM with column blocks: the cut table was made from these column indices
    int32_t valueType = -1;        // ... and for B rows of this element type
    int32_t spmvInfo[B200SP_SPMV_PLAN_INFO_INTS] = {};  // SpMV only: plan_info written by b200sp_spmv_analyze
    uint64_t generation = 0;  // BufferGeneration(buffer) when the analysis was written
};

// Every library call that writes an analysis or scratch data into a caller buffer stamps that buffer with a new
// generation; a recorded plan is valid only while its generation is still the buffer's current one.  Without it
// a stale plan would be trusted after its bytes were overwritten: Preprocess(A, buf), then a call that re-analyses
// into buf for another operation or another matrix, then a compute call on A with buf.
uint64_t NoteBufferWrite(const void *buffer);   // returns the new generation (never 0)
uint64_t BufferGeneration(const void *buffer);  // 0 = no library call has written this buffer

}  // namespace b200sp

struct aclsparseContext {
    cudaStream_t stream = nullptr;
    aclsparsePointerMode_t pointerMode = ACL_SPARSE_POINTER_MODE_HOST;
    void *ownedWorkspace = nullptr;  // allocated by aclsparseCreate, freed by aclsparseDestroy
    size_t ownedWorkspaceBytes = 0;
    void *userWorkspace = nullptr;   // borrowed
    size_t userWorkspaceBytes = 0;
    bool userWorkspaceActive = false;
    int device = 0;

    void *Workspace() const { return userWorkspaceActive ? userWorkspace : ownedWorkspace; }
    size_t WorkspaceBytes() const { return userWorkspaceActive ? userWorkspaceBytes : ownedWorkspaceBytes; }
};

struct aclsparseSpMatDescr {
    aclsparseFormat_t format = ACL_SPARSE_FORMAT_CSR;
    int64_t rows = 0;
    int64_t cols = 0;
    int64_t nnz = 0;
    void *offsets = nullptr;  // CSR: row offsets
    void *indices = nullptr;  // CSR: column indices
    void *values = nullptr;
    aclsparseIndexType_t offsetType = ACL_SPARSE_INDEX_32I;
    aclsparseIndexType_t indexType = ACL_SPARSE_INDEX_32I;
    aclsparseIndexBase_t base = ACL_SPARSE_INDEX_BASE_ZERO;
    aclDataType valueType = ACL_FLOAT;
    // Written by *Preprocess through a const descriptor, as in the reference
    // (spmm_host.cpp:341,360): the compute call compares its buffer argument against it.
    mutable b200sp::ActivePlan active;
};

struct aclsparseDnVecDescr {
    uint32_t magic = 0;
    int64_t size = 0;
    void *values = nullptr;
    aclDataType valueType = ACL_FLOAT;
};

struct aclsparseDnMatDescr {
    int64_t rows = 0;
    int64_t cols = 0;
    int64_t ld = 0;
    aclsparseOrder_t order = ACL_SPARSE_ORDER_ROW;
    void *values = nullptr;
    aclDataType valueType = ACL_FLOAT;
};

namespace b200sp {

// True for the value types the reference's descriptor constructors accept
// (IsValidSparseValueType, aclsparse_descr.cpp:42-67).
bool IsDescriptorValueType(aclDataType t);

// Execute-path index rule: only (32I, 32I) (AclsparseValidateSupportedCsrIndexTypes,
// aclsparse_descr_internal.h:72-83).
inline aclsparseStatus_t CheckExecIndexTypes(aclsparseIndexType_t offsets, aclsparseIndexType_t indices)
{
    if (offsets != indices || offsets != ACL_SPARSE_INDEX_32I) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    return ACL_SPARSE_STATUS_SUCCESS;
}

// Maps an ACL data type to the kernel-side type id; returns -1 for types the kernels do not take.
inline int KernelTypeOf(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT: return B200SP_F32;
        case ACL_FLOAT16: return B200SP_F16;
        case ACL_BF16: return B200SP_BF16;
        case ACL_INT32: return B200SP_I32;
        case ACL_INT8: return B200SP_I8;
        default: return -1;
    }
}

}  // namespace b200sp
