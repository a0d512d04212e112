// aclsparseSpMV / SpMVGetBufferSize / SpMVPreprocess host layer.
//
// Argument checks, their order and their status codes follow the reference
// (sparse/spmv/arch22/spmv_host.cpp:121-295).  Differences, all supersets:
//   * GetBufferSize and Preprocess exist (the reference only declares them,
//     include/cann_ops_sparse.h:490-514);
//   * a NULL stream means the CUDA default stream (the reference returns INVALID_VALUE);
//   * no per-call device->host copy of row offsets and no maximum row length
//     (the reference bounds rows by its on-chip buffer size, spmv_host.cpp:86-112, 243-252);
//   * alpha / beta honour POINTER_MODE_DEVICE (the reference always dereferences on the host);
//   * an unknown value / output type is NOT_SUPPORTED instead of silently running as fp32
//     (reference spmv.h:86-102).
#include "../common/internal.h"

namespace {

using b200sp::ActivePlan;
using b200sp::PlanKind;

struct SpmvCall {
    const aclsparseSpMatDescr *A = nullptr;
    const aclsparseDnVecDescr *x = nullptr;
    aclsparseDnVecDescr *y = nullptr;
    bool trans = false;
    int compType = 0, valType = 0, outType = 0;
};

bool SupportedTriple(int comp, int val, int out)
{
    if (comp == B200SP_I32) return val == B200SP_I32 && out == B200SP_I32;
    if (comp != B200SP_F32) return false;
    switch (val) {
        case B200SP_F32: return out == B200SP_F32;
        case B200SP_F16: return out == B200SP_F32 || out == B200SP_F16;
        case B200SP_BF16: return out == B200SP_F32 || out == B200SP_BF16;
        case B200SP_I32: return out == B200SP_F32;
        default: return false;
    }
}

aclsparseStatus_t ValidateSpmv(const char *api, aclsparseHandle_t handle, aclsparseOperation_t opA,
                               aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                               aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                               SpmvCall *call)
{
    if (handle == nullptr) {
        B200SP_LOGE("%s: handle is nullptr", api);
        return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    }
    if (matA == nullptr || vecX == nullptr || vecY == nullptr) {
        B200SP_LOGE("%s: matA / vecX / vecY is nullptr", api);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (alg != ACL_SPARSE_SPMV_ALG_DEFAULT) {
        B200SP_LOGE("%s: only ACL_SPARSE_SPMV_ALG_DEFAULT is supported, got %d", api, (int)alg);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (computeType != ACL_FLOAT && computeType != ACL_INT32) {
        B200SP_LOGE("%s: unsupported computeType %d", api, (int)computeType);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (matA->format != ACL_SPARSE_FORMAT_CSR) {
        B200SP_LOGE("%s: unsupported matrix format %d", api, (int)matA->format);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (matA->base != ACL_SPARSE_INDEX_BASE_ZERO) {
        B200SP_LOGE("%s: one-based indices are not supported", api);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    const aclsparseStatus_t idx = b200sp::CheckExecIndexTypes(matA->offsetType, matA->indexType);
    if (idx != ACL_SPARSE_STATUS_SUCCESS) {
        B200SP_LOGE("%s: only 32-bit row offsets and column indices are supported", api);
        return idx;
    }
    if (opA != ACL_SPARSE_OP_NON_TRANSPOSE && opA != ACL_SPARSE_OP_TRANSPOSE) {
        B200SP_LOGE("%s: conjugate transpose is not supported", api);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (matA->offsets == nullptr || matA->indices == nullptr || matA->values == nullptr) {
        B200SP_LOGE("%s: matrix device pointers are null", api);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (vecX->values == nullptr || vecY->values == nullptr) {
        B200SP_LOGE("%s: vector device pointers are null", api);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    const bool trans = (opA == ACL_SPARSE_OP_TRANSPOSE);
    const int64_t needX = trans ? matA->rows : matA->cols;
    const int64_t needY = trans ? matA->cols : matA->rows;
    if (vecX->size < needX || vecY->size < needY) {  // ">=" rule, spmv_host.cpp:231-240
        B200SP_LOGE("%s: vecX size %lld (need %lld) / vecY size %lld (need %lld)", api, (long long)vecX->size,
                    (long long)needX, (long long)vecY->size, (long long)needY);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (matA->rows > INT32_MAX || matA->cols > INT32_MAX || matA->nnz > INT32_MAX) {
        B200SP_LOGE("%s: dimensions beyond 32-bit indexing", api);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (vecX->valueType != matA->valueType) {
        B200SP_LOGE("%s: matrix value type %d and vecX type %d must match", api, (int)matA->valueType,
                    (int)vecX->valueType);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    if (computeType == ACL_INT32 && (matA->valueType != ACL_INT32 || vecY->valueType != ACL_INT32)) {
        B200SP_LOGE("%s: computeType INT32 requires INT32 values and output", api);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    call->A = matA;
    call->x = vecX;
    call->y = vecY;
    call->trans = trans;
    call->compType = b200sp::KernelTypeOf(computeType);
    call->valType = b200sp::KernelTypeOf(matA->valueType);
    call->outType = b200sp::KernelTypeOf(vecY->valueType);
    if (!SupportedTriple(call->compType, call->valType, call->outType)) {
        B200SP_LOGE("%s: unsupported (compute, value, output) types (%d, %d, %d)", api, (int)computeType,
                    (int)matA->valueType, (int)vecY->valueType);
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// Bytes a transposed product needs besides y: an fp32 accumulator when y is 16-bit.
size_t TransScratchBytes(const SpmvCall &c)
{
    const bool narrow = (c.outType == B200SP_F16 || c.outType == B200SP_BF16);
    return narrow ? sizeof(float) * (size_t)c.A->cols : 0;
}

b200spScalars ReadScalars(const aclsparseContext *h, const void *alpha, const void *beta, int compType)
{
    b200spScalars s{};
    s.alpha_f = 1.0f;  // NULL alpha = 1, NULL beta = 0 (spmv_host.cpp:183-199)
    s.beta_f = 0.0f;
    s.alpha_i = 1;
    s.beta_i = 0;
    if (h->pointerMode == ACL_SPARSE_POINTER_MODE_DEVICE) {
        s.alpha_dev = alpha;
        s.beta_dev = beta;
        return s;
    }
    if (alpha != nullptr) {
        if (compType == B200SP_F32) s.alpha_f = *static_cast<const float *>(alpha);
        else s.alpha_i = *static_cast<const int32_t *>(alpha);
    }
    if (beta != nullptr) {
        if (compType == B200SP_F32) s.beta_f = *static_cast<const float *>(beta);
        else s.beta_i = *static_cast<const int32_t *>(beta);
    }
    return s;
}

constexpr int32_t kTransPlan = 3;       // ActivePlan::spmvInfo[0] of a transposed-product analysis ([1] = longest row)
constexpr int32_t kTransLongRow = 2048;  // a lane group walks at most this many entries of one row alone

bool PlanMatches(const ActivePlan &p, const void *buffer, const aclsparseSpMatDescr *A)
{
    return buffer != nullptr && p.kind == PlanKind::kSpmv && p.buffer == buffer && p.rowPtr == A->offsets &&
           p.rows == A->rows && p.nnz == A->nnz && p.generation == b200sp::BufferGeneration(buffer);
}

}  // namespace

extern "C" {

aclsparseStatus_t aclsparseSpMVGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                             const void *beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                             aclsparseSpMVAlg_t alg, size_t *bufferSize)
{
    (void)alpha;
    (void)beta;
    if (bufferSize == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    SpmvCall c;
    const aclsparseStatus_t st =
        ValidateSpmv("aclsparseSpMVGetBufferSize", handle, opA, matA, vecX, vecY, computeType, alg, &c);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    const size_t plan = b200sp_spmv_plan_bytes(matA->rows, matA->cols, matA->nnz);
    const size_t trans = TransScratchBytes(c);
    size_t need = c.trans ? trans : plan;
    if (need == 0) need = 256;  // never report 0: callers malloc the result
    *bufferSize = need;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                          aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                          const void *beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                          aclsparseSpMVAlg_t alg, void *externalBuffer)
{
    (void)alpha;
    (void)beta;
    SpmvCall c;
    const aclsparseStatus_t st =
        ValidateSpmv("aclsparseSpMVPreprocess", handle, opA, matA, vecX, vecY, computeType, alg, &c);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (externalBuffer == nullptr) return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
    if (c.trans) {
        // The scatter path only wants to know whether some row is far longer than a warp should walk alone.
        ActivePlan t;
        int32_t maxLen = 0;
        t.generation = b200sp::NoteBufferWrite(externalBuffer);
        const int rcT = b200sp_spmv_max_row_length(static_cast<const int32_t *>(matA->offsets), matA->rows,
                                                   externalBuffer, &maxLen, handle->stream);
        if (rcT != 0) {
            B200SP_LOGE("aclsparseSpMVPreprocess: analysis failed (cuda error %d)", rcT);
            return ACL_SPARSE_STATUS_EXECUTION_FAILED;
        }
        t.buffer = externalBuffer;
        t.kind = PlanKind::kSpmv;
        t.rowPtr = matA->offsets;
        t.rows = matA->rows;
        t.nnz = matA->nnz;
        t.spmvInfo[0] = kTransPlan;
        t.spmvInfo[1] = maxLen;
        matA->active = t;
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    const size_t bytes = b200sp_spmv_plan_bytes(matA->rows, matA->cols, matA->nnz);
    ActivePlan p;
    p.generation = b200sp::NoteBufferWrite(externalBuffer);
    // Preprocess is the one place that may synchronise: it asks for the binned plan.
    const int rc = b200sp_spmv_analyze(static_cast<const int32_t *>(matA->offsets),
                                       static_cast<const int32_t *>(matA->indices), matA->rows, matA->cols,
                                       matA->nnz, externalBuffer, bytes, p.spmvInfo, handle->stream);
    if (rc != 0) {
        B200SP_LOGE("aclsparseSpMVPreprocess: analysis failed (cuda error %d)", rc);
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    p.buffer = externalBuffer;
    p.kind = PlanKind::kSpmv;
    p.rowPtr = matA->offsets;
    p.rows = matA->rows;
    p.nnz = matA->nnz;
    matA->active = p;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMV(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX, const void *beta,
                                aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                void *externalBuffer)
{
    SpmvCall c;
    const aclsparseStatus_t st = ValidateSpmv("aclsparseSpMV", handle, opA, matA, vecX, vecY, computeType, alg, &c);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;

    const b200spScalars sc = ReadScalars(handle, alpha, beta, c.compType);
    const auto *rowPtr = static_cast<const int32_t *>(matA->offsets);
    const auto *colInd = static_cast<const int32_t *>(matA->indices);
    cudaStream_t stream = handle->stream;
    int rc = 0;

    if (c.trans) {
        void *scratch = externalBuffer;
        size_t scratchBytes = TransScratchBytes(c);  // a caller buffer is trusted to hold GetBufferSize bytes
        if (scratch == nullptr && scratchBytes > 0) {
            scratch = handle->Workspace();
            if (handle->WorkspaceBytes() < scratchBytes) {
                B200SP_LOGE("aclsparseSpMV: transposed product with 16-bit y needs %zu bytes of buffer", scratchBytes);
                return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
            }
        }
        // Preprocess'ed and a row of kTransLongRow entries or more: cut the scatter by non-zeros.  (A transposed
        // plan is host-side knowledge only, so it survives the accumulator written into the buffer below.)
        const bool byNnz = PlanMatches(matA->active, externalBuffer, matA) &&
                           matA->active.spmvInfo[0] == kTransPlan && matA->active.spmvInfo[1] >= kTransLongRow;
        // A 16-bit y accumulates in the buffer: whatever analysis any matrix had in it is gone.
        if (scratch == externalBuffer && scratchBytes > 0) {
            const uint64_t gen = b200sp::NoteBufferWrite(externalBuffer);
            if (byNnz) matA->active.generation = gen;
        }
        rc = b200sp_spmv_trans_launch(rowPtr, colInd, matA->values, vecX->values, vecY->values, matA->rows,
                                      matA->cols, matA->nnz, &sc, c.compType, c.valType, c.outType, scratch,
                                      scratchBytes, byNnz ? 1 : 0, stream);
    } else {
        void *plan = nullptr;
        const int32_t *info = nullptr;
        const bool active = PlanMatches(matA->active, externalBuffer, matA);
        if (active && matA->active.spmvInfo[0] == kTransPlan) {
            // The buffer was sized and analysed for the transposed product (GetBufferSize with op = T may have
            // returned as little as 256 bytes): a tile plan must not be written into it.
            B200SP_LOGE("aclsparseSpMV: externalBuffer was preprocessed for the transposed product; "
                        "run aclsparseSpMVGetBufferSize / Preprocess with ACL_SPARSE_OP_NON_TRANSPOSE");
            return ACL_SPARSE_STATUS_INVALID_VALUE;
        }
        if (active) {
            plan = externalBuffer;  // analysed by Preprocess: nothing to redo
            info = matA->active.spmvInfo;
        } else {
            // Per-call analysis stays asynchronous: a tile plan, in the caller's buffer or the handle workspace.
            const size_t bytes = b200sp_spmv_tile_plan_bytes(matA->rows, matA->nnz);
            if (externalBuffer != nullptr) plan = externalBuffer;
            else if (handle->WorkspaceBytes() >= bytes) plan = handle->Workspace();
            if (plan != nullptr) {
                (void)b200sp::NoteBufferWrite(plan);  // a plan recorded for this buffer, of any matrix, is stale now
                rc = b200sp_spmv_analyze(rowPtr, colInd, matA->rows, matA->cols, matA->nnz, plan, bytes, nullptr, stream);
                if (rc != 0) {
                    B200SP_LOGE("aclsparseSpMV: analysis launch failed (cuda error %d)", rc);
                    return ACL_SPARSE_STATUS_EXECUTION_FAILED;
                }
            }
        }
        rc = b200sp_spmv_launch(rowPtr, colInd, matA->values, vecX->values, vecY->values, matA->rows, matA->cols,
                                matA->nnz, &sc, c.compType, c.valType, c.outType, plan, info, stream);
    }
    if (rc != 0) {
        B200SP_LOGE("aclsparseSpMV: kernel launch failed (cuda error %d)", rc);
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
