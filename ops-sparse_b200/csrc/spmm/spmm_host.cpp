// aclsparseSpMM / SpMMGetBufferSize / SpMMPreprocess host layer.
//
// Checks, their order and status codes follow the reference's three-stage flow
// (sparse/spmm/arch35/spmm_host.cpp:152-191 validation, 213-234 size, 335-362 preprocess,
// 364-394 compute).  alpha / beta are per-call (read at every aclsparseSpMM, as arch35's
// refresh step does, spmm_host.cpp:281-308) but travel as kernel arguments, so the compute
// call makes no host<->device copy.  Pointer mode DEVICE is honoured (as arch22 does,
// sparse/spmm/arch22/spmm_host.cpp:26-43) without the synchronous read-back.
// Extension: (bf16, bf16, f32 | bf16, compute f32) is accepted besides the reference's
// three type combinations (spmm_host.cpp:108-112).
#include "../common/internal.h"
#include "b200sp_bench.h"

namespace {

using b200sp::ActivePlan;
using b200sp::PlanKind;

bool SupportedTypes(aclDataType a, aclDataType b, aclDataType c, aclDataType compute)
{
    if (a != b) return false;
    if (a == ACL_FLOAT) return c == ACL_FLOAT && compute == ACL_FLOAT;
    if (a == ACL_FLOAT16) return c == ACL_FLOAT16 && compute == ACL_FLOAT;
    if (a == ACL_INT8) return c == ACL_INT32 && compute == ACL_INT32;
    if (a == ACL_BF16) return (c == ACL_BF16 || c == ACL_FLOAT) && compute == ACL_FLOAT;
    return false;
}

aclsparseStatus_t ValidateSpmm(aclsparseOperation_t opA, aclsparseOperation_t opB, const aclsparseSpMatDescr *A,
                               const aclsparseDnMatDescr *B, const aclsparseDnMatDescr *C, aclDataType computeType,
                               aclsparseSpMMAlg_t alg)
{
    if (A == nullptr || B == nullptr || C == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (opA != ACL_SPARSE_OP_NON_TRANSPOSE) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (opB != ACL_SPARSE_OP_NON_TRANSPOSE && opB != ACL_SPARSE_OP_TRANSPOSE) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (A->format != ACL_SPARSE_FORMAT_CSR) return ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED;
    const aclsparseStatus_t idx = b200sp::CheckExecIndexTypes(A->offsetType, A->indexType);
    if (idx != ACL_SPARSE_STATUS_SUCCESS) return idx;
    if (A->base != ACL_SPARSE_INDEX_BASE_ZERO) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (!SupportedTypes(A->valueType, B->valueType, C->valueType, computeType)) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    // The B descriptor is always K x N, also for opB = T (spmm_host.cpp:122-131).
    if (A->cols != B->rows || A->rows != C->rows || B->cols != C->cols) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (alg != ACL_SPARSE_SPMM_ALG_DEFAULT && alg != ACL_SPARSE_SPMM_CSR_ALG1 &&
        alg != ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG)
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (A->rows > INT32_MAX || C->cols > INT32_MAX || A->nnz > INT32_MAX) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    return ACL_SPARSE_STATUS_SUCCESS;
}

struct Analysis {
    int32_t segments = 0, blockUnits = 0, longRows = 0;
};

size_t ElemBytes(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT: case ACL_INT32: return 4;
        case ACL_FLOAT16: case ACL_BF16: return 2;
        default: return 1;
    }
}

aclsparseStatus_t Analyse(const aclsparseSpMatDescr *A, int64_t n, void *buffer, cudaStream_t stream, Analysis *out)
{
    int32_t *segments = &out->segments;
    const size_t bytes = b200sp_spmm_plan_bytes(A->rows, A->nnz, n);
    // Whatever plan this buffer held is overwritten now; an active plan that is not re-recorded below goes stale.
    (void)b200sp::NoteBufferWrite(buffer);
    const int rc = b200sp_spmm_analyze(static_cast<const int32_t *>(A->offsets), A->rows, A->nnz, n, buffer, bytes,
                                       segments, stream);
    if (rc != 0) {
        B200SP_LOGE("aclsparseSpMM: analysis failed (cuda error %d)", rc);
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (*segments > 0 && A->indices != nullptr) {  // long rows: by column blocks of B where that pays
        const int rb = b200sp_spmm_analyze_blocks(static_cast<const int32_t *>(A->offsets),
                                                  static_cast<const int32_t *>(A->indices), A->rows, A->cols, A->nnz,
                                                  n, n * (int64_t)ElemBytes(A->valueType), buffer, bytes,
                                                  &out->blockUnits, &out->longRows, stream);
        if (rb != 0) {
            B200SP_LOGE("aclsparseSpMM: column-block analysis failed (cuda error %d)", rb);
            return ACL_SPARSE_STATUS_EXECUTION_FAILED;
        }
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

bool PlanMatches(const ActivePlan &p, const void *buffer, const aclsparseSpMatDescr *A, int64_t n)
{
    return p.kind == PlanKind::kSpmm && p.buffer == buffer && p.rowPtr == A->offsets && p.rows == A->rows &&
           p.nnz == A->nnz && p.n == n && p.generation == b200sp::BufferGeneration(buffer) &&
           (p.blockUnits == 0 || (p.colInd == A->indices && p.valueType == (int32_t)A->valueType));
}

}  // namespace

extern "C" {

aclsparseStatus_t aclsparseSpMMGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseOperation_t opB, const void *alpha,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                             const void *beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                             aclsparseSpMMAlg_t alg, size_t *size)
{
    (void)handle;
    (void)alpha;
    (void)beta;
    if (size == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const aclsparseStatus_t st = ValidateSpmm(opA, opB, matA, matB, matC, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    *size = b200sp_spmm_plan_bytes(matA->rows, matA->nnz, matC->cols);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMMPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                          aclsparseOperation_t opB, const void *alpha,
                                          aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                          const void *beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                          aclsparseSpMMAlg_t alg, void *buffer)
{
    (void)alpha;
    (void)beta;
    const aclsparseStatus_t st = ValidateSpmm(opA, opB, matA, matB, matC, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (buffer == nullptr) return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
    if (matA->offsets == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Analysis found;
    const aclsparseStatus_t an =
        Analyse(matA, matC->cols, buffer, handle != nullptr ? handle->stream : nullptr, &found);
    if (an != ACL_SPARSE_STATUS_SUCCESS) return an;
    // The analysis has just synchronised: the one place on this path where a row-stream product that gave up on a
    // copy (see b200sp_spmm_stream_error) can be reported without adding a synchronisation to a compute call.
    if (b200sp_spmm_stream_error() == 1) {
        (void)b200sp_spmm_stream_error_clear();
        B200SP_LOGE("aclsparseSpMMPreprocess: an earlier aclsparseSpMM gave up waiting for a copy; its C is incomplete");
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    ActivePlan p;
    p.buffer = buffer;
    p.kind = PlanKind::kSpmm;
    p.rowPtr = matA->offsets;
    p.rows = matA->rows;
    p.nnz = matA->nnz;
    p.n = matC->cols;
    p.segments = found.segments;
    p.blockUnits = found.blockUnits;
    p.longRows = found.longRows;
    p.colInd = matA->indices;
    p.valueType = (int32_t)matA->valueType;
    p.generation = b200sp::BufferGeneration(buffer);
    matA->active = p;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMM(aclsparseHandle_t handle, aclsparseOperation_t opA, aclsparseOperation_t opB,
                                const void *alpha, aclsparseConstSpMatDescr_t matA,
                                aclsparseConstDnMatDescr_t matB, const void *beta, aclsparseDnMatDescr_t matC,
                                aclDataType computeType, aclsparseSpMMAlg_t alg, void *buffer)
{
    const aclsparseStatus_t st = ValidateSpmm(opA, opB, matA, matB, matC, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (buffer == nullptr) return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (matA->offsets == nullptr || (matA->nnz > 0 && (matA->indices == nullptr || matA->values == nullptr)))
        return ACL_SPARSE_STATUS_INVALID_VALUE;

    Analysis found;
    if (PlanMatches(matA->active, buffer, matA, matC->cols)) {
        found.segments = matA->active.segments;
        found.blockUnits = matA->active.blockUnits;
        found.longRows = matA->active.longRows;
    } else {
        // Not the active buffer: analyse into it now, as the reference rebuilds its tiling
        // in place (spmm_host.cpp:310-321).  This path synchronises the stream once.
        const aclsparseStatus_t an = Analyse(matA, matC->cols, buffer, handle->stream, &found);
        if (an != ACL_SPARSE_STATUS_SUCCESS) return an;
    }

    b200spScalars sc{};  // NULL scalar reads as 0 (spmm_host.cpp:62-74)
    if (handle->pointerMode == ACL_SPARSE_POINTER_MODE_DEVICE) {
        sc.alpha_dev = alpha;
        sc.beta_dev = beta;
    } else if (computeType == ACL_INT32) {
        if (alpha != nullptr) sc.alpha_i = *static_cast<const int32_t *>(alpha);
        if (beta != nullptr) sc.beta_i = *static_cast<const int32_t *>(beta);
    } else {
        if (alpha != nullptr) sc.alpha_f = *static_cast<const float *>(alpha);
        if (beta != nullptr) sc.beta_f = *static_cast<const float *>(beta);
    }

    b200spSpmmShape sh{};
    sh.m = matA->rows;
    sh.k = matA->cols;
    sh.n = matC->cols;
    sh.nnz = matA->nnz;
    sh.ldb = matB->ld;
    sh.ldc = matC->ld;
    sh.order_b = (matB->order == ACL_SPARSE_ORDER_COL) ? 1 : 0;
    sh.order_c = (matC->order == ACL_SPARSE_ORDER_COL) ? 1 : 0;
    sh.op_b = (opB == ACL_SPARSE_OP_TRANSPOSE) ? 1 : 0;
    sh.block_units = found.blockUnits;
    sh.long_rows = found.longRows;
    sh.kahan = (alg == ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG && matA->valueType == ACL_FLOAT) ? 1 : 0;

    const int rc = b200sp_spmm_launch(static_cast<const int32_t *>(matA->offsets),
                                      static_cast<const int32_t *>(matA->indices), matA->values, matB->values,
                                      matC->values, &sh, &sc, b200sp::KernelTypeOf(matA->valueType),
                                      b200sp::KernelTypeOf(matC->valueType), buffer, found.segments, handle->stream);
    if (rc != 0) {
        B200SP_LOGE("aclsparseSpMM: kernel launch failed (cuda error %d)", rc);
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// What the analysis recorded in matA's active SpMM plan: info = {segments, units of the column-block path, long
// rows, 1 if a plan is recorded at all}.  For benchmarks and tests that must say which kernels a product runs.
aclsparseStatus_t b200spSpMMPlanInfo(aclsparseConstSpMatDescr_t matA, int32_t info[4])
{
    if (matA == nullptr || info == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const bool on = matA->active.kind == PlanKind::kSpmm;
    info[0] = on ? matA->active.segments : 0;
    info[1] = on ? matA->active.blockUnits : 0;
    info[2] = on ? matA->active.longRows : 0;
    info[3] = on ? 1 : 0;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
