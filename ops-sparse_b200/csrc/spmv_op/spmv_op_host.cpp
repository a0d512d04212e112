// aclsparseSpMVOp_*: the plan API for Z = alpha * A * X + beta * Y.
// Argument checks, their order and their status codes follow the reference host layer
// (sparse/spmv_op/arch35/spmv_op_host.cpp:65-297, 496-745); the device work is in spmv_op_kernels.cu.
#include <climits>
#include <new>

#include "b200sp_kernels.h"
#include "common/internal.h"

struct aclsparseSpMVOpDescr {
    int64_t m = 0, n = 0, nnz = 0;
    aclsparseIndexBase_t indexBase = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseIndexType_t rowOffsetType = ACL_SPARSE_INDEX_32I;
    const void *csrRowOffsets = nullptr;
    const void *csrColInd = nullptr;
    const void *csrValues = nullptr;
    aclsparseSpMVOpAlg_t alg = ACL_SPARSE_SPMVOP_ALG1;
    void *userBuffer = nullptr;                         // ALG2: the caller's workspace (row order)
    int32_t classStart[B200SP_SPMVOP_CLASSES + 1] = {};  // ALG2: where each length class starts in it
};

struct aclsparseSpMVOpPlan {
    aclsparseSpMVOpDescr *descr = nullptr;
    aclsparseSpMVOpAlg_t alg = ACL_SPARSE_SPMVOP_ALG1;
};

namespace {

constexpr const char *kTag = "aclsparseSpMVOp";

// spmv_op_host.cpp:65-97
aclsparseStatus_t ValidateSpMat(aclsparseConstSpMatDescr_t matA)
{
    if (matA == nullptr) {
        B200SP_LOGE("%s: matA is nullptr", kTag);
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    }
    if (matA->format != ACL_SPARSE_FORMAT_CSR) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (matA->valueType != ACL_FLOAT) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (matA->indexType != ACL_SPARSE_INDEX_32I) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (matA->offsetType != ACL_SPARSE_INDEX_32I && matA->offsetType != ACL_SPARSE_INDEX_64I)
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    return ACL_SPARSE_STATUS_SUCCESS;
}

// spmv_op_host.cpp:100-114
aclsparseStatus_t ValidateCommon(aclsparseOperation_t opA, aclDataType computeType)
{
    if (opA != ACL_SPARSE_OP_NON_TRANSPOSE) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (computeType != ACL_FLOAT) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    return ACL_SPARSE_STATUS_SUCCESS;
}

// spmv_op_host.cpp:117-126
aclsparseStatus_t ValidateAlg(aclsparseSpMVOpAlg_t alg)
{
    if (alg != ACL_SPARSE_SPMVOP_ALG_DEFAULT && alg != ACL_SPARSE_SPMVOP_ALG1 && alg != ACL_SPARSE_SPMVOP_ALG2)
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

aclsparseStatus_t aclsparseSpMVOp_bufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                             aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ,
                                             aclDataType computeType, aclsparseSpMVOpAlg_t alg, size_t *bufferSize)
{
    (void)vecX;
    (void)vecY;
    (void)vecZ;
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    // order of spmv_op_host.cpp:135-150
    aclsparseStatus_t st = ValidateCommon(opA, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    st = ValidateSpMat(matA);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    st = ValidateAlg(alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (bufferSize == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (matA->rows > (int64_t)INT32_MAX) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    // ALG1 needs nothing (the reference reports 0 as well); ALG2 holds the row order.
    *bufferSize = alg == ACL_SPARSE_SPMVOP_ALG2 ? b200sp_spmvop_plan_bytes(matA->rows) : 0;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVOp_createDescr(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t *descr,
                                              aclsparseOperation_t opA, aclsparseConstSpMatDescr_t matA,
                                              aclsparseConstDnVecDescr_t vecX, aclsparseConstDnVecDescr_t vecY,
                                              aclsparseDnVecDescr_t vecZ, aclDataType computeType,
                                              aclsparseSpMVOpAlg_t alg, void *buffer)
{
    (void)vecX;
    (void)vecY;
    (void)vecZ;
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    // order of spmv_op_host.cpp:156-177, 603-621
    if (descr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    aclsparseStatus_t st = ValidateSpMat(matA);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    st = ValidateAlg(alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (alg == ACL_SPARSE_SPMVOP_ALG2 && buffer == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    st = ValidateCommon(opA, computeType);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (matA->rows > (int64_t)INT32_MAX) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (matA->base != ACL_SPARSE_INDEX_BASE_ZERO && matA->base != ACL_SPARSE_INDEX_BASE_ONE)
        return ACL_SPARSE_STATUS_INVALID_VALUE;

    auto *d = new (std::nothrow) aclsparseSpMVOpDescr();
    if (d == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;
    d->m = matA->rows;
    d->n = matA->cols;
    d->nnz = matA->nnz;
    d->indexBase = matA->base;
    d->rowOffsetType = matA->offsetType;
    d->csrRowOffsets = matA->offsets;
    d->csrColInd = matA->indices;
    d->csrValues = matA->values;
    d->alg = alg == ACL_SPARSE_SPMVOP_ALG_DEFAULT ? ACL_SPARSE_SPMVOP_ALG1 : alg;
    if (d->alg == ACL_SPARSE_SPMVOP_ALG2) {
        const int rc = b200sp_spmvop_analyze(d->csrRowOffsets, d->rowOffsetType == ACL_SPARSE_INDEX_64I, d->m,
                                             buffer, b200sp_spmvop_plan_bytes(d->m), d->classStart, handle->stream);
        if (rc != 0) {
            B200SP_LOGE("%s_createDescr: row ordering failed (cuda error %d)", kTag, rc);
            delete d;
            return ACL_SPARSE_STATUS_EXECUTION_FAILED;
        }
        d->userBuffer = buffer;
    }
    *descr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVOp_destroyDescr(aclsparseSpMVOpDescr_t descr)
{
    delete descr;  // NULL is accepted (spmv_op_host.cpp:650-657)
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVOp_createPlan(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t descr,
                                             aclsparseSpMVOpPlan_t *plan, const void *epilogueLTOBuffer,
                                             size_t epilogueLTOBufferSize)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    // spmv_op_host.cpp:183-202
    if (descr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (plan == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (epilogueLTOBuffer != nullptr || epilogueLTOBufferSize > 0) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    auto *p = new (std::nothrow) aclsparseSpMVOpPlan();
    if (p == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;
    p->descr = descr;
    p->alg = descr->alg;
    *plan = p;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVOp_destroyPlan(aclsparseSpMVOpPlan_t plan)
{
    delete plan;  // NULL is accepted (spmv_op_host.cpp:689-696)
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVOp_setGlobalUserData(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan,
                                                    const char *epilogueDataName, void *epilogueData,
                                                    size_t epilogueDataSize)
{
    (void)epilogueDataName;
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (plan == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    // data and size must agree (spmv_op_host.cpp:713-717); the identity epilogue has nothing to set
    if ((epilogueData == nullptr) != (epilogueDataSize == 0)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMVOp(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan, const void *alpha,
                                  const void *beta, aclsparseConstDnVecDescr_t vecX,
                                  aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    // spmv_op_host.cpp:208-234
    if (plan == nullptr || plan->descr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (alpha == nullptr || beta == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (vecX == nullptr || vecY == nullptr || vecZ == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const aclsparseSpMVOpDescr *d = plan->descr;
    // spmv_op_host.cpp:236-287
    if (vecX->valueType != ACL_FLOAT || vecY->valueType != ACL_FLOAT || vecZ->valueType != ACL_FLOAT)
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (d->n > 0 && vecX->values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const bool hostScalars = handle->pointerMode == ACL_SPARSE_POINTER_MODE_HOST;
    // With device scalars beta cannot be read here; the kernel does not touch Y when beta == 0.
    const bool skipYCheck = hostScalars ? (*static_cast<const float *>(beta) == 0.0f) : true;
    if (!skipYCheck && d->m > 0 && vecY->values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (d->m > 0 && vecZ->values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (vecX->size != d->n || vecY->size != d->m || vecZ->size != d->m) return ACL_SPARSE_STATUS_INVALID_VALUE;

    // spmv_op_host.cpp:465-492
    if (d->m > (int64_t)INT32_MAX) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (d->m == 0) return ACL_SPARSE_STATUS_SUCCESS;
    const float a = hostScalars ? *static_cast<const float *>(alpha) : 0.0f;
    const float b = hostScalars ? *static_cast<const float *>(beta) : 0.0f;
    const float *aDev = hostScalars ? nullptr : static_cast<const float *>(alpha);
    const float *bDev = hostScalars ? nullptr : static_cast<const float *>(beta);
    auto *y = static_cast<const float *>(vecY->values);
    auto *z = static_cast<float *>(vecZ->values);
    int rc;
    if (d->nnz == 0) {
        rc = b200sp_spmvop_scale(y, z, d->m, b, bDev, handle->stream);
    } else {
        const bool planned = d->alg == ACL_SPARSE_SPMVOP_ALG2 && d->userBuffer != nullptr;
        rc = b200sp_spmvop_launch(d->csrRowOffsets, d->rowOffsetType == ACL_SPARSE_INDEX_64I,
                                  static_cast<const int32_t *>(d->csrColInd), static_cast<const float *>(d->csrValues),
                                  static_cast<const float *>(vecX->values), y, z, d->m, d->nnz,
                                  d->indexBase == ACL_SPARSE_INDEX_BASE_ONE ? 1 : 0, a, b, aDev, bDev,
                                  planned ? d->userBuffer : nullptr, planned ? d->classStart : nullptr,
                                  handle->stream);
    }
    if (rc != 0) {
        B200SP_LOGE("%s: kernel launch failed (cuda error %d)", kTag, rc);
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
