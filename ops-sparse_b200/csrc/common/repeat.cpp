// A compiled caller's loop over the compute entry points, for benchmarks driven from an interpreter.
//
// A product on a small matrix takes a few microseconds of GPU time; a Python / ctypes call takes longer than
// that, so a loop written in Python measures the interpreter.  These helpers issue the same aclsparseSpMV /
// aclsparseSpMM call `reps` times back to back, exactly as the reference's own benchmark loop does from C++
// (test/spmm/arch22/spmm_test.cpp:385-393), and return the first status that is not SUCCESS.
#include "internal.h"
#include "b200sp_bench.h"
#include "b200sp_mg.h"

extern "C" {

aclsparseStatus_t b200spRepeatSpMV(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                   aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX, const void *beta,
                                   aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                   void *externalBuffer, int reps)
{
    for (int i = 0; i < reps; ++i) {
        const aclsparseStatus_t st =
            aclsparseSpMV(handle, opA, alpha, matA, vecX, beta, vecY, computeType, alg, externalBuffer);
        if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t b200spRepeatSpMM(aclsparseHandle_t handle, aclsparseOperation_t opA, aclsparseOperation_t opB,
                                   const void *alpha, aclsparseConstSpMatDescr_t matA,
                                   aclsparseConstDnMatDescr_t matB, const void *beta, aclsparseDnMatDescr_t matC,
                                   aclDataType computeType, aclsparseSpMMAlg_t alg, void *buffer, int reps)
{
    for (int i = 0; i < reps; ++i) {
        const aclsparseStatus_t st =
            aclsparseSpMM(handle, opA, opB, alpha, matA, matB, beta, matC, computeType, alg, buffer);
        if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

// The same for a row-sharded operator on several GPUs: every step is one exchange of this rank's slice of the
// dense operand (b200spMgPush into replica seq % replicas, waiting for every rank) followed by the product
// against that replica's descriptor.
aclsparseStatus_t b200spMgRepeatSpMV(b200spMgExchange *ex, const void *slice, size_t offset, size_t bytes,
                                     uint32_t firstSeq, int replicas, uint32_t waitMask, aclsparseHandle_t handle,
                                     aclsparseOperation_t opA, const void *alpha, aclsparseConstSpMatDescr_t matA,
                                     const aclsparseConstDnVecDescr_t *vecXOfReplica, const void *beta,
                                     aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                     void *externalBuffer, int reps)
{
    if (ex == nullptr || vecXOfReplica == nullptr || replicas < 1) return ACL_SPARSE_STATUS_INVALID_VALUE;
    aclrtStream stream = nullptr;
    aclsparseStatus_t st = aclsparseGetStream(handle, &stream);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    for (int i = 0; i < reps; ++i) {
        const uint32_t seq = firstSeq + (uint32_t)i;
        const int replica = (int)(seq % (uint32_t)replicas);
        if (b200spMgPush(ex, replica, slice, offset, bytes, seq, waitMask, stream) != 0)
            return ACL_SPARSE_STATUS_EXECUTION_FAILED;
        st = aclsparseSpMV(handle, opA, alpha, matA, vecXOfReplica[replica], beta, vecY, computeType, alg,
                           externalBuffer);
        if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t b200spMgRepeatSpMM(b200spMgExchange *ex, const void *slice, size_t offset, size_t bytes,
                                     uint32_t firstSeq, int replicas, uint32_t waitMask, aclsparseHandle_t handle,
                                     aclsparseOperation_t opA, aclsparseOperation_t opB, const void *alpha,
                                     aclsparseConstSpMatDescr_t matA, const aclsparseConstDnMatDescr_t *matBOfReplica,
                                     const void *beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                     aclsparseSpMMAlg_t alg, void *buffer, int reps)
{
    if (ex == nullptr || matBOfReplica == nullptr || replicas < 1) return ACL_SPARSE_STATUS_INVALID_VALUE;
    aclrtStream stream = nullptr;
    aclsparseStatus_t st = aclsparseGetStream(handle, &stream);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    for (int i = 0; i < reps; ++i) {
        const uint32_t seq = firstSeq + (uint32_t)i;
        const int replica = (int)(seq % (uint32_t)replicas);
        if (b200spMgPush(ex, replica, slice, offset, bytes, seq, waitMask, stream) != 0)
            return ACL_SPARSE_STATUS_EXECUTION_FAILED;
        st = aclsparseSpMM(handle, opA, opB, alpha, matA, matBOfReplica[replica], beta, matC, computeType, alg, buffer);
        if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
