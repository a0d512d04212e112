/*
 * b200sp_bench.h -- a compiled caller's loop over the two compute entry points (one GPU, or one rank of several).
 *
 * No counterpart in the reference library; the reference's own benchmark loop is C++ that calls the compute
 * entry point repeatedly (test/spmm/arch22/spmm_test.cpp:385-393).  A benchmark driven from an interpreter
 * uses these instead of looping itself, so that what is timed is the library and the GPU, not the interpreter's
 * call overhead (several microseconds per call, more than a small product takes).
 * Each function makes `reps` identical calls back to back and returns the first status that is not SUCCESS.
 */
#ifndef B200SP_BENCH_H_
#define B200SP_BENCH_H_

#include "cann_ops_sparse.h"
#include "b200sp_mg.h"

#ifdef __cplusplus
extern "C" {
#endif

aclsparseStatus_t b200spRepeatSpMV(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                   aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX, const void *beta,
                                   aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                   void *externalBuffer, int reps);

aclsparseStatus_t b200spRepeatSpMM(aclsparseHandle_t handle, aclsparseOperation_t opA, aclsparseOperation_t opB,
                                   const void *alpha, aclsparseConstSpMatDescr_t matA,
                                   aclsparseConstDnMatDescr_t matB, const void *beta, aclsparseDnMatDescr_t matC,
                                   aclDataType computeType, aclsparseSpMMAlg_t alg, void *buffer, int reps);

/* What aclsparseSpMMPreprocess recorded for matA: info = {long-row segments, units of the column-block path
 * (0 = the long rows are summed by segments), long rows, 1 if a plan is recorded}. */
aclsparseStatus_t b200spSpMMPlanInfo(aclsparseConstSpMatDescr_t matA, int32_t info[4]);

/* Row-sharded operator on several GPUs: `reps` steps, step i = b200spMgPush of this rank's slice (`slice`,
 * `offset`, `bytes` as for b200spMgPush) with sequence number firstSeq + i into replica (firstSeq + i) % replicas,
 * on the handle's stream, followed by the product against that replica's descriptor
 * (vecXOfReplica / matBOfReplica: `replicas` descriptors over b200spMgExchangeReplica(ex, r)). */
aclsparseStatus_t b200spMgRepeatSpMV(b200spMgExchange *ex, const void *slice, size_t offset, size_t bytes,
                                     uint32_t firstSeq, int replicas, uint32_t waitMask, aclsparseHandle_t handle,
                                     aclsparseOperation_t opA, const void *alpha, aclsparseConstSpMatDescr_t matA,
                                     const aclsparseConstDnVecDescr_t *vecXOfReplica, const void *beta,
                                     aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                     void *externalBuffer, int reps);

aclsparseStatus_t b200spMgRepeatSpMM(b200spMgExchange *ex, const void *slice, size_t offset, size_t bytes,
                                     uint32_t firstSeq, int replicas, uint32_t waitMask, aclsparseHandle_t handle,
                                     aclsparseOperation_t opA, aclsparseOperation_t opB, const void *alpha,
                                     aclsparseConstSpMatDescr_t matA, const aclsparseConstDnMatDescr_t *matBOfReplica,
                                     const void *beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                     aclsparseSpMMAlg_t alg, void *buffer, int reps);

#ifdef __cplusplus
}
#endif

#endif /* B200SP_BENCH_H_ */
