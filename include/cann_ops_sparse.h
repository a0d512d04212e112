/*
 * cann_ops_sparse.h -- aclsparse C API, CSR SpMV / SpMM path, B200 (sm_100a) build.
 *
 * This is the public boundary of libops_sparse.so.  Every type, enumerator order and
 * function signature below is the one the reference library declares in
 * include/cann_ops_sparse.h (line ranges are cited per block), so a program written
 * against the reference for this path recompiles against this header unchanged.
 * Only the hot path is declared: handle, CSR / dense-vector / dense-matrix
 * descriptors, and the SpMV / SpMM  GetBufferSize -> Preprocess -> compute triplets.
 * All pointers named "DEVICE" are CUDA device pointers; descriptors borrow them and
 * never free them.
 */
#ifndef CANN_OPS_SPARSE_H_
#define CANN_OPS_SPARSE_H_

#include <unistd.h>
#include <stdint.h>
#include <acl/acl_base_rt.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums (reference include/cann_ops_sparse.h:24-28, 50-53, 81-95, 98-168, 213-248, 898-901).
 * Enumerator order is part of the ABI and is kept exactly. ---- */

typedef enum aclsparseOperation_t {
    ACL_SPARSE_OP_NON_TRANSPOSE = 0,
    ACL_SPARSE_OP_TRANSPOSE,
    ACL_SPARSE_OP_CONJUGATE_TRANSPOSE
} aclsparseOperation_t;

typedef enum aclsparseOrder_t {
    ACL_SPARSE_ORDER_ROW = 0,
    ACL_SPARSE_ORDER_COL = 1
} aclsparseOrder_t;

typedef enum aclsparseSpMMAlg_t {
    ACL_SPARSE_SPMM_ALG_DEFAULT = 0,
    ACL_SPARSE_SPMM_CSR_ALG1,
    /* fp32 only: Kahan-compensated accumulation; ignored for other value types. */
    ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG
} aclsparseSpMMAlg_t;

typedef enum aclsparseStatus_t {
    ACL_SPARSE_STATUS_SUCCESS = 0,
    ACL_SPARSE_STATUS_NOT_INITIALIZED,
    ACL_SPARSE_STATUS_ALLOC_FAILED,
    ACL_SPARSE_STATUS_INVALID_VALUE,
    ACL_SPARSE_STATUS_ARCH_MISMATCH,
    ACL_SPARSE_STATUS_EXECUTION_FAILED,
    ACL_SPARSE_STATUS_INTERNAL_ERROR,
    ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED,
    ACL_SPARSE_STATUS_NOT_SUPPORTED,
    ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES,
    ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
} aclsparseStatus_t;

typedef enum aclsparseSpMVAlg_t {
    ACL_SPARSE_SPMV_ALG_DEFAULT,
    ACL_SPARSE_SPMV_COO_ALG1,
    ACL_SPARSE_SPMV_COO_ALG2,
    ACL_SPARSE_SPMV_CSR_ALG1,
    ACL_SPARSE_SPMV_CSR_ALG2,
    ACL_SPARSE_SPMV_SELL_ALG1
} aclsparseSpMVAlg_t;

typedef enum aclsparseIndexType_t {
    ACL_SPARSE_INDEX_32I = 0,
    ACL_SPARSE_INDEX_64I
} aclsparseIndexType_t;

typedef enum aclsparseIndexBase_t {
    ACL_SPARSE_INDEX_BASE_ZERO = 0,
    ACL_SPARSE_INDEX_BASE_ONE
} aclsparseIndexBase_t;

typedef enum aclsparseFormat_t {
    ACL_SPARSE_FORMAT_COO = 0,
    ACL_SPARSE_FORMAT_CSR,
    ACL_SPARSE_FORMAT_CSC,
    ACL_SPARSE_FORMAT_BLOCKED_ELL,
    ACL_SPARSE_FORMAT_SLICED_ELL,
    ACL_SPARSE_FORMAT_BSR
} aclsparseFormat_t;

typedef enum aclsparsePointerMode_t {
    ACL_SPARSE_POINTER_MODE_HOST = 0,
    ACL_SPARSE_POINTER_MODE_DEVICE = 1
} aclsparsePointerMode_t;

/* Algorithms of the SpMVOp plan API (reference include/cann_ops_sparse.h:55-70).  DEFAULT routes to
 * ALG1.  ALG1 needs no workspace; ALG2 orders the rows by length in createDescr and needs the
 * workspace that aclsparseSpMVOp_bufferSize reports.  Neither looks at the values of A, so csrValues
 * may be updated in place under both (the reference forbids that under its ALG2). */
typedef enum aclsparseSpMVOpAlg_t {
    ACL_SPARSE_SPMVOP_ALG_DEFAULT = 0,
    ACL_SPARSE_SPMVOP_ALG1,
    ACL_SPARSE_SPMVOP_ALG2
} aclsparseSpMVOpAlg_t;

/* Legacy matrix descriptor and its enums (reference include/cann_ops_sparse.h:188-210). */
struct aclsparseMatDescr;
typedef struct aclsparseMatDescr *aclsparseMatDescr_t;
typedef enum aclsparseMatrixType_t {
    ACL_SPARSE_MATRIX_TYPE_GENERAL = 0,
    ACL_SPARSE_MATRIX_TYPE_SYMMETRIC,
    ACL_SPARSE_MATRIX_TYPE_HERMITIAN,
    ACL_SPARSE_MATRIX_TYPE_TRIANGULAR
} aclsparseMatrixType_t;
typedef enum aclsparseDiagType_t {
    ACL_SPARSE_DIAG_TYPE_NON_UNIT = 0,
    ACL_SPARSE_DIAG_TYPE_UNIT
} aclsparseDiagType_t;
typedef enum aclsparseFillMode_t {
    ACL_SPARSE_FILL_MODE_LOWER = 0,
    ACL_SPARSE_FILL_MODE_UPPER
} aclsparseFillMode_t;

/* CSR -> CSC conversion (reference include/cann_ops_sparse.h:1369-1379). */
typedef enum aclsparseAction_t {
    ACL_SPARSE_ACTION_SYMBOLIC = 0, /* structure only (colPtr, rowInd) */
    ACL_SPARSE_ACTION_NUMERIC       /* structure and values */
} aclsparseAction_t;
typedef enum aclsparseCsr2CscAlg_t {
    ACL_SPARSE_CSR2CSC_ALG_DEFAULT = 0,
    ACL_SPARSE_CSR2CSC_ALG1
} aclsparseCsr2CscAlg_t;

/* SDDMM algorithms (reference include/cann_ops_sparse.h:712-715). */
typedef enum aclsparseSDDMMAlg_t {
    ACL_SPARSE_SDDMM_ALG_DEFAULT = 0
} aclsparseSDDMMAlg_t;

/* ---- opaque types (reference :30-47, 72-78) ---- */
struct aclsparseSpMVOpDescr;
struct aclsparseSpMVOpPlan;
typedef struct aclsparseSpMVOpDescr *aclsparseSpMVOpDescr_t;
typedef struct aclsparseSpMVOpDescr const *aclsparseConstSpMVOpDescr_t;
typedef struct aclsparseSpMVOpPlan *aclsparseSpMVOpPlan_t;
struct aclsparseContext;
struct aclsparseSpMatDescr;
struct aclsparseDnVecDescr;
struct aclsparseDnMatDescr;

typedef struct aclsparseContext *aclsparseHandle_t;
typedef struct aclsparseSpMatDescr *aclsparseSpMatDescr_t;
typedef struct aclsparseDnVecDescr *aclsparseDnVecDescr_t;
typedef struct aclsparseDnMatDescr *aclsparseDnMatDescr_t;
typedef struct aclsparseSpMatDescr const *aclsparseConstSpMatDescr_t;
typedef struct aclsparseDnVecDescr const *aclsparseConstDnVecDescr_t;
typedef struct aclsparseDnMatDescr const *aclsparseConstDnMatDescr_t;

/* ======================================================================================
 * Handle (reference :817-904; behaviour from sparse/common/aclsparse_auxiliary.cpp:64-198,
 * 253-279).  Create needs *handle == NULL on entry and allocates a 4 MiB device
 * workspace; Destroy drains the handle's stream first.  SetWorkspace(NULL) switches back
 * to the built-in workspace; a user workspace only ever grows.
 * ====================================================================================== */
aclsparseStatus_t aclsparseCreate(aclsparseHandle_t *handle);
aclsparseStatus_t aclsparseDestroy(aclsparseHandle_t handle);
aclsparseStatus_t aclsparseSetStream(aclsparseHandle_t handle, aclrtStream stream);
aclsparseStatus_t aclsparseGetStream(aclsparseHandle_t handle, aclrtStream *stream);
aclsparseStatus_t aclsparseSetWorkspace(aclsparseHandle_t handle, void *workspace, size_t workspaceSize);
aclsparseStatus_t aclsparseGetWorkspace(aclsparseHandle_t handle, void **workspace, size_t *workspaceSize);
aclsparseStatus_t aclsparseGetVersion(aclsparseHandle_t handle, int *version);
aclsparseStatus_t aclsparseSetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t mode);
aclsparseStatus_t aclsparseGetPointerMode(aclsparseHandle_t handle, aclsparsePointerMode_t *mode);

/* ======================================================================================
 * Dense vector descriptor (reference :259-273, 335-366; sparse/common/aclsparse_descr.cpp:
 * 96-147, 306-368).  size >= 0; values may be NULL only when size == 0.
 * DestroyDnVec(NULL) is INVALID_VALUE.
 * ====================================================================================== */
aclsparseStatus_t aclsparseCreateDnVec(aclsparseDnVecDescr_t *dnVecDescr, int64_t size, void *values,
                                       aclDataType valueType);
aclsparseStatus_t aclsparseCreateConstDnVec(aclsparseConstDnVecDescr_t *dnVecDescr, int64_t size,
                                            const void *values, aclDataType valueType);
aclsparseStatus_t aclsparseDestroyDnVec(aclsparseConstDnVecDescr_t dnVecDescr);
aclsparseStatus_t aclsparseDnVecGet(aclsparseDnVecDescr_t dnVecDescr, int64_t *size, void **values,
                                    aclDataType *valueType);
aclsparseStatus_t aclsparseConstDnVecGet(aclsparseConstDnVecDescr_t dnVecDescr, int64_t *size,
                                         const void **values, aclDataType *valueType);
aclsparseStatus_t aclsparseDnVecGetValues(aclsparseDnVecDescr_t dnVecDescr, void **values);
aclsparseStatus_t aclsparseConstDnVecGetValues(aclsparseConstDnVecDescr_t dnVecDescr, const void **values);
aclsparseStatus_t aclsparseDnVecSetValues(aclsparseDnVecDescr_t dnVecDescr, void *values);

/* ======================================================================================
 * CSR matrix descriptor (reference :393-402, 443-473; aclsparse_descr.cpp:370-422, 473-492,
 * 517-586).  Create accepts 32- or 64-bit index types; SpMV / SpMM execute only
 * (32I, 32I), zero-based.  DestroySpMat(NULL) is SUCCESS.
 * ====================================================================================== */
aclsparseStatus_t aclsparseCreateCsr(aclsparseSpMatDescr_t *spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                     void *csrRowOffsets, void *csrColInd, void *csrValues,
                                     aclsparseIndexType_t csrRowOffsetsType, aclsparseIndexType_t csrColIndType,
                                     aclsparseIndexBase_t idxBase, aclDataType valueType);
aclsparseStatus_t aclsparseCreateConstCsr(aclsparseConstSpMatDescr_t *spMatDescr, int64_t rows, int64_t cols,
                                          int64_t nnz, const void *csrRowOffsets, const void *csrColInd,
                                          const void *csrValues, aclsparseIndexType_t csrRowOffsetsType,
                                          aclsparseIndexType_t csrColIndType, aclsparseIndexBase_t idxBase,
                                          aclDataType valueType);
aclsparseStatus_t aclsparseCsrSetPointers(aclsparseSpMatDescr_t descr, void *rowOffsets, void *colIndices,
                                          void *values);
aclsparseStatus_t aclsparseDestroySpMat(aclsparseConstSpMatDescr_t spMatDescr);
aclsparseStatus_t aclsparseSpMatGetFormat(aclsparseConstSpMatDescr_t spMatDescr, aclsparseFormat_t *format);
aclsparseStatus_t aclsparseSpMatGetValues(aclsparseSpMatDescr_t spMatDescr, void **values);
aclsparseStatus_t aclsparseConstSpMatGetValues(aclsparseConstSpMatDescr_t spMatDescr, const void **values);
aclsparseStatus_t aclsparseSpMatSetValues(aclsparseSpMatDescr_t spMatDescr, void *values);
aclsparseStatus_t aclsparseSpMatGetSize(aclsparseConstSpMatDescr_t spMatDescr, int64_t *rows, int64_t *cols,
                                        int64_t *nnz);

/* ======================================================================================
 * Dense matrix descriptor (reference :551-614; aclsparse_descr.cpp:588-743).
 * rows, cols, ld > 0 and values != NULL are required; ld >= cols (row-major) or
 * ld >= rows (column-major).  DestroyDnMat(NULL) is INVALID_VALUE.
 * ====================================================================================== */
aclsparseStatus_t aclsparseCreateDnMat(aclsparseDnMatDescr_t *dnMatDescr, int64_t rows, int64_t cols, int64_t ld,
                                       void *values, aclDataType valueType, aclsparseOrder_t order);
aclsparseStatus_t aclsparseCreateConstDnMat(aclsparseConstDnMatDescr_t *dnMatDescr, int64_t rows, int64_t cols,
                                            int64_t ld, const void *values, aclDataType valueType,
                                            aclsparseOrder_t order);
aclsparseStatus_t aclsparseDestroyDnMat(aclsparseConstDnMatDescr_t dnMatDescr);
aclsparseStatus_t aclsparseDnMatGet(aclsparseDnMatDescr_t dnMatDescr, int64_t *rows, int64_t *cols, int64_t *ld,
                                    void **values, aclDataType *valueType, aclsparseOrder_t *order);
aclsparseStatus_t aclsparseConstDnMatGet(aclsparseConstDnMatDescr_t dnMatDescr, int64_t *rows, int64_t *cols,
                                         int64_t *ld, const void **values, aclDataType *valueType,
                                         aclsparseOrder_t *order);
aclsparseStatus_t aclsparseDnMatGetValues(aclsparseDnMatDescr_t dnMatDescr, void **values);
aclsparseStatus_t aclsparseConstDnMatGetValues(aclsparseConstDnMatDescr_t dnMatDescr, const void **values);
aclsparseStatus_t aclsparseDnMatSetValues(aclsparseDnMatDescr_t dnMatDescr, void *values);

/* ======================================================================================
 * SpMV:  y = alpha * op(A) * x + beta * y        (reference :490-533;
 * host logic sparse/spmv/arch22/spmv_host.cpp:121-295).
 *
 * Type rules: x has A's value type; (A/x, y, compute) is one of
 *   (f32,f32,f32) (f16,f16|f32,f32) (bf16,bf16|f32,f32) (i32,i32,i32) (i32,f32,f32).
 * alpha / beta point to a float or int32 (by computeType); NULL means alpha = 1, beta = 0.
 * They are read on the host in HOST pointer mode and by the kernel in DEVICE pointer mode.
 * x.size >= cols and y.size >= rows (swapped for op = TRANSPOSE).
 *
 * The reference declares GetBufferSize / Preprocess but ships no definition; here
 * they exist.  Preprocess fills `externalBuffer` (>= GetBufferSize bytes) with the
 * row-length analysis for A's sparsity pattern and records it as A's active buffer; a
 * later SpMV given the same buffer reuses it.  SpMV with externalBuffer == NULL runs the
 * analysis in the handle workspace on every call.  All three enqueue on the handle's
 * stream and return without synchronising.
 * ====================================================================================== */
aclsparseStatus_t aclsparseSpMVGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                             const void *beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                             aclsparseSpMVAlg_t alg, size_t *bufferSize);
aclsparseStatus_t aclsparseSpMVPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                          aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                          const void *beta, aclsparseDnVecDescr_t vecY, aclDataType computeType,
                                          aclsparseSpMVAlg_t alg, void *externalBuffer);
aclsparseStatus_t aclsparseSpMV(aclsparseHandle_t handle, aclsparseOperation_t opA, const void *alpha,
                                aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX, const void *beta,
                                aclsparseDnVecDescr_t vecY, aclDataType computeType, aclsparseSpMVAlg_t alg,
                                void *externalBuffer);

/* ======================================================================================
 * SpMM:  C = alpha * A * op(B) + beta * C        (reference :682-704;
 * host logic sparse/spmm/arch35/spmm_host.cpp:152-394).
 *
 * opA = NON_TRANSPOSE only; opB in {N, T}; B and C row- or column-major with ld.
 * (A, B, C, compute) is one of (f32,f32,f32,f32) (f16,f16,f16,f32) (i8,i8,i32,i32), plus
 * the B200 extension (bf16,bf16,f32|bf16,f32).  NULL alpha / beta read as 0.
 * `buffer` must hold GetBufferSize bytes; NULL is INSUFFICIENT_RESOURCES.  SpMM on a
 * buffer that is not A's active buffer re-runs the analysis into it first.
 * ====================================================================================== */
aclsparseStatus_t aclsparseSpMMGetBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseOperation_t opB, const void *alpha,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                             const void *beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                             aclsparseSpMMAlg_t alg, size_t *size);
aclsparseStatus_t aclsparseSpMMPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                          aclsparseOperation_t opB, const void *alpha,
                                          aclsparseConstSpMatDescr_t matA, aclsparseConstDnMatDescr_t matB,
                                          const void *beta, aclsparseDnMatDescr_t matC, aclDataType computeType,
                                          aclsparseSpMMAlg_t alg, void *buffer);
aclsparseStatus_t aclsparseSpMM(aclsparseHandle_t handle, aclsparseOperation_t opA, aclsparseOperation_t opB,
                                const void *alpha, aclsparseConstSpMatDescr_t matA,
                                aclsparseConstDnMatDescr_t matB, const void *beta, aclsparseDnMatDescr_t matC,
                                aclDataType computeType, aclsparseSpMMAlg_t alg, void *buffer);

/* ---- SpMVOp plan API: Z = alpha * A * X + beta * Y (reference include/cann_ops_sparse.h:1564-1637,
 * sparse/spmv_op/arch35/spmv_op_host.cpp:496-745).  fp32 only, opA = NON_TRANSPOSE only, CSR with int32
 * column indices, int32 or int64 row offsets, index base 0 or 1; X has exactly cols entries, Y and Z
 * exactly rows; Z may be Y.  Every row is summed with the doubly compensated dot product of the
 * reference kernel (spmv_op_kernel.cpp:88-127) on a fixed reduction shape, so results are reproducible
 * bit for bit.  alpha and beta are required and follow the handle's pointer mode; with beta == 0, Y is
 * not read.  The epilogue arguments exist for signature compatibility: a non-NULL epilogue buffer is
 * NOT_SUPPORTED, setGlobalUserData checks its arguments and does nothing. ---- */
aclsparseStatus_t aclsparseSpMVOp_bufferSize(aclsparseHandle_t handle, aclsparseOperation_t opA,
                                             aclsparseConstSpMatDescr_t matA, aclsparseConstDnVecDescr_t vecX,
                                             aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ,
                                             aclDataType computeType, aclsparseSpMVOpAlg_t alg, size_t *bufferSize);
aclsparseStatus_t aclsparseSpMVOp_createDescr(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t *descr,
                                              aclsparseOperation_t opA, aclsparseConstSpMatDescr_t matA,
                                              aclsparseConstDnVecDescr_t vecX, aclsparseConstDnVecDescr_t vecY,
                                              aclsparseDnVecDescr_t vecZ, aclDataType computeType,
                                              aclsparseSpMVOpAlg_t alg, void *buffer);
aclsparseStatus_t aclsparseSpMVOp_destroyDescr(aclsparseSpMVOpDescr_t descr);
aclsparseStatus_t aclsparseSpMVOp_createPlan(aclsparseHandle_t handle, aclsparseSpMVOpDescr_t descr,
                                             aclsparseSpMVOpPlan_t *plan, const void *epilogueLTOBuffer,
                                             size_t epilogueLTOBufferSize);
aclsparseStatus_t aclsparseSpMVOp_destroyPlan(aclsparseSpMVOpPlan_t plan);
aclsparseStatus_t aclsparseSpMVOp_setGlobalUserData(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan,
                                                    const char *epilogueDataName, void *epilogueData,
                                                    size_t epilogueDataSize);
aclsparseStatus_t aclsparseSpMVOp(aclsparseHandle_t handle, aclsparseSpMVOpPlan_t plan, const void *alpha,
                                  const void *beta, aclsparseConstDnVecDescr_t vecX,
                                  aclsparseConstDnVecDescr_t vecY, aclsparseDnVecDescr_t vecZ);

/* ---- COO row indices -> CSR row offsets (reference include/cann_ops_sparse.h:1796-1822,
 * sparse/coo2csr/arch35/coo2csr_host.cpp:38-78).  cooRowInd[0..nnz) is sorted non-decreasing, DEVICE;
 * csrRowPtr[0..m] is written, DEVICE; both carry the index base.  The step before the products in
 * pipelines that assemble A as triplets. ---- */
aclsparseStatus_t aclsparseXcoo2csr(aclsparseHandle_t handle, const int *cooRowInd, int nnz, int m, int *csrRowPtr,
                                    aclsparseIndexBase_t idxBase);

/* ---- Legacy matrix descriptor (reference include/cann_ops_sparse.h:906-919,
 * sparse/common/aclsparse_matdescr.cpp:25-108): setters ignore a NULL descriptor, getters return the
 * default for one. ---- */
aclsparseStatus_t aclsparseCreateMatDescr(aclsparseMatDescr_t *descr);
aclsparseStatus_t aclsparseDestroyMatDescr(aclsparseMatDescr_t descr);
void aclsparseSetMatType(aclsparseMatDescr_t descr, aclsparseMatrixType_t type);
void aclsparseSetMatIndexBase(aclsparseMatDescr_t descr, aclsparseIndexBase_t base);
void aclsparseSetMatDiagType(aclsparseMatDescr_t descr, aclsparseDiagType_t diagType);
void aclsparseSetMatFillMode(aclsparseMatDescr_t descr, aclsparseFillMode_t fillMode);
aclsparseMatrixType_t aclsparseGetMatType(aclsparseMatDescr_t descr);
aclsparseIndexBase_t aclsparseGetMatIndexBase(aclsparseMatDescr_t descr);
aclsparseDiagType_t aclsparseGetMatDiagType(aclsparseMatDescr_t descr);
aclsparseFillMode_t aclsparseGetMatFillMode(aclsparseMatDescr_t descr);

/* ---- Stable sort of the column indices inside every CSR row, permutation P carried along (reference
 * include/cann_ops_sparse.h:1664-1711, sparse/csrsort/arch35/csrsort_host.cpp:146-222).  csrRowPtr,
 * csrColInd, P and pBuffer are DEVICE pointers; P is permuted like csrColInd (pass the identity to get
 * the gather indices for the values).  Only descrA's index base is used.  The workspace is larger than
 * the reference's 8 bytes per entry (the library sort's own storage comes on top). ---- */
aclsparseStatus_t aclsparseXcsrsort_bufferSizeExt(aclsparseHandle_t handle, int m, int n, int nnz, const int *csrRowPtr,
                                                  const int *csrColInd, size_t *pBufferSizeInBytes);
aclsparseStatus_t aclsparseXcsrsort(aclsparseHandle_t handle, int m, int n, int nnz, const aclsparseMatDescr_t descrA,
                                    const int *csrRowPtr, int *csrColInd, int *P, void *pBuffer);

/* ---- CSR -> CSC (reference include/cann_ops_sparse.h:1366-1440,
 * sparse/csr2csc_ex2/arch35/csr2csc_ex2_host.cpp:106-232, 539-640).  m x n matrix; all array arguments are
 * DEVICE pointers; values are int8, fp16, bf16 or fp32 (copied as bytes); entries of one column keep their
 * row order; with SYMBOLIC, cscVal is not written.  bufferSize ignores its array arguments.  The workspace is
 * 12 bytes per entry plus the library sort's own storage (the reference needs a few offsets arrays). ---- */
aclsparseStatus_t aclsparseCsr2cscEx2_bufferSize(aclsparseHandle_t handle, int m, int n, int nnz, const void *csrVal,
                                                 const int *csrRowPtr, const int *csrColInd, void *cscVal,
                                                 int *cscColPtr, int *cscRowInd, aclDataType valType,
                                                 aclsparseAction_t copyValues, aclsparseIndexBase_t idxBase,
                                                 aclsparseCsr2CscAlg_t alg, size_t *bufferSize);
aclsparseStatus_t aclsparseCsr2cscEx2(aclsparseHandle_t handle, int m, int n, int nnz, const void *csrVal,
                                      const int *csrRowPtr, const int *csrColInd, void *cscVal, int *cscColPtr,
                                      int *cscRowInd, aclDataType valType, aclsparseAction_t copyValues,
                                      aclsparseIndexBase_t idxBase, aclsparseCsr2CscAlg_t alg, void *buffer);

/* ---- SDDMM: C = (alpha * op(X) * op(Y) + beta * C) on the pattern of C, values of C updated in place
 * (reference include/cann_ops_sparse.h:706-745, sparse/sddmm/arch35/sddmm_host.cpp:145-320, 478-764).  op(X) is
 * m x k, op(Y) is k x n, C is m x n CSR with int32 zero-based indices; (X, Y, C, compute) all fp32 or all fp16
 * (fp32 accumulation, result saturated to +-65504 before rounding); alpha / beta have the compute type.  The
 * buffer must not be NULL; nothing is kept in it. ---- */
aclsparseStatus_t aclsparseSDDMMBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opX, aclsparseOperation_t opY,
                                           const void *alpha, aclsparseConstDnMatDescr_t matX,
                                           aclsparseConstDnMatDescr_t matY, const void *beta, aclsparseSpMatDescr_t matC,
                                           aclDataType computeType, aclsparseSDDMMAlg_t alg, size_t *size);
aclsparseStatus_t aclsparseSDDMMPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opX, aclsparseOperation_t opY,
                                           const void *alpha, aclsparseConstDnMatDescr_t matX,
                                           aclsparseConstDnMatDescr_t matY, const void *beta, aclsparseSpMatDescr_t matC,
                                           aclDataType computeType, aclsparseSDDMMAlg_t alg, void *buffer);
aclsparseStatus_t aclsparseSDDMM(aclsparseHandle_t handle, aclsparseOperation_t opX, aclsparseOperation_t opY,
                                 const void *alpha, aclsparseConstDnMatDescr_t matX, aclsparseConstDnMatDescr_t matY,
                                 const void *beta, aclsparseSpMatDescr_t matC, aclDataType computeType,
                                 aclsparseSDDMMAlg_t alg, void *buffer);

#ifdef __cplusplus
}
#endif

#endif /* CANN_OPS_SPARSE_H_ */
