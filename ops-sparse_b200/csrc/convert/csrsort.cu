// aclsparseXcsrsort: stable in-place sort of the column indices of every CSR row, with the permutation P
// carried along; and the legacy matrix descriptor it takes its index base from.
// Checks, their order and status codes follow the reference host layer
// (sparse/csrsort/arch35/csrsort_host.cpp:52-74, 146-222; sparse/common/aclsparse_matdescr.cpp:25-108).
// The sort itself is CUB's segmented stable sort (a library routine: this converter is not on the SpMV /
// SpMM hot path, it prepares its input -- ascending columns are what lets the long-row SpMV kernel cut
// rows at the block boundaries of x).  Sorted keys and values land in the caller's workspace and are
// copied back; the workspace therefore holds 8 bytes per entry (what the reference asks for) plus CUB's
// own temporary storage.
#include <cstdint>
#include <limits>
#include <new>

#include <cub/device/device_segmented_sort.cuh>
#include <cub/iterator/counting_input_iterator.cuh>
#include <cub/iterator/transform_input_iterator.cuh>
#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "common/internal.h"

struct aclsparseMatDescr {  // aclsparse_descr_internal.h:131-136
    aclsparseMatrixType_t type = ACL_SPARSE_MATRIX_TYPE_GENERAL;
    aclsparseIndexBase_t indexBase = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseDiagType_t diagType = ACL_SPARSE_DIAG_TYPE_NON_UNIT;
    aclsparseFillMode_t fillMode = ACL_SPARSE_FILL_MODE_LOWER;
};

namespace {

struct MinusBase {  // row offsets with the index base taken off
    const int *p;
    int base;
    __host__ __device__ int operator()(int i) const { return p[i] - base; }
};
using OffsetIt = cub::TransformInputIterator<int, MinusBase, cub::CountingInputIterator<int>>;

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

aclsparseStatus_t ValidateCommon(int m, int n, int nnz, const int *csrRowPtr, const int *csrColInd)
{
    if (m < 0 || n < 0 || nnz < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if ((m == 0 || n == 0) && nnz != 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (m > 0 && csrRowPtr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && csrColInd == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    return ACL_SPARSE_STATUS_SUCCESS;
}

cudaError_t SortCall(void *temp, size_t &tempBytes, const int *keysIn, int *keysOut, const int *valsIn, int *valsOut,
                     int nnz, int m, const int *rowPtr, int base, cudaStream_t st)
{
    OffsetIt begin(cub::CountingInputIterator<int>(0), MinusBase{rowPtr, base});
    OffsetIt end(cub::CountingInputIterator<int>(1), MinusBase{rowPtr, base});
    return cub::DeviceSegmentedSort::StableSortPairs(temp, tempBytes, keysIn, keysOut, valsIn, valsOut, nnz, m, begin,
                                                     end, st);
}

}  // namespace

extern "C" {

aclsparseStatus_t aclsparseCreateMatDescr(aclsparseMatDescr_t *descr)
{
    if (descr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    auto *d = new (std::nothrow) aclsparseMatDescr();
    if (d == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;
    *descr = d;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDestroyMatDescr(aclsparseMatDescr_t descr)
{
    delete descr;  // NULL is accepted
    return ACL_SPARSE_STATUS_SUCCESS;
}

void aclsparseSetMatType(aclsparseMatDescr_t descr, aclsparseMatrixType_t type) { if (descr) descr->type = type; }
void aclsparseSetMatIndexBase(aclsparseMatDescr_t descr, aclsparseIndexBase_t base) { if (descr) descr->indexBase = base; }
void aclsparseSetMatDiagType(aclsparseMatDescr_t descr, aclsparseDiagType_t diagType) { if (descr) descr->diagType = diagType; }
void aclsparseSetMatFillMode(aclsparseMatDescr_t descr, aclsparseFillMode_t fillMode) { if (descr) descr->fillMode = fillMode; }
aclsparseMatrixType_t aclsparseGetMatType(aclsparseMatDescr_t descr) { return descr ? descr->type : ACL_SPARSE_MATRIX_TYPE_GENERAL; }
aclsparseIndexBase_t aclsparseGetMatIndexBase(aclsparseMatDescr_t descr) { return descr ? descr->indexBase : ACL_SPARSE_INDEX_BASE_ZERO; }
aclsparseDiagType_t aclsparseGetMatDiagType(aclsparseMatDescr_t descr) { return descr ? descr->diagType : ACL_SPARSE_DIAG_TYPE_NON_UNIT; }
aclsparseFillMode_t aclsparseGetMatFillMode(aclsparseMatDescr_t descr) { return descr ? descr->fillMode : ACL_SPARSE_FILL_MODE_LOWER; }

aclsparseStatus_t aclsparseXcsrsort_bufferSizeExt(aclsparseHandle_t handle, int m, int n, int nnz, const int *csrRowPtr,
                                                  const int *csrColInd, size_t *pBufferSizeInBytes)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (pBufferSizeInBytes == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const aclsparseStatus_t st = ValidateCommon(m, n, nnz, csrRowPtr, csrColInd);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (nnz == 0) {
        *pBufferSizeInBytes = 0;
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    size_t tempBytes = 0;  // a size query: nothing is launched, nothing is read
    const cudaError_t e = SortCall(nullptr, tempBytes, nullptr, nullptr, nullptr, nullptr, nnz, m, csrRowPtr, 0, nullptr);
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseXcsrsort_bufferSizeExt: size query failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    *pBufferSizeInBytes = 2 * AlignUp(sizeof(int32_t) * (size_t)nnz, 256) + AlignUp(tempBytes, 256);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseXcsrsort(aclsparseHandle_t handle, int m, int n, int nnz, const aclsparseMatDescr_t descrA,
                                    const int *csrRowPtr, int *csrColInd, int *P, void *pBuffer)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    const aclsparseStatus_t st = ValidateCommon(m, n, nnz, csrRowPtr, csrColInd);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (descrA == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const aclsparseIndexBase_t base = aclsparseGetMatIndexBase(descrA);
    if (base != ACL_SPARSE_INDEX_BASE_ZERO && base != ACL_SPARSE_INDEX_BASE_ONE) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz == 0) return ACL_SPARSE_STATUS_SUCCESS;
    if (P == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (pBuffer == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;

    cudaStream_t stream = handle->stream;
    const size_t half = AlignUp(sizeof(int32_t) * (size_t)nnz, 256);
    auto *keysOut = static_cast<int *>(pBuffer);
    auto *valsOut = reinterpret_cast<int *>(static_cast<char *>(pBuffer) + half);
    void *temp = static_cast<char *>(pBuffer) + 2 * half;
    size_t tempBytes = 0;
    const int b = base == ACL_SPARSE_INDEX_BASE_ONE ? 1 : 0;
    cudaError_t e = SortCall(nullptr, tempBytes, csrColInd, keysOut, P, valsOut, nnz, m, csrRowPtr, b, stream);
    if (e == cudaSuccess) e = SortCall(temp, tempBytes, csrColInd, keysOut, P, valsOut, nnz, m, csrRowPtr, b, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(csrColInd, keysOut, sizeof(int) * (size_t)nnz, cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(P, valsOut, sizeof(int) * (size_t)nnz, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseXcsrsort: sort failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
