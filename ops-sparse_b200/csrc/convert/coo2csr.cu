// aclsparseXcoo2csr: sorted COO row indices -> CSR row offsets.
// Checks and their order follow the reference host layer (sparse/coo2csr/arch35/coo2csr_host.cpp:38-78);
// the reference counts the entries of every row and prefix-sums the counts, which for the sorted input the
// API requires is the same as csrRowPtr[i] = base + |{k : cooRowInd[k] < i + base}|.  Here one thread per
// output looks that position up by binary search: one pass, no workspace, no atomics.
#include <climits>
#include <cstdint>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "common/internal.h"

namespace {

__global__ void Coo2CsrKernel(const int *__restrict__ cooRowInd, int nnz, int m, int *__restrict__ csrRowPtr,
                              int base)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i <= m;
         i += (long long)gridDim.x * blockDim.x) {
        const int key = (int)i + base;  // first entry whose row index is >= key
        int lo = 0, hi = nnz;
        while (lo < hi) {
            const int mid = lo + ((hi - lo) >> 1);
            if (__ldg(cooRowInd + mid) < key) lo = mid + 1;
            else hi = mid;
        }
        csrRowPtr[i] = lo + base;
    }
}

}  // namespace

extern "C" aclsparseStatus_t aclsparseXcoo2csr(aclsparseHandle_t handle, const int *cooRowInd, int nnz, int m,
                                               int *csrRowPtr, aclsparseIndexBase_t idxBase)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (nnz < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz == INT32_MAX && idxBase == ACL_SPARSE_INDEX_BASE_ONE) return ACL_SPARSE_STATUS_INVALID_VALUE;  // nnz + 1 overflows
    if (m < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && m == 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (idxBase != ACL_SPARSE_INDEX_BASE_ZERO && idxBase != ACL_SPARSE_INDEX_BASE_ONE)
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && cooRowInd == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (csrRowPtr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;

    const long long want = ((long long)m + 1 + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 32;
    Coo2CsrKernel<<<(unsigned)(want < cap ? want : cap), 256, 0, handle->stream>>>(
        cooRowInd, nnz, m, csrRowPtr, idxBase == ACL_SPARSE_INDEX_BASE_ONE ? 1 : 0);
    b200sp_note_launches(1);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseXcoo2csr: kernel launch failed (%s)", cudaGetErrorString(e));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}
