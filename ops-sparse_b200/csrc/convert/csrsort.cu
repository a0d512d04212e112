// aclsparseXcsrsort: stable in-place sort of the column indices of every CSR row, with the permutation P
// carried along; and the legacy matrix descriptor it takes its index base from.
// Checks, their order and status codes follow the reference host layer
// (sparse/csrsort/arch35/csrsort_host.cpp:52-74, 146-222; sparse/common/aclsparse_matdescr.cpp:25-108).
// The sort: every entry becomes a 64-bit key (column in the high word, position inside its row in the low word),
// which makes keys unique and the ascending order of keys exactly the stable order the golden defines
// (test/csrsort/arch35/csrsort_golden.h:38-70); the rows are then sorted by the segmented sort of segsort.cuh
// (registers for rows of up to 32 entries, shared memory up to 2048, chunk sort + merge passes beyond), and a last
// pass splits the keys again: the high word is the sorted column, the low word says which entry of P moves here.
// Workspace: 8 bytes per entry for the keys, 8 for the merge scratch (whose first half also holds the permuted P
// until it is copied back) and a list of the rows too long for a warp.
#include <cstdint>
#include <limits>
#include <new>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "common/internal.h"
#include "convert/segsort.cuh"

struct aclsparseMatDescr {  // aclsparse_descr_internal.h:131-136
    aclsparseMatrixType_t type = ACL_SPARSE_MATRIX_TYPE_GENERAL;
    aclsparseIndexBase_t indexBase = ACL_SPARSE_INDEX_BASE_ZERO;
    aclsparseDiagType_t diagType = ACL_SPARSE_DIAG_TYPE_NON_UNIT;
    aclsparseFillMode_t fillMode = ACL_SPARSE_FILL_MODE_LOWER;
};

namespace {

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

aclsparseStatus_t ValidateCommon(int m, int n, int nnz, const int *csrRowPtr, const int *csrColInd)
{
    if (m < 0 || n < 0 || nnz < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if ((m == 0 || n == 0) && nnz != 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (m > 0 && csrRowPtr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && csrColInd == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    return ACL_SPARSE_STATUS_SUCCESS;
}

struct SortLayout {
    size_t offKeys, offScratch, offList, total;
};
SortLayout SortLayoutFor(int m, int nnz)
{
    SortLayout L;
    const size_t keys = AlignUp(sizeof(unsigned long long) * (size_t)nnz, 256);
    L.offKeys = 0;
    L.offScratch = keys;
    L.offList = 2 * keys;
    L.total = 2 * keys + b200sp_segsort::ListBytes(m);
    return L;
}

// A warp per row: keys[e] = column << 32 | (e - row start).
__global__ void __launch_bounds__(256) CsrsortPackKernel(const int *__restrict__ rowPtr, const int *__restrict__ colInd,
                                                         int m, int base, unsigned long long *__restrict__ keys)
{
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < m; r += warpsTotal) {
        const int a = rowPtr[r] - base, b = rowPtr[r + 1] - base;
        for (int e = a + lane; e < b; e += 32)
            keys[e] = ((unsigned long long)(unsigned)colInd[e] << 32) | (unsigned)(e - a);
    }
}

// A warp per row: colInd[e] = high word of keys[e]; permuted[e] = P[row start + low word].
__global__ void __launch_bounds__(256) CsrsortUnpackKernel(const int *__restrict__ rowPtr, int m, int base,
                                                           const unsigned long long *__restrict__ keys,
                                                           int *__restrict__ colInd, const int *__restrict__ P,
                                                           int *__restrict__ permuted)
{
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < m; r += warpsTotal) {
        const int a = rowPtr[r] - base, b = rowPtr[r + 1] - base;
        for (int e = a + lane; e < b; e += 32) {
            const unsigned long long k = keys[e];
            colInd[e] = (int)(unsigned)(k >> 32);
            permuted[e] = P[a + (int)(unsigned)(k & 0xffffffffu)];
        }
    }
}

unsigned WarpRowBlocks(int m)
{
    const long long want = ((long long)m + 7) / 8;
    const long long cap = (long long)b200sp_sm_count() * 32;
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
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
    *pBufferSizeInBytes = SortLayoutFor(m, nnz).total;  // computed from the sizes alone: nothing is read
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
    const SortLayout L = SortLayoutFor(m, nnz);
    char *w = static_cast<char *>(pBuffer);
    auto *keys = reinterpret_cast<unsigned long long *>(w + L.offKeys);
    auto *scratch = reinterpret_cast<unsigned long long *>(w + L.offScratch);
    auto *list = reinterpret_cast<int *>(w + L.offList);
    const int b = base == ACL_SPARSE_INDEX_BASE_ONE ? 1 : 0;
    CsrsortPackKernel<<<WarpRowBlocks(m), 256, 0, stream>>>(csrRowPtr, csrColInd, m, b, keys);
    b200sp_note_launches(1);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = b200sp_segsort::Sort(csrRowPtr, b, m, keys, scratch, list, stream);
    if (e == cudaSuccess) {
        // the merge scratch is free again: its first half takes the permuted P until it is copied over P
        int *permuted = reinterpret_cast<int *>(scratch);
        CsrsortUnpackKernel<<<WarpRowBlocks(m), 256, 0, stream>>>(csrRowPtr, m, b, keys, csrColInd, P, permuted);
        b200sp_note_launches(1);
        e = cudaGetLastError();
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(P, permuted, sizeof(int) * (size_t)nnz, cudaMemcpyDeviceToDevice, stream);
    }
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseXcsrsort: sort failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
