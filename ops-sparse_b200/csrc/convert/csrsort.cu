// aclsparseXcsrsort: stable in-place sort of the column indices of every CSR row, with the permutation P
// carried along; and the legacy matrix descriptor it takes its index base from.
// Checks, their order and status codes follow the reference host layer
// (sparse/csrsort/arch35/csrsort_host.cpp:52-74, 146-222; sparse/common/aclsparse_matdescr.cpp:25-108).
// The sort: every entry becomes a 64-bit key (column in the high word, position inside its row in the low word),
// which makes keys unique and the ascending order of keys exactly the stable order the golden defines
// (test/csrsort/arch35/csrsort_golden.h:38-70); the rows are sorted by the segmented sort of segsort.cuh
// (registers for rows of up to 256 entries, shared memory up to 2048, chunk sort + merge passes beyond), which
// forms the keys while it loads a row and splits them while it stores it: the high word is the sorted column, the
// low word says which entry of P moves here.  Two launches, no pass of its own over the arrays.
// Workspace: 8 bytes per entry for the keys and 8 for the merge scratch (both touched only for rows of more than
// 2048 entries) and a list of the rows too long for a warp.
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

// How the sort reads and writes this operator's arrays: the key of entry i of a row is (column << 32 | i), made on
// the fly from csrColInd; a sorted key puts its high word back into csrColInd and moves P[row start + low word] to
// its place (read for the whole row before any of it is written: the sort is in place in both arrays).
struct CsrsortIo {
    int *colInd;
    int *P;
    using Payload = int;
    __device__ __forceinline__ unsigned long long Load(int a, int i) const
    {
        return ((unsigned long long)(unsigned)colInd[a + i] << 32) | (unsigned)i;
    }
    __device__ __forceinline__ int Fetch(int a, unsigned long long key) const { return P[a + (int)(unsigned)(key & 0xffffffffu)]; }
    __device__ __forceinline__ void Commit(int a, int i, unsigned long long key, int moved) const
    {
        colInd[a + i] = (int)(unsigned)(key >> 32);
        P[a + i] = moved;
    }
    static __device__ __forceinline__ unsigned Pack(int v) { return (unsigned)v; }
    static __device__ __forceinline__ int Unpack(unsigned v) { return (int)v; }
};

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
    const cudaError_t e = b200sp_segsort::Sort(csrRowPtr, b, m, CsrsortIo{csrColInd, P}, keys, scratch, list, stream);
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseXcsrsort: sort failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
