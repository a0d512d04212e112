// aclsparseCsr2cscEx2: CSR -> CSC (the transpose's CSR), structure and optionally values.
// Checks, their order and status codes follow the reference host layer
// (sparse/csr2csc_ex2/arch35/csr2csc_ex2_host.cpp:44-57, 106-232, 255-288, 539-640).
// Entries of one column keep their row order (the reference scatters stripes in ascending entry order for
// the same reason), so the result is unique and the tests compare it bit for bit.
//
// Here: a stable key-value radix sort of (column, entry index) -- CUB's device radix sort, a library
// routine: this converter is off the SpMV / SpMM hot path -- then three small kernels: column offsets by
// binary search in the sorted columns, the row of every entry by binary search in the CSR row offsets,
// and the gather of the values through the permutation.  A CSC copy of A gives y = A^T x without
// atomics: aclsparseSpMV (non-transposed) on the CSC arrays read as CSR.
#include <climits>
#include <cstdint>

#include <cub/device/device_radix_sort.cuh>
#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "common/internal.h"

namespace {

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

int ValueBytes(aclDataType t)  // csr2csc_ex2_host.cpp:44-57
{
    switch (t) {
        case ACL_INT8: return 1;
        case ACL_FLOAT16:
        case ACL_BF16: return 2;
        case ACL_FLOAT: return 4;
        default: return 0;
    }
}

aclsparseStatus_t ValidateCommon(aclsparseHandle_t handle, int m, int n, int nnz, aclDataType valType,
                                 aclsparseAction_t copyValues, aclsparseIndexBase_t idxBase, aclsparseCsr2CscAlg_t alg)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    if (m < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (n < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (n > INT32_MAX - 1) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (ValueBytes(valType) == 0) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (copyValues != ACL_SPARSE_ACTION_SYMBOLIC && copyValues != ACL_SPARSE_ACTION_NUMERIC)
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (idxBase != ACL_SPARSE_INDEX_BASE_ZERO && idxBase != ACL_SPARSE_INDEX_BASE_ONE)
        return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (alg != ACL_SPARSE_CSR2CSC_ALG_DEFAULT && alg != ACL_SPARSE_CSR2CSC_ALG1) return ACL_SPARSE_STATUS_INVALID_VALUE;
    return ACL_SPARSE_STATUS_SUCCESS;
}

struct Layout {
    size_t offIota, offKeys, offPerm, offTemp, total;
};
Layout LayoutFor(int nnz, size_t tempBytes)
{
    const size_t arr = AlignUp(sizeof(int32_t) * (size_t)nnz, 256);
    Layout L;
    L.offIota = 0;
    L.offKeys = arr;
    L.offPerm = 2 * arr;
    L.offTemp = 3 * arr;
    L.total = 3 * arr + AlignUp(tempBytes, 256);
    return L;
}

cudaError_t SortCall(void *temp, size_t &tempBytes, const int *keysIn, int *keysOut, const int *valsIn, int *valsOut,
                     int nnz, int n, cudaStream_t st)
{
    int bits = 1;  // column indices (with the base) are below n + 1
    while (bits < 31 && (1ll << bits) <= (long long)n + 1) ++bits;
    return cub::DeviceRadixSort::SortPairs(temp, tempBytes, keysIn, keysOut, valsIn, valsOut, nnz, 0, bits, st);
}

__global__ void IotaKernel(int *out, int n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = (int)i;
}

// out[i] = base + |{k : sorted[k] < i + base}| for i = 0..n: the offsets of the runs of equal keys.
__global__ void RunOffsetsKernel(const int *__restrict__ sorted, int nnz, int n, int *__restrict__ out, int base)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i <= n; i += (long long)gridDim.x * blockDim.x) {
        const int key = (int)i + base;
        int lo = 0, hi = nnz;
        while (lo < hi) {
            const int mid = lo + ((hi - lo) >> 1);
            if (__ldg(sorted + mid) < key) lo = mid + 1;
            else hi = mid;
        }
        out[i] = lo + base;
    }
}

// cscRowInd[k] = row that holds entry perm[k]; cscVal[k] = csrVal[perm[k]] (kBytes per value, 0 = no values).
template <int kBytes>
__global__ void GatherKernel(const int *__restrict__ perm, const int *__restrict__ csrRowPtr, int m, int base,
                             const void *__restrict__ csrVal, int nnz, int *__restrict__ cscRowInd,
                             void *__restrict__ cscVal)
{
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += (long long)gridDim.x * blockDim.x) {
        const int p = perm[k];
        int lo = 0, hi = m - 1;  // largest r with csrRowPtr[r] - base <= p
        while (lo < hi) {
            const int mid = lo + ((hi - lo + 1) >> 1);
            if (__ldg(csrRowPtr + mid) - base <= p) lo = mid;
            else hi = mid - 1;
        }
        cscRowInd[k] = lo + base;
        if constexpr (kBytes == 1) static_cast<uint8_t *>(cscVal)[k] = static_cast<const uint8_t *>(csrVal)[p];
        if constexpr (kBytes == 2) static_cast<uint16_t *>(cscVal)[k] = static_cast<const uint16_t *>(csrVal)[p];
        if constexpr (kBytes == 4) static_cast<uint32_t *>(cscVal)[k] = static_cast<const uint32_t *>(csrVal)[p];
    }
}

unsigned Blocks(long long items)
{
    const long long want = (items + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 32;
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace

extern "C" {

aclsparseStatus_t aclsparseCsr2cscEx2_bufferSize(aclsparseHandle_t handle, int m, int n, int nnz, const void *csrVal,
                                                 const int *csrRowPtr, const int *csrColInd, void *cscVal,
                                                 int *cscColPtr, int *cscRowInd, aclDataType valType,
                                                 aclsparseAction_t copyValues, aclsparseIndexBase_t idxBase,
                                                 aclsparseCsr2CscAlg_t alg, size_t *bufferSize)
{
    (void)csrVal; (void)csrRowPtr; (void)csrColInd; (void)cscVal; (void)cscColPtr; (void)cscRowInd;
    const aclsparseStatus_t st = ValidateCommon(handle, m, n, nnz, valType, copyValues, idxBase, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (bufferSize == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (m == 0 || n == 0 || nnz == 0) {
        *bufferSize = 0;
        return ACL_SPARSE_STATUS_SUCCESS;
    }
    size_t tempBytes = 0;  // a size query: nothing is launched
    const cudaError_t e = SortCall(nullptr, tempBytes, nullptr, nullptr, nullptr, nullptr, nnz, n, nullptr);
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseCsr2cscEx2_bufferSize: size query failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    *bufferSize = LayoutFor(nnz, tempBytes).total;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCsr2cscEx2(aclsparseHandle_t handle, int m, int n, int nnz, const void *csrVal,
                                      const int *csrRowPtr, const int *csrColInd, void *cscVal, int *cscColPtr,
                                      int *cscRowInd, aclDataType valType, aclsparseAction_t copyValues,
                                      aclsparseIndexBase_t idxBase, aclsparseCsr2CscAlg_t alg, void *buffer)
{
    aclsparseStatus_t st = ValidateCommon(handle, m, n, nnz, valType, copyValues, idxBase, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    const bool numeric = copyValues == ACL_SPARSE_ACTION_NUMERIC;
    // csr2csc_ex2_host.cpp:200-232
    if (m > 0 && csrRowPtr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && csrColInd == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && numeric && csrVal == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (cscColPtr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && cscRowInd == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && numeric && cscVal == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (m == 0 && nnz > 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (n == 0 && nnz > 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const int base = idxBase == ACL_SPARSE_INDEX_BASE_ONE ? 1 : 0;
    if (nnz > INT32_MAX - base) return ACL_SPARSE_STATUS_INVALID_VALUE;

    cudaStream_t stream = handle->stream;
    if (nnz == 0) {  // every column is empty: n + 1 offsets equal to the base
        RunOffsetsKernel<<<Blocks((long long)n + 1), 256, 0, stream>>>(nullptr, 0, n, cscColPtr, base);
        b200sp_note_launches(1);
        return cudaGetLastError() == cudaSuccess ? ACL_SPARSE_STATUS_SUCCESS : ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (buffer == nullptr) return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;  // csr2csc_ex2_host.cpp:298-310

    size_t tempBytes = 0;
    cudaError_t e = SortCall(nullptr, tempBytes, nullptr, nullptr, nullptr, nullptr, nnz, n, stream);
    if (e != cudaSuccess) return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    const Layout L = LayoutFor(nnz, tempBytes);
    char *p = static_cast<char *>(buffer);
    int *iota = reinterpret_cast<int *>(p + L.offIota);
    int *keys = reinterpret_cast<int *>(p + L.offKeys);
    int *perm = reinterpret_cast<int *>(p + L.offPerm);
    IotaKernel<<<Blocks(nnz), 256, 0, stream>>>(iota, nnz);
    e = SortCall(p + L.offTemp, tempBytes, csrColInd, keys, iota, perm, nnz, n, stream);
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseCsr2cscEx2: sort failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    RunOffsetsKernel<<<Blocks((long long)n + 1), 256, 0, stream>>>(keys, nnz, n, cscColPtr, base);
    const int bytes = numeric ? ValueBytes(valType) : 0;
    const unsigned g = Blocks(nnz);
    switch (bytes) {
        case 1: GatherKernel<1><<<g, 256, 0, stream>>>(perm, csrRowPtr, m, base, csrVal, nnz, cscRowInd, cscVal); break;
        case 2: GatherKernel<2><<<g, 256, 0, stream>>>(perm, csrRowPtr, m, base, csrVal, nnz, cscRowInd, cscVal); break;
        case 4: GatherKernel<4><<<g, 256, 0, stream>>>(perm, csrRowPtr, m, base, csrVal, nnz, cscRowInd, cscVal); break;
        default: GatherKernel<0><<<g, 256, 0, stream>>>(perm, csrRowPtr, m, base, nullptr, nnz, cscRowInd, nullptr); break;
    }
    b200sp_note_launches(3);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseCsr2cscEx2: kernel launch failed (%s)", cudaGetErrorString(e));
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
