// aclsparseCsr2cscEx2: CSR -> CSC (the transpose's CSR), structure and optionally values.
// Checks, their order and status codes follow the reference host layer
// (sparse/csr2csc_ex2/arch35/csr2csc_ex2_host.cpp:44-57, 106-232, 255-288, 539-640).
// Entries of one column keep their row order (the golden drops them into their columns row by row,
// test/csr2csc_ex2/csr2csc_ex2_golden.h:50-110), so the result is unique and the tests compare it bit for bit.
//
// Here, with kernels of this library only:
//   1. a histogram of the columns (one atomic add per entry) into cscColPtr;
//   2. an exclusive scan of it (block sums, a one-CTA scan of the sums, a second sweep) -> the column offsets;
//   3. every entry is dropped into SOME free slot of its column (an atomic cursor per column) as a 64-bit key:
//      entry index in the high word, row in the low word;
//   4. every column segment is sorted by that key (segsort.cuh): ascending entry index IS the golden's order,
//      whatever order the atomics produced; while a sorted segment is stored, its keys are split again: row index
//      from the low word, value fetched through the high word.
// A CSC copy of A gives y = A^T x without atomics: aclsparseSpMV (non-transposed) on the CSC arrays read as CSR.
#include <climits>
#include <cstdint>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "common/internal.h"
#include "convert/segsort.cuh"

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
    size_t offKeys, offScratch, offCursor, offSums, offList, total;
};
constexpr int kScanBlock = 1024;  // counts one CTA scans in one sweep
Layout LayoutFor(int n, int nnz)
{
    const size_t keys = AlignUp(sizeof(unsigned long long) * (size_t)nnz, 256);
    Layout L;
    L.offKeys = 0;
    L.offScratch = keys;
    L.offCursor = 2 * keys;
    L.offSums = L.offCursor + AlignUp(sizeof(int32_t) * ((size_t)n + 1), 256);
    L.offList = L.offSums + AlignUp(sizeof(int32_t) * ((size_t)n / kScanBlock + 2), 256);
    L.total = L.offList + b200sp_segsort::ListBytes(n);
    return L;
}

__global__ void FillKernel(int *out, long long count, int value)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        out[i] = value;
}

// counts[col] += 1 for every entry (counts has n + 1 slots, zeroed before; slot n stays 0)
__global__ void ColumnHistogramKernel(const int *__restrict__ colInd, int nnz, int base, int *__restrict__ counts)
{
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += (long long)gridDim.x * blockDim.x)
        atomicAdd(counts + (__ldg(colInd + k) - base), 1);
}

// Exclusive scan of count values in place, in three steps.  Step 1: the sum of every kScanBlock-wide block.
__global__ void __launch_bounds__(256) ScanBlockSumsKernel(const int *__restrict__ v, long long count, int *__restrict__ sums)
{
    __shared__ int sWarp[8];
    const long long b0 = (long long)blockIdx.x * kScanBlock;
    int acc = 0;
    for (int i = threadIdx.x; i < kScanBlock; i += 256)
        if (b0 + i < count) acc += v[b0 + i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) sWarp[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < 8; ++w) t += sWarp[w];
        sums[blockIdx.x] = t;
    }
}

// Inclusive scan of the calling CTA's 256 values (one per thread); returns this thread's inclusive prefix.
__device__ __forceinline__ int CtaInclusiveScan(int x, int *sWarp)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += t;
    }
    if (lane == 31) sWarp[warp] = x;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += sWarp[w];
    __syncthreads();
    return x + before;
}

// Step 2: exclusive scan of the block sums by one CTA, 256 at a time with a running carry.
__global__ void __launch_bounds__(256) ScanSumsKernel(int *__restrict__ sums, int blocks)
{
    __shared__ int sWarp[8];
    __shared__ int sCarry;
    if (threadIdx.x == 0) sCarry = 0;
    __syncthreads();
    for (int b0 = 0; b0 < blocks; b0 += 256) {
        const int i = b0 + threadIdx.x;
        const int x = i < blocks ? sums[i] : 0;
        const int incl = CtaInclusiveScan(x, sWarp);
        const int carry = sCarry;
        if (i < blocks) sums[i] = carry + incl - x;
        __syncthreads();
        if (threadIdx.x == 255) sCarry = carry + incl;
        __syncthreads();
    }
}

// Step 3: exclusive scan inside every block plus the block's offset; `plus` (the index base) is added to every
// result written to out, the zero-based result also goes to cursor (the next free slot of every column).
__global__ void __launch_bounds__(256) ScanApplyKernel(const int *__restrict__ v, long long count,
                                                       const int *__restrict__ sums, int plus, int *__restrict__ out,
                                                       int *__restrict__ cursor)
{
    __shared__ int sWarp[8];
    const long long b0 = (long long)blockIdx.x * kScanBlock;
    int carry = sums[blockIdx.x];
    for (int c = 0; c < kScanBlock; c += 256) {
        const long long i = b0 + c + threadIdx.x;
        const int x = i < count ? v[i] : 0;
        const int incl = CtaInclusiveScan(x, sWarp);
        if (i < count) {
            out[i] = carry + incl - x + plus;
            cursor[i] = carry + incl - x;
        }
        __shared__ int sTotal;
        if (threadIdx.x == 255) sTotal = incl;
        __syncthreads();
        carry += sTotal;
        __syncthreads();
    }
}

// Every entry takes the next free slot of its column and leaves (entry index, row) there.  A warp owns
// kScatterTile consecutive entries, whatever rows they belong to (a row of 16,384 entries is 16 warps' work, a
// thousand one-entry rows one warp's): the rows of its first and last entry are found by one search each, every
// entry's row by a search between the two.
constexpr int kScatterTile = 1024;
__device__ __forceinline__ int RowOfEntry(const int *__restrict__ rowPtr, int base, int lo, int hi, int e)
{
    while (lo < hi) {  // largest r in [lo, hi] with rowPtr[r] - base <= e
        const int mid = lo + ((hi - lo + 1) >> 1);
        if (rowPtr[mid] - base <= e) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}
__global__ void __launch_bounds__(256) ScatterKeysKernel(const int *__restrict__ rowPtr, const int *__restrict__ colInd,
                                                         int m, int nnz, int base, int *__restrict__ cursor,
                                                         unsigned long long *__restrict__ keys)
{
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    const long long tiles = ((long long)nnz + kScatterTile - 1) / kScatterTile;
    for (long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < tiles; t += warpsTotal) {
        const int e0 = (int)(t * kScatterTile);
        const int e1 = e0 + kScatterTile < nnz ? e0 + kScatterTile : nnz;
        int bound = 0;
        if (lane < 2) bound = RowOfEntry(rowPtr, base, 0, m - 1, lane == 0 ? e0 : e1 - 1);
        const int r0 = __shfl_sync(0xffffffffu, bound, 0), r1 = __shfl_sync(0xffffffffu, bound, 1);
        for (int e = e0 + lane; e < e1; e += 32) {
            const int r = RowOfEntry(rowPtr, base, r0, r1, e);
            const int slot = atomicAdd(cursor + (colInd[e] - base), 1);
            keys[slot] = ((unsigned long long)(unsigned)e << 32) | (unsigned)r;
        }
    }
}

// How the sort reads and writes this operator's arrays: the keys lie in the workspace; a sorted key gives its low
// word (the row) to cscRowInd and fetches the value of the entry its high word names (kBytes per value, 0 = none).
template <int kBytes>
struct Csr2cscIo {
    const unsigned long long *keys;
    int base;
    const void *csrVal;
    int *cscRowInd;
    void *cscVal;
    using Payload = unsigned;
    __device__ __forceinline__ unsigned long long Load(int a, int i) const { return keys[a + i]; }
    __device__ __forceinline__ unsigned Fetch(int, unsigned long long key) const
    {
        const unsigned p = (unsigned)(key >> 32);
        if constexpr (kBytes == 1) return static_cast<const uint8_t *>(csrVal)[p];
        if constexpr (kBytes == 2) return static_cast<const uint16_t *>(csrVal)[p];
        if constexpr (kBytes == 4) return static_cast<const uint32_t *>(csrVal)[p];
        return 0u;
    }
    __device__ __forceinline__ void Commit(int a, int i, unsigned long long key, unsigned value) const
    {
        cscRowInd[a + i] = (int)(unsigned)(key & 0xffffffffu) + base;
        if constexpr (kBytes == 1) static_cast<uint8_t *>(cscVal)[a + i] = (uint8_t)value;
        if constexpr (kBytes == 2) static_cast<uint16_t *>(cscVal)[a + i] = (uint16_t)value;
        if constexpr (kBytes == 4) static_cast<uint32_t *>(cscVal)[a + i] = value;
    }
    static __device__ __forceinline__ unsigned Pack(unsigned v) { return v; }
    static __device__ __forceinline__ unsigned Unpack(unsigned v) { return v; }
};

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
    *bufferSize = LayoutFor(n, nnz).total;  // from the sizes alone: nothing is launched
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
        FillKernel<<<Blocks((long long)n + 1), 256, 0, stream>>>(cscColPtr, (long long)n + 1, base);
        b200sp_note_launches(1);
        return cudaGetLastError() == cudaSuccess ? ACL_SPARSE_STATUS_SUCCESS : ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (buffer == nullptr) return ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES;  // csr2csc_ex2_host.cpp:298-310

    const Layout L = LayoutFor(n, nnz);
    char *p = static_cast<char *>(buffer);
    auto *keys = reinterpret_cast<unsigned long long *>(p + L.offKeys);
    auto *scratch = reinterpret_cast<unsigned long long *>(p + L.offScratch);
    int *cursor = reinterpret_cast<int *>(p + L.offCursor);
    int *sums = reinterpret_cast<int *>(p + L.offSums);
    int *list = reinterpret_cast<int *>(p + L.offList);
    const long long counts = (long long)n + 1;
    const int scanBlocks = (int)((counts + kScanBlock - 1) / kScanBlock);
    const long long scatterBlocks = (((long long)nnz + kScatterTile - 1) / kScatterTile + 7) / 8;
    const long long cap = (long long)b200sp_sm_count() * 32;
    cudaError_t e = cudaMemsetAsync(cscColPtr, 0, sizeof(int) * (size_t)counts, stream);
    if (e != cudaSuccess) return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    ColumnHistogramKernel<<<Blocks(nnz), 256, 0, stream>>>(csrColInd, nnz, base, cscColPtr);
    ScanBlockSumsKernel<<<(unsigned)scanBlocks, 256, 0, stream>>>(cscColPtr, counts, sums);
    ScanSumsKernel<<<1, 256, 0, stream>>>(sums, scanBlocks);
    ScanApplyKernel<<<(unsigned)scanBlocks, 256, 0, stream>>>(cscColPtr, counts, sums, base, cscColPtr, cursor);
    ScatterKeysKernel<<<(unsigned)(scatterBlocks < cap ? scatterBlocks : cap), 256, 0, stream>>>(
        csrRowPtr, csrColInd, m, nnz, base, cursor, keys);
    b200sp_note_launches(5);
    e = cudaGetLastError();
    if (e == cudaSuccess) {
        auto sort = [&]<int kBytes>() {
            return b200sp_segsort::Sort(cscColPtr, base, n, Csr2cscIo<kBytes>{keys, base, csrVal, cscRowInd, cscVal}, keys,
                                        scratch, list, stream);
        };
        switch (numeric ? ValueBytes(valType) : 0) {
            case 1: e = sort.template operator()<1>(); break;
            case 2: e = sort.template operator()<2>(); break;
            case 4: e = sort.template operator()<4>(); break;
            default: e = sort.template operator()<0>(); break;
        }
    }
    if (e != cudaSuccess) {
        B200SP_LOGE("aclsparseCsr2cscEx2: scatter or sort failed (%s)", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
