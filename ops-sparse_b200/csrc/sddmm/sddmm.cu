// aclsparseSDDMM*: C = (alpha * op(X) * op(Y) + beta * C) sampled on the pattern of C (CSR, values in place).
// op(X) is m x k, op(Y) is k x n; fp32, or fp16 storage with fp32 accumulation and a saturating cast back
// (the reference's device arithmetic, sparse/sddmm/arch35/sddmm_kernel.cpp:26-27, 424-437).  Checks, their
// order and status codes follow the reference host layer (sparse/sddmm/arch35/sddmm_host.cpp:145-320, 478-510,
// 660-764).  The reference reorders rows greedily over its cores in Preprocess; here the work is cut by
// non-zeros (a warp per 32 consecutive entries of C, the lanes splitting k), which needs no analysis:
// BufferSize reports a token 256 bytes (the API wants a buffer), Preprocess only checks its arguments.
#include <climits>
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "common/internal.h"

namespace {

struct Strides {  // op(X)(i, kk) = X[i * xi + kk * xk];  op(Y)(kk, j) = Y[kk * yk + j * yj]
    long long xi, xk, yk, yj;
};

template <typename T> __device__ __forceinline__ float Load(const T *p);
template <> __device__ __forceinline__ float Load<float>(const float *p) { return __ldg(p); }
template <> __device__ __forceinline__ float Load<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <typename T> __device__ __forceinline__ T Store(float v);
template <> __device__ __forceinline__ float Store<float>(float v) { return v; }
template <> __device__ __forceinline__ __half Store<__half>(float v)
{
    return __float2half_rn(fminf(fmaxf(v, -65504.0f), 65504.0f));  // saturate, then round
}

template <typename T>
__global__ void __launch_bounds__(256) SddmmKernel(const int32_t *__restrict__ rowPtr, const int32_t *__restrict__ colInd,
                                                   T *__restrict__ cVal, const T *__restrict__ X,
                                                   const T *__restrict__ Y, int m, int k, long long nnz, Strides st,
                                                   float alpha, float beta, const T *alphaDev, const T *betaDev)
{
    const float a = alphaDev ? Load<T>(alphaDev) : alpha;
    const float b = betaDev ? Load<T>(betaDev) : beta;
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    const long long chunks = (nnz + 31) / 32;
    for (long long c = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < chunks; c += warpsTotal) {
        const long long p0 = c * 32;
        const long long p1 = p0 + 32 < nnz ? p0 + 32 : nnz;
        int lo = 0, hi = m - 1;  // row of entry p0: largest r with rowPtr[r] <= p0 (the same search in every lane)
        while (lo < hi) {
            const int mid = lo + ((hi - lo + 1) >> 1);
            if ((long long)__ldg(rowPtr + mid) <= p0) lo = mid;
            else hi = mid - 1;
        }
        int r = lo;
        for (long long p = p0; p < p1; ++p) {
            while ((long long)__ldg(rowPtr + r + 1) <= p) ++r;
            const int j = __ldg(colInd + p);
            const T *xr = X + (long long)r * st.xi;
            const T *yc = Y + (long long)j * st.yj;
            float acc = 0.0f;
            for (int kk = lane; kk < k; kk += 32) acc = fmaf(Load<T>(xr + kk * st.xk), Load<T>(yc + kk * st.yk), acc);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0) {
                float z = a * acc;
                if (b != 0.0f) z += b * Load<T>(cVal + p);
                cVal[p] = Store<T>(z);
            }
        }
    }
}

// 16 bytes of both operands per lane and step: 4 fp32 or 8 fp16 products.
__device__ __forceinline__ float Dot16(const uint4 &x, const uint4 &y, float acc, float)
{
    acc = fmaf(__uint_as_float(x.x), __uint_as_float(y.x), acc);
    acc = fmaf(__uint_as_float(x.y), __uint_as_float(y.y), acc);
    acc = fmaf(__uint_as_float(x.z), __uint_as_float(y.z), acc);
    return fmaf(__uint_as_float(x.w), __uint_as_float(y.w), acc);
}
__device__ __forceinline__ float Dot16(const uint4 &x, const uint4 &y, float acc, __half)
{
    const __half2 *hx = reinterpret_cast<const __half2 *>(&x);
    const __half2 *hy = reinterpret_cast<const __half2 *>(&y);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(hx[i]), b = __half22float2(hy[i]);
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
    }
    return acc;
}

// The same product when k runs along the contiguous direction of both operands and rows are 16-byte
// aligned: 128-bit loads.  The first 16-byte piece of the X row of every lane stays in registers while
// consecutive entries of C share their row (rows of up to 32 pieces -- 128 fp32 or 256 fp16 -- are then
// read once per row and chunk).
constexpr int kSddmmBatch = 4;  // entries of C a warp works on at once
template <typename T>
__global__ void __launch_bounds__(256) SddmmVecKernel(const int32_t *__restrict__ rowPtr, const int32_t *__restrict__ colInd,
                                                      T *__restrict__ cVal, const T *__restrict__ X,
                                                      const T *__restrict__ Y, int m, int pieces, long long nnz,
                                                      long long xRow16, long long yRow16, float alpha, float beta,
                                                      const T *alphaDev, const T *betaDev)
{
    const float a = alphaDev ? Load<T>(alphaDev) : alpha;
    const float b = betaDev ? Load<T>(betaDev) : beta;
    const int lane = threadIdx.x & 31;
    const uint4 *X16 = reinterpret_cast<const uint4 *>(X);
    const uint4 *Y16 = reinterpret_cast<const uint4 *>(Y);
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    const long long chunks = (nnz + 31) / 32;
    for (long long c = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < chunks; c += warpsTotal) {
        const long long p0 = c * 32;
        const long long p1 = p0 + 32 < nnz ? p0 + 32 : nnz;
        // The row of the chunk's first entry (largest r with rowPtr[r] <= p0): the 32 lanes probe 32 places
        // per round, so a million rows take four dependent loads instead of twenty.
        int lo = 0, hi = m;
        while (hi - lo > 1) {
            const int step = (hi - lo + 31) / 32;
            const long long idx = (long long)lo + (long long)(lane + 1) * step;
            const bool ok = idx < hi && (long long)__ldg(rowPtr + idx) <= p0;
            const int k = __popc(__ballot_sync(0xffffffffu, ok));  // offsets ascend: the lanes that pass are a prefix
            lo += k * step;
            hi = hi < lo + step ? hi : lo + step;
        }
        int r = lo, cachedRow = -1;
        uint4 x0 = make_uint4(0, 0, 0, 0);
        const int myCol = p0 + lane < p1 ? __ldg(colInd + p0 + lane) : 0;  // the chunk's columns, one per lane
        // Four entries at a time: their Y rows are requested together, so that a warp has four rows in flight
        // instead of one (the gather of Y rows from DRAM is what this kernel waits for).
        for (long long p = p0; p < p1; p += kSddmmBatch) {
            int rows[kSddmmBatch];
            uint4 y[kSddmmBatch];
#pragma unroll
            for (int u = 0; u < kSddmmBatch; ++u) {
                const bool live = p + u < p1;
                if (live) {
                    while ((long long)__ldg(rowPtr + r + 1) <= p + u) ++r;
                }
                rows[u] = r;
                const int j = __shfl_sync(0xffffffffu, myCol, (int)(p + u - p0) & 31);
                y[u] = make_uint4(0, 0, 0, 0);
                if (live && lane < pieces) y[u] = __ldg(Y16 + (long long)j * yRow16 + lane);
            }
            float acc[kSddmmBatch];
#pragma unroll
            for (int u = 0; u < kSddmmBatch; ++u) {
                acc[u] = 0.0f;
                if (p + u >= p1) continue;
                const uint4 *xr = X16 + (long long)rows[u] * xRow16;
                if (rows[u] != cachedRow) {
                    if (lane < pieces) x0 = __ldg(xr + lane);
                    cachedRow = rows[u];
                }
                if (lane < pieces) acc[u] = Dot16(x0, y[u], acc[u], T());
                if (pieces > 32) {
                    const int j = __shfl_sync(0xffffffffu, myCol, (int)(p + u - p0) & 31);
                    const uint4 *yc = Y16 + (long long)j * yRow16;
                    for (int q = lane + 32; q < pieces; q += 32) acc[u] = Dot16(__ldg(xr + q), __ldg(yc + q), acc[u], T());
                }
            }
#pragma unroll
            for (int u = 0; u < kSddmmBatch; ++u) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], off);
            }
            // every lane holds all sums now: lane u writes entry p + u
            float mine = 0.0f;
#pragma unroll
            for (int u = 0; u < kSddmmBatch; ++u) mine = lane == u ? acc[u] : mine;
            if (lane < kSddmmBatch && p + lane < p1) {
                float z = a * mine;
                if (b != 0.0f) z += b * Load<T>(cVal + p + lane);
                cVal[p + lane] = Store<T>(z);
            }
        }
    }
}

float HalfBitsToFloat(uint16_t h) { return __half2float(__ushort_as_half(h)); }

float ReadScalar(const void *p, aclDataType computeType)  // sddmm_host.cpp:128-139
{
    if (computeType == ACL_FLOAT16) {
        uint16_t bits;
        __builtin_memcpy(&bits, p, sizeof(bits));
        return HalfBitsToFloat(bits);
    }
    float v;
    __builtin_memcpy(&v, p, sizeof(v));
    return v;
}

aclsparseStatus_t ValidateInputs(const aclsparseDnMatDescr *X, const aclsparseDnMatDescr *Y, const aclsparseSpMatDescr *C,
                                 aclsparseOperation_t opX, aclsparseOperation_t opY, aclDataType computeType,
                                 aclsparseSDDMMAlg_t alg)
{
    // descriptors (sddmm_host.cpp:209-232)
    if (X == nullptr || Y == nullptr || C == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (C->format != ACL_SPARSE_FORMAT_CSR) return ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED;
    if (C->offsetType != C->indexType || C->offsetType != ACL_SPARSE_INDEX_32I) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (C->base != ACL_SPARSE_INDEX_BASE_ZERO) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    // operations (:194-207)
    if (opX != ACL_SPARSE_OP_NON_TRANSPOSE && opX != ACL_SPARSE_OP_TRANSPOSE) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (opY != ACL_SPARSE_OP_NON_TRANSPOSE && opY != ACL_SPARSE_OP_TRANSPOSE) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    // types and dimensions (:234-269)
    const bool f32 = X->valueType == ACL_FLOAT && Y->valueType == ACL_FLOAT && C->valueType == ACL_FLOAT &&
                     computeType == ACL_FLOAT;
    const bool f16 = X->valueType == ACL_FLOAT16 && Y->valueType == ACL_FLOAT16 && C->valueType == ACL_FLOAT16 &&
                     computeType == ACL_FLOAT16;
    if (!f32 && !f16) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    const int64_t m = C->rows, n = C->cols;
    int64_t k;
    if (opX == ACL_SPARSE_OP_NON_TRANSPOSE) {
        if (X->rows != m) return ACL_SPARSE_STATUS_INVALID_VALUE;
        k = X->cols;
    } else {
        if (X->cols != m) return ACL_SPARSE_STATUS_INVALID_VALUE;
        k = X->rows;
    }
    const bool yOk = opY == ACL_SPARSE_OP_NON_TRANSPOSE ? (Y->rows == k && Y->cols == n) : (Y->rows == n && Y->cols == k);
    if (!yOk) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (alg != ACL_SPARSE_SDDMM_ALG_DEFAULT) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    if (C->rows > INT32_MAX || C->cols > INT32_MAX || X->rows > INT32_MAX || X->cols > INT32_MAX ||
        Y->rows > INT32_MAX || Y->cols > INT32_MAX)
        return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    // CSR data (:271-294)
    if (C->nnz > INT32_MAX) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (C->offsets == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (C->nnz > 0 && (C->indices == nullptr || C->values == nullptr)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    return ACL_SPARSE_STATUS_SUCCESS;
}

// sddmm_host.cpp:660-692
aclsparseStatus_t ValidateCall(aclsparseHandle_t handle, const aclsparseDnMatDescr *X, const aclsparseDnMatDescr *Y,
                               const aclsparseSpMatDescr *C, const void *alpha, const void *beta, void *buffer,
                               bool isPreprocess, aclsparseOperation_t opX, aclsparseOperation_t opY,
                               aclDataType computeType, aclsparseSDDMMAlg_t alg)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;
    const aclsparseStatus_t st = ValidateInputs(X, Y, C, opX, opY, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (alpha == nullptr || beta == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (buffer == nullptr) return isPreprocess ? ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES : ACL_SPARSE_STATUS_INVALID_VALUE;
    return ACL_SPARSE_STATUS_SUCCESS;
}

template <typename T>
int Launch(const aclsparseSpMatDescr *C, const aclsparseDnMatDescr *X, const aclsparseDnMatDescr *Y, int k, Strides st,
           float alpha, float beta, const void *alphaDev, const void *betaDev, cudaStream_t stream)
{
    const long long chunks = (C->nnz + 31) / 32;
    const long long want = (chunks + 7) / 8;
    const long long cap = (long long)b200sp_sm_count() * 32;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    const long long rowBytes = (long long)k * (long long)sizeof(T);
    const bool vec = st.xk == 1 && st.yk == 1 && rowBytes % 16 == 0 && (st.xi * (long long)sizeof(T)) % 16 == 0 &&
                     (st.yj * (long long)sizeof(T)) % 16 == 0 && reinterpret_cast<uintptr_t>(X->values) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(Y->values) % 16 == 0;
    if (vec) {
        SddmmVecKernel<T><<<grid, 256, 0, stream>>>(
            static_cast<const int32_t *>(C->offsets), static_cast<const int32_t *>(C->indices),
            static_cast<T *>(C->values), static_cast<const T *>(X->values), static_cast<const T *>(Y->values),
            (int)C->rows, (int)(rowBytes / 16), (long long)C->nnz, st.xi * (long long)sizeof(T) / 16,
            st.yj * (long long)sizeof(T) / 16, alpha, beta, static_cast<const T *>(alphaDev),
            static_cast<const T *>(betaDev));
        b200sp_note_launches(1);
        return (int)cudaGetLastError();
    }
    SddmmKernel<T><<<grid, 256, 0, stream>>>(
        static_cast<const int32_t *>(C->offsets), static_cast<const int32_t *>(C->indices), static_cast<T *>(C->values),
        static_cast<const T *>(X->values), static_cast<const T *>(Y->values), (int)C->rows, k, (long long)C->nnz, st,
        alpha, beta, static_cast<const T *>(alphaDev), static_cast<const T *>(betaDev));
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

aclsparseStatus_t aclsparseSDDMMBufferSize(aclsparseHandle_t handle, aclsparseOperation_t opX, aclsparseOperation_t opY,
                                           const void *alpha, aclsparseConstDnMatDescr_t matX,
                                           aclsparseConstDnMatDescr_t matY, const void *beta, aclsparseSpMatDescr_t matC,
                                           aclDataType computeType, aclsparseSDDMMAlg_t alg, size_t *size)
{
    if (handle == nullptr) return ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR;  // order of sddmm_host.cpp:487-505
    if (size == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (alpha == nullptr || beta == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const aclsparseStatus_t st = ValidateInputs(matX, matY, matC, opX, opY, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    *size = 256;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSDDMMPreprocess(aclsparseHandle_t handle, aclsparseOperation_t opX, aclsparseOperation_t opY,
                                           const void *alpha, aclsparseConstDnMatDescr_t matX,
                                           aclsparseConstDnMatDescr_t matY, const void *beta, aclsparseSpMatDescr_t matC,
                                           aclDataType computeType, aclsparseSDDMMAlg_t alg, void *buffer)
{
    return ValidateCall(handle, matX, matY, matC, alpha, beta, buffer, true, opX, opY, computeType, alg);
}

aclsparseStatus_t aclsparseSDDMM(aclsparseHandle_t handle, aclsparseOperation_t opX, aclsparseOperation_t opY,
                                 const void *alpha, aclsparseConstDnMatDescr_t matX, aclsparseConstDnMatDescr_t matY,
                                 const void *beta, aclsparseSpMatDescr_t matC, aclDataType computeType,
                                 aclsparseSDDMMAlg_t alg, void *buffer)
{
    const aclsparseStatus_t st = ValidateCall(handle, matX, matY, matC, alpha, beta, buffer, false, opX, opY, computeType, alg);
    if (st != ACL_SPARSE_STATUS_SUCCESS) return st;
    if (matC->nnz == 0 || matC->rows == 0) return ACL_SPARSE_STATUS_SUCCESS;
    const bool xT = opX == ACL_SPARSE_OP_TRANSPOSE, yT = opY == ACL_SPARSE_OP_TRANSPOSE;
    const bool xRow = matX->order == ACL_SPARSE_ORDER_ROW, yRow = matY->order == ACL_SPARSE_ORDER_ROW;
    const int k = (int)(xT ? matX->rows : matX->cols);
    Strides s;
    // stored X is (m x k) or, transposed, (k x m); element (row, col) sits at row * ld + col (row-major) or
    // row + col * ld (column-major)
    const bool xContigK = xT ? !xRow : xRow;  // k runs along the contiguous direction
    s.xi = xContigK ? matX->ld : 1;
    s.xk = xContigK ? 1 : matX->ld;
    const bool yContigK = yT ? yRow : !yRow;  // stored Y is (k x n) or, transposed, (n x k)
    s.yk = yContigK ? 1 : matY->ld;
    s.yj = yContigK ? matY->ld : 1;
    const bool host = handle->pointerMode == ACL_SPARSE_POINTER_MODE_HOST;
    const float a = host ? ReadScalar(alpha, computeType) : 0.0f;
    const float b = host ? ReadScalar(beta, computeType) : 0.0f;
    const void *aDev = host ? nullptr : alpha;
    const void *bDev = host ? nullptr : beta;
    const int rc = computeType == ACL_FLOAT16
                       ? Launch<__half>(matC, matX, matY, k, s, a, b, aDev, bDev, handle->stream)
                       : Launch<float>(matC, matX, matY, k, s, a, b, aDev, bDev, handle->stream);
    if (rc != 0) {
        B200SP_LOGE("aclsparseSDDMM: kernel launch failed (cuda error %d)", rc);
        return ACL_SPARSE_STATUS_EXECUTION_FAILED;
    }
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
