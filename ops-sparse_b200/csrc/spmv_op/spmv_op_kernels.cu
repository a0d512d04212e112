// SpMVOp kernels for sm_100a: Z = alpha * A * X + beta * Y with doubly compensated row sums.
//
// The reference gives every row to one SIMT thread, which walks the row's entries in CSR order
// with Priest's doubly compensated dot product: three accumulators hi + md + lo, the product split
// into its rounded value and its rounding error by one fused multiply-add
// (sparse/spmv_op/arch35/spmv_op_kernel.cpp:88-127), and combines
//     z = fma(alpha, hi, fma(alpha, md + lo, beta * y))                         (:172-176).
// Here a row gets G lanes (G a power of two up to 32): every lane runs exactly that recurrence
// over the entries lane, lane + G, lane + 2G, ... and the G triples are then joined pairwise by
// error-free additions on a fixed butterfly, so a row's result does not depend on scheduling and is
// the same bits on every run; the final combination is the reference's.  With G = 1 the arithmetic
// is the reference's, operation for operation.
//
// Two ways to pick G:
//   no plan (ALG1)   one G for the whole matrix, from nnz / rows; nothing is analysed;
//   plan (ALG2)      the analysis orders the rows by descending length class (class c: lengths that
//                    need c bits); rows of 1024 entries and more get a CTA each, rows of 64 and more
//                    a warp, the rest four lanes, longest rows first -- the
//                    counterpart of the reference's reorder / bin_edge tables
//                    (spmv_op_kernel.cpp:425-540), built here by a histogram and a scatter.
#include <cstdint>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "../common/side_stream.h"

namespace {

constexpr int kClasses = B200SP_SPMVOP_CLASSES;

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct OpPlanLayout {
    size_t offReorder, offHist, total;
};
inline OpPlanLayout OpLayoutFor(int64_t rows)
{
    OpPlanLayout L;
    L.offReorder = 0;
    L.offHist = AlignUp(sizeof(int32_t) * (size_t)(rows > 0 ? rows : 1), 256);
    L.total = L.offHist + 256;  // kClasses cursors
    return L;
}

struct Triple {
    float hi, md, lo;
};

// One step of the reference recurrence (spmv_op_kernel.cpp:101-122).
__device__ __forceinline__ void PriestStep(Triple &t, float val, float xv)
{
    const float prod = __fmul_rn(val, xv);
    const float pi = __fmaf_rn(val, xv, -prod);
    const float s1 = __fadd_rn(t.hi, prod);
    const float v1 = __fsub_rn(s1, t.hi);
    const float e1 = __fadd_rn(__fsub_rn(t.hi, __fsub_rn(s1, v1)), __fsub_rn(prod, v1));
    t.hi = s1;
    const float ee = __fadd_rn(e1, pi);
    const float s2 = __fadd_rn(t.md, ee);
    const float v2 = __fsub_rn(s2, t.md);
    const float e2 = __fadd_rn(__fsub_rn(t.md, __fsub_rn(s2, v2)), __fsub_rn(ee, v2));
    t.md = s2;
    t.lo = __fadd_rn(t.lo, e2);
}

__device__ __forceinline__ void TwoSum(float a, float b, float &s, float &e)
{
    s = __fadd_rn(a, b);
    const float v = __fsub_rn(s, a);
    e = __fadd_rn(__fsub_rn(a, __fsub_rn(s, v)), __fsub_rn(b, v));
}

// a += b without losing what the additions round away.
__device__ __forceinline__ void JoinTriples(Triple &a, const Triple &b)
{
    float hi, e1, md, e2, md2, e3;
    TwoSum(a.hi, b.hi, hi, e1);
    TwoSum(a.md, b.md, md, e2);
    TwoSum(md, e1, md2, e3);
    a.hi = hi;
    a.md = md2;
    a.lo = __fadd_rn(__fadd_rn(a.lo, b.lo), __fadd_rn(e2, e3));
}

__device__ __forceinline__ long long LoadOffset(const void *rowOffsets, bool is64, long long i)
{
    return is64 ? static_cast<const long long *>(rowOffsets)[i] : (long long)static_cast<const int32_t *>(rowOffsets)[i];
}

struct OpArgs {
    const void *rowOffsets;
    const int32_t *colInd;
    const float *val;
    const float *x;
    const float *y;
    float *z;
    const int32_t *reorder;  // NULL: row i is row i
    long long first;         // first position of this launch in the row sequence
    long long count;         // positions in this launch
    int indexBase;
    float alpha, beta;
    const float *alphaDev, *betaDev;
};

template <int G, bool kIs64>
__global__ void __launch_bounds__(256) SpmvOpRowsKernel(const OpArgs a)
{
    const float alpha = a.alphaDev ? *a.alphaDev : a.alpha;
    const float beta = a.betaDev ? *a.betaDev : a.beta;
    const int lane = threadIdx.x & (G - 1);
    const long long groupsTotal = (long long)gridDim.x * blockDim.x / G;
    const long long firstGroup = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
    // every lane of a warp makes the same number of trips, so the shuffles below are full-warp
    const long long padded = (a.count + groupsTotal - 1) / groupsTotal * groupsTotal;
    for (long long i = firstGroup; i < padded; i += groupsTotal) {
        const bool live = i < a.count;
        long long row = 0, s = 0, e = 0;
        if (live) {
            row = a.reorder ? (long long)a.reorder[a.first + i] : a.first + i;
            s = LoadOffset(a.rowOffsets, kIs64, row) - a.indexBase;
            e = LoadOffset(a.rowOffsets, kIs64, row + 1) - a.indexBase;
        }
        float yOld = 0.0f;
        if (live && lane == 0 && beta != 0.0f) yOld = a.y[row];  // requested now, used at the end
        Triple t{0.0f, 0.0f, 0.0f};
        // Four entries are requested before the first of them is used; the steps run in entry order.
        long long p = s + lane;
        for (; p + 3 * G < e; p += 4 * G) {
            float v[4], xv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int col = __ldcs(a.colInd + p + u * G) - a.indexBase;
                v[u] = __ldcs(a.val + p + u * G);
                xv[u] = __ldg(a.x + col);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) PriestStep(t, v[u], xv[u]);
        }
        for (; p < e; p += G) {
            const int col = __ldcs(a.colInd + p) - a.indexBase;
            PriestStep(t, __ldcs(a.val + p), __ldg(a.x + col));
        }
#pragma unroll
        for (int off = G >> 1; off > 0; off >>= 1) {
            Triple o;
            o.hi = __shfl_down_sync(0xffffffffu, t.hi, off, G);
            o.md = __shfl_down_sync(0xffffffffu, t.md, off, G);
            o.lo = __shfl_down_sync(0xffffffffu, t.lo, off, G);
            JoinTriples(t, o);  // lanes >= off of a group compute values nobody reads
        }
        if (live && lane == 0) {
            // spmv_op_kernel.cpp:172-176
            const float corr = __fadd_rn(t.md, t.lo);
            const float step1 = __fmaf_rn(alpha, corr, __fmul_rn(beta, yOld));
            a.z[row] = __fmaf_rn(alpha, t.hi, step1);
        }
    }
}

// Rows of kLongBits bits or more (1024 entries and up): one CTA per row.  Thread t runs the recurrence on
// entries t, t + 256, ...; the lanes of a warp are joined on the butterfly, then warp 0 joins the eight
// warp triples the same way: a fixed shape again.
constexpr int kLongBits = 11;
template <bool kIs64>
__global__ void __launch_bounds__(256) SpmvOpLongRowsKernel(const OpArgs a)
{
    __shared__ Triple sWarp[8];
    const float alpha = a.alphaDev ? *a.alphaDev : a.alpha;
    const float beta = a.betaDev ? *a.betaDev : a.beta;
    const int tid = threadIdx.x;
    const long long row = a.reorder ? (long long)a.reorder[a.first + blockIdx.x] : a.first + blockIdx.x;
    const long long s = LoadOffset(a.rowOffsets, kIs64, row) - a.indexBase;
    const long long e = LoadOffset(a.rowOffsets, kIs64, row + 1) - a.indexBase;
    float yOld = 0.0f;
    if (tid == 0 && beta != 0.0f) yOld = a.y[row];
    Triple t{0.0f, 0.0f, 0.0f};
    long long p = s + tid;
    for (; p + 3 * 256 < e; p += 4 * 256) {
        float v[4], xv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int col = __ldcs(a.colInd + p + u * 256) - a.indexBase;
            v[u] = __ldcs(a.val + p + u * 256);
            xv[u] = __ldg(a.x + col);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) PriestStep(t, v[u], xv[u]);
    }
    for (; p < e; p += 256) {
        const int col = __ldcs(a.colInd + p) - a.indexBase;
        PriestStep(t, __ldcs(a.val + p), __ldg(a.x + col));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        Triple o;
        o.hi = __shfl_down_sync(0xffffffffu, t.hi, off);
        o.md = __shfl_down_sync(0xffffffffu, t.md, off);
        o.lo = __shfl_down_sync(0xffffffffu, t.lo, off);
        JoinTriples(t, o);
    }
    if ((tid & 31) == 0) sWarp[tid >> 5] = t;
    __syncthreads();
    if (tid < 32) {
        Triple w = tid < 8 ? sWarp[tid] : Triple{0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
            Triple o;
            o.hi = __shfl_down_sync(0xffffffffu, w.hi, off);
            o.md = __shfl_down_sync(0xffffffffu, w.md, off);
            o.lo = __shfl_down_sync(0xffffffffu, w.lo, off);
            JoinTriples(w, o);
        }
        if (tid == 0) {
            const float corr = __fadd_rn(w.md, w.lo);
            const float step1 = __fmaf_rn(alpha, corr, __fmul_rn(beta, yOld));
            a.z[row] = __fmaf_rn(alpha, w.hi, step1);
        }
    }
}

__global__ void SpmvOpScaleKernel(const float *__restrict__ y, float *__restrict__ z, long long rows, float beta,
                                  const float *betaDev)
{
    const float b = betaDev ? *betaDev : beta;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows;
         i += (long long)gridDim.x * blockDim.x)
        z[i] = b != 0.0f ? __fmul_rn(b, y[i]) : 0.0f;
}

__device__ __forceinline__ int LengthClass(long long len)
{
    return len <= 0 ? 0 : 64 - __clzll((unsigned long long)len);  // bits needed: 1 -> 1, 2..3 -> 2, 4..7 -> 3, ...
}

// cursors[c] += rows of class c
template <bool kIs64>
__global__ void SpmvOpHistogramKernel(const void *rowOffsets, long long rows, int32_t *cursors)
{
    __shared__ int sHist[kClasses];
    if (threadIdx.x < kClasses) sHist[threadIdx.x] = 0;
    __syncthreads();
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
         r += (long long)gridDim.x * blockDim.x) {
        const long long len = LoadOffset(rowOffsets, kIs64, r + 1) - LoadOffset(rowOffsets, kIs64, r);
        int c = LengthClass(len);
        if (c >= kClasses) c = kClasses - 1;
        atomicAdd(&sHist[c], 1);
    }
    __syncthreads();
    if (threadIdx.x < kClasses && sHist[threadIdx.x] != 0) atomicAdd(&cursors[threadIdx.x], sHist[threadIdx.x]);
}

template <bool kIs64>
__global__ void SpmvOpScatterKernel(const void *rowOffsets, long long rows, int32_t *cursors, int32_t *reorder)
{
    // A CTA first counts its rows per class, reserves that many slots of each class with one atomic,
    // then places its rows; the order inside a class is arbitrary and no result depends on it.
    __shared__ int sCount[kClasses];
    __shared__ int sBase[kClasses];
    const long long chunk = (rows + gridDim.x - 1) / gridDim.x;
    const long long r0 = (long long)blockIdx.x * chunk;
    const long long r1 = r0 + chunk < rows ? r0 + chunk : rows;
    if (threadIdx.x < kClasses) sCount[threadIdx.x] = 0;
    __syncthreads();
    for (long long r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
        const long long len = LoadOffset(rowOffsets, kIs64, r + 1) - LoadOffset(rowOffsets, kIs64, r);
        int c = LengthClass(len);
        if (c >= kClasses) c = kClasses - 1;
        atomicAdd(&sCount[c], 1);
    }
    __syncthreads();
    if (threadIdx.x < kClasses) {
        sBase[threadIdx.x] = sCount[threadIdx.x] != 0 ? atomicAdd(&cursors[threadIdx.x], sCount[threadIdx.x]) : 0;
        sCount[threadIdx.x] = 0;
    }
    __syncthreads();
    for (long long r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
        const long long len = LoadOffset(rowOffsets, kIs64, r + 1) - LoadOffset(rowOffsets, kIs64, r);
        int c = LengthClass(len);
        if (c >= kClasses) c = kClasses - 1;
        reorder[sBase[c] + atomicAdd(&sCount[c], 1)] = (int32_t)r;
    }
}

// Lanes for rows whose length needs `bits` bits.  Two ranges only: a launch per class of short rows cost
// 15 us each for a few hundred thousand entries (five launches, 81 us on the power-law matrix).
inline int LanesForClass(int bits) { return bits >= 7 ? 32 : 4; }  // 64 entries and more: a warp per row

template <bool kIs64>
void LaunchRows(const OpArgs &a, int G, cudaStream_t st)
{
    if (a.count <= 0) return;
    const long long want = (a.count * G + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 64;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    switch (G) {
        case 1: SpmvOpRowsKernel<1, kIs64><<<blocks, 256, 0, st>>>(a); break;
        case 2: SpmvOpRowsKernel<2, kIs64><<<blocks, 256, 0, st>>>(a); break;
        case 4: SpmvOpRowsKernel<4, kIs64><<<blocks, 256, 0, st>>>(a); break;
        case 8: SpmvOpRowsKernel<8, kIs64><<<blocks, 256, 0, st>>>(a); break;
        case 16: SpmvOpRowsKernel<16, kIs64><<<blocks, 256, 0, st>>>(a); break;
        default: SpmvOpRowsKernel<32, kIs64><<<blocks, 256, 0, st>>>(a); break;
    }
    b200sp_note_launches(1);
}

}  // namespace

extern "C" {

size_t b200sp_spmvop_plan_bytes(int64_t rows) { return OpLayoutFor(rows).total; }

int b200sp_spmvop_analyze(const void *row_offsets, int offsets_are_64, int64_t rows, void *plan, size_t plan_bytes,
                          int32_t *class_start, void *stream)
{
    const OpPlanLayout L = OpLayoutFor(rows);
    if (plan == nullptr || class_start == nullptr || plan_bytes < L.total) return (int)cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *p = static_cast<char *>(plan);
    auto *reorder = reinterpret_cast<int32_t *>(p + L.offReorder);
    auto *cursors = reinterpret_cast<int32_t *>(p + L.offHist);
    cudaError_t e = cudaMemsetAsync(cursors, 0, 256, st);
    if (e != cudaSuccess) return (int)e;
    for (int c = 0; c <= kClasses; ++c) class_start[c] = 0;
    if (rows <= 0) return 0;
    const long long want = (rows + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 8;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    // Histogram on the device; the 33 counts come back once and the class starts are summed on the host.
    if (offsets_are_64) SpmvOpHistogramKernel<true><<<blocks, 256, 0, st>>>(row_offsets, rows, cursors);
    else SpmvOpHistogramKernel<false><<<blocks, 256, 0, st>>>(row_offsets, rows, cursors);
    b200sp_note_launches(1);
    int32_t hist[kClasses];
    e = cudaMemcpyAsync(hist, cursors, sizeof(hist), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    int32_t cursorInit[kClasses];
    int running = 0;
    for (int k = 0; k < kClasses; ++k) {
        const int c = kClasses - 1 - k;
        class_start[k] = running;
        cursorInit[c] = running;
        running += hist[c];
    }
    class_start[kClasses] = running;
    e = cudaMemcpyAsync(cursors, cursorInit, sizeof(cursorInit), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return (int)e;
    if (offsets_are_64) SpmvOpScatterKernel<true><<<blocks, 256, 0, st>>>(row_offsets, rows, cursors, reorder);
    else SpmvOpScatterKernel<false><<<blocks, 256, 0, st>>>(row_offsets, rows, cursors, reorder);
    b200sp_note_launches(1);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    // cursorInit lives on this frame: the copy above must have read it before we return
    return (int)cudaStreamSynchronize(st);
}

int b200sp_spmvop_launch(const void *row_offsets, int offsets_are_64, const int32_t *col_ind, const float *val,
                         const float *x, const float *y, float *z, int64_t rows, int64_t nnz, int index_base,
                         float alpha, float beta, const float *alpha_dev, const float *beta_dev, const void *plan,
                         const int32_t *class_start, void *stream)
{
    if (rows <= 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    OpArgs a;
    a.rowOffsets = row_offsets;
    a.colInd = col_ind;
    a.val = val;
    a.x = x;
    a.y = y;
    a.z = z;
    a.indexBase = index_base;
    a.alpha = alpha;
    a.beta = beta;
    a.alphaDev = alpha_dev;
    a.betaDev = beta_dev;
    if (plan == nullptr || class_start == nullptr) {
        a.reorder = nullptr;
        a.first = 0;
        a.count = rows;
        const long long avg = nnz / rows;
        int G = 1;
        while (G < 32 && 4 * G < avg) G <<= 1;
        if (offsets_are_64) LaunchRows<true>(a, G, st);
        else LaunchRows<false>(a, G, st);
        return (int)cudaGetLastError();
    }
    a.reorder = static_cast<const int32_t *>(plan);
    // Classes of kLongBits bits and more: a CTA per row.
    int k = kClasses - kLongBits;  // class_start index of class kLongBits - 1
    a.first = class_start[0];
    a.count = (long long)class_start[k] - class_start[0];
    // The rows of the ranges are disjoint, so the long-row grid goes onto the side stream and runs beside the
    // other ranges (each of them is bound by latency, not by a throughput the others would take away).
    b200sp::SideLanes *lanes = nullptr;
    if (a.count > 0) {
        cudaStream_t sL = st;
        lanes = b200sp::GetSideLanes();
        if (lanes != nullptr) {
            if (cudaEventRecord(lanes->fork, st) != cudaSuccess ||
                cudaStreamWaitEvent(lanes->stream[0], lanes->fork, 0) != cudaSuccess)
                return (int)cudaGetLastError();
            sL = lanes->stream[0];
        }
        if (offsets_are_64) SpmvOpLongRowsKernel<true><<<(unsigned)a.count, 256, 0, sL>>>(a);
        else SpmvOpLongRowsKernel<false><<<(unsigned)a.count, 256, 0, sL>>>(a);
        b200sp_note_launches(1);
        if (lanes != nullptr && cudaEventRecord(lanes->join[0], sL) != cudaSuccess) return (int)cudaGetLastError();
    }
    // Then one launch per run of classes that share a lane count, longest rows first.
    while (k < kClasses) {
        const int G = LanesForClass(kClasses - 1 - k);
        int k2 = k;
        while (k2 < kClasses && LanesForClass(kClasses - 1 - k2) == G) ++k2;
        a.first = class_start[k];
        a.count = (long long)class_start[k2] - class_start[k];
        if (offsets_are_64) LaunchRows<true>(a, G, st);
        else LaunchRows<false>(a, G, st);
        k = k2;
    }
    if (lanes != nullptr && cudaStreamWaitEvent(st, lanes->join[0], 0) != cudaSuccess) return (int)cudaGetLastError();
    return (int)cudaGetLastError();
}

int b200sp_spmvop_scale(const float *y, float *z, int64_t rows, float beta, const float *beta_dev, void *stream)
{
    if (rows <= 0) return 0;
    const long long want = (rows + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 16;
    SpmvOpScaleKernel<<<(unsigned)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        y, z, rows, beta, beta_dev);
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

}  // extern "C"
