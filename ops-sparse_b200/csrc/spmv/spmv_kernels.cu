// CSR SpMV kernels for sm_100a and their extern "C" launchers.
//
// The reference's device code for this operator (sparse/spmv/arch22/kernels/spmv_kernel.h:
// 27-310 non-transpose, 321-640 transpose) gives every core an equal count of rows and
// walks them one at a time.  Here the work is cut by *merge path* instead: the rows' end
// markers and the non-zeros form one merged sequence of rows + nnz items and every CTA takes
// an equal slice (a tile) of it, whatever the row lengths are.  A tile
//   1. streams its slice of col_ind / values with 128-bit evict-first loads, gathers x
//      through the read-only path and parks the products in shared memory;
//   2. lets every thread walk 15 consecutive merge items (add a product, or close a row),
//      then joins rows that span threads with a segmented scan over the threads' carries;
//   3. writes y with one coalesced pass (alpha * sum + beta * y).
// Short rows therefore cost a few instructions each (scalar-row work inside a thread), long
// rows are summed by as many threads as they have items (vector-row), and a row cut by a
// tile boundary is finished without a second kernel and without waiting: every tile that
// holds a piece stores its partial sum, then bumps an arrival counter owned by the tile in
// which the row ends; whichever tile arrives last adds the pieces in tile order (so the
// result does not depend on scheduling) and writes y.
//
// Numerics follow the reference golden SpmvCpu (test/spmv/arch22/spmv_test.cpp:156-173):
// values and x are widened to the compute type before the multiply, sums are kept in the
// compute type, the result is alpha*sum + beta*y rounded once to the output type.
// beta == 0 never reads y.
#include <cstdint>
#include <cstdio>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "b200sp_kernels.h"

namespace {

constexpr int kTileThreads = 256;
constexpr int kItemsPerThread = 15;  // odd: consecutive threads start in different shared-memory banks
constexpr int kTileItems = kTileThreads * kItemsPerThread;  // merge items (row ends + non-zeros) per tile
constexpr int kSmemWords = kTileItems + 12;                 // row offsets + products, with alignment slack
constexpr int kVecPerThread = (kTileItems + 6 + 4 * kTileThreads - 1) / (4 * kTileThreads);

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct PlanLayout {
    int64_t ntiles;
    size_t offTileRow, offCounters, offHead, offTail, total;
};

inline PlanLayout LayoutFor(int64_t rows, int64_t nnz)
{
    PlanLayout L;
    L.ntiles = (rows + nnz + kTileItems - 1) / kTileItems;
    L.offTileRow = 0;
    L.offCounters = AlignUp(L.offTileRow + sizeof(int32_t) * (size_t)(L.ntiles + 1), 256);
    L.offHead = AlignUp(L.offCounters + sizeof(int32_t) * (size_t)L.ntiles, 256);
    L.offTail = AlignUp(L.offHead + 4 * (size_t)L.ntiles, 256);
    L.total = AlignUp(L.offTail + 4 * (size_t)L.ntiles, 256);
    if (L.total == 0) L.total = 256;
    return L;
}

// ---------------------------------------------------------------- element helpers

template <typename CompT, typename T>
__device__ __forceinline__ CompT Widen(T v);
template <> __device__ __forceinline__ float Widen<float, float>(float v) { return v; }
template <> __device__ __forceinline__ float Widen<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float Widen<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float Widen<float, int32_t>(int32_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ int32_t Widen<int32_t, int32_t>(int32_t v) { return v; }

template <typename OutT, typename CompT>
__device__ __forceinline__ OutT Narrow(CompT v);
template <> __device__ __forceinline__ float Narrow<float, float>(float v) { return v; }
template <> __device__ __forceinline__ __half Narrow<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 Narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ int32_t Narrow<int32_t, int32_t>(int32_t v) { return v; }

template <typename CompT>
struct Scalars {
    CompT alpha, beta;
    const CompT *alphaDev, *betaDev;
    __device__ __forceinline__ CompT Alpha() const { return alphaDev ? *alphaDev : alpha; }
    __device__ __forceinline__ CompT Beta() const { return betaDev ? *betaDev : beta; }
};

// Four consecutive matrix values, streamed (evict-first) so they do not push x out of cache.
template <typename T>
struct Quad {
    T v[4];
};
__device__ __forceinline__ Quad<float> LoadQuad(const float *p)
{
    const float4 q = __ldcs(reinterpret_cast<const float4 *>(p));
    return {{q.x, q.y, q.z, q.w}};
}
__device__ __forceinline__ Quad<int32_t> LoadQuad(const int32_t *p)
{
    const int4 q = __ldcs(reinterpret_cast<const int4 *>(p));
    return {{q.x, q.y, q.z, q.w}};
}
__device__ __forceinline__ Quad<__half> LoadQuad(const __half *p)
{
    const uint2 q = __ldcs(reinterpret_cast<const uint2 *>(p));
    Quad<__half> r;
    *reinterpret_cast<uint2 *>(r.v) = q;
    return r;
}
__device__ __forceinline__ Quad<__nv_bfloat16> LoadQuad(const __nv_bfloat16 *p)
{
    const uint2 q = __ldcs(reinterpret_cast<const uint2 *>(p));
    Quad<__nv_bfloat16> r;
    *reinterpret_cast<uint2 *>(r.v) = q;
    return r;
}

template <typename CompT>
__device__ __forceinline__ CompT GroupSum(CompT v, int lanes)
{
    for (int off = lanes >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// ---------------------------------------------------------------- analysis

// One thread per tile boundary: binary search of diagonal t*kTileItems on the merge grid of
// (row end offsets, non-zero indices).  tileRow[t] = number of rows that end before the tile.
__global__ void SpmvTileSearchKernel(const int32_t *__restrict__ rowPtr, int rows, int nnz, int ntiles,
                                     int32_t *__restrict__ tileRow, int32_t *__restrict__ counters)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > ntiles) return;
    const long long total = (long long)rows + nnz;
    long long d = (long long)t * kTileItems;
    if (d > total) d = total;
    long long lo = d - nnz > 0 ? d - nnz : 0;
    long long hi = d < rows ? d : rows;
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)rowPtr[mid + 1] <= d - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    tileRow[t] = (int32_t)lo;
    if (t < ntiles) counters[t] = 0;
}

// ---------------------------------------------------------------- tile kernel

template <typename CompT, typename ValT, typename OutT>
struct TileArgs {
    const int32_t *rowPtr;
    const int32_t *colInd;
    const ValT *val;
    const ValT *x;
    OutT *y;
    int rows;
    int nnz;
    Scalars<CompT> sc;
    const int32_t *tileRow;
    int32_t *counters;
    CompT *partHead;
    CompT *partTail;
};

template <typename CompT, typename ValT, typename OutT, bool kVec>
__global__ void __launch_bounds__(kTileThreads) SpmvTileKernel(const TileArgs<CompT, ValT, OutT> a)
{
    __shared__ __align__(16) int32_t smem[kSmemWords];   // row offsets, then products
    __shared__ CompT sRowSum[kTileItems];                // finished sum of every row that ends here
    __shared__ CompT sScan[kTileThreads];                // per-thread carry after the segmented scan
    __shared__ int32_t sWarpKeyFirst[kTileThreads / 32];
    __shared__ int32_t sWarpKeyLast[kTileThreads / 32];
    __shared__ CompT sWarpValLast[kTileThreads / 32];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int t = blockIdx.x;
    const int i0 = a.tileRow[t];
    const int i1 = a.tileRow[t + 1];
    const long long total = (long long)a.rows + a.nnz;
    const long long d0 = (long long)t * kTileItems;
    const long long d1 = d0 + kTileItems < total ? d0 + kTileItems : total;
    const int j0 = (int)(d0 - i0);
    const int j1 = (int)(d1 - i1);
    const int R = i1 - i0;       // rows whose end lies in this tile
    const int nn = j1 - j0;      // non-zeros in this tile

    int32_t *sRow = smem;        // sRow[k] = rowPtr[i0 + k], k = 0..R
    const int prodOff = (R + 4) & ~3;
    CompT *sProd = reinterpret_cast<CompT *>(smem + prodOff);
    const int base = j0 & ~3;    // products are stored at sProd[index - base]

    for (int k = tid; k <= R; k += kTileThreads) sRow[k] = a.rowPtr[i0 + k];

    // ---- phase 1: stream the tile's non-zeros, gather x, store products -------------
    if (kVec) {
        const int nvec = (j1 - base + 3) >> 2;  // <= kVecPerThread * kTileThreads
        int4 c[kVecPerThread];
        Quad<ValT> v[kVecPerThread];
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) {
            const int q = tid + u * kTileThreads;
            const int idx = base + 4 * q;
            c[u] = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[u].v[e] = ValT(0);
            if (q < nvec) {
                if (idx + 4 <= a.nnz) {
                    c[u] = __ldcs(reinterpret_cast<const int4 *>(a.colInd + idx));
                    v[u] = LoadQuad(a.val + idx);
                } else {  // last quad of the arrays: stay inside them
                    int cc[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (idx + e < a.nnz) {
                            cc[e] = a.colInd[idx + e];
                            v[u].v[e] = a.val[idx + e];
                        }
                    }
                    c[u] = make_int4(cc[0], cc[1], cc[2], cc[3]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) {
            const int q = tid + u * kTileThreads;
            if (q < nvec) {
                const int idx = base + 4 * q;
                const int cc[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
                alignas(16) CompT p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // Entries past the end of the arrays were zero-filled above (column 0, value 0).
                    const bool live = idx + e < a.nnz;
                    const ValT xv = live ? __ldg(a.x + cc[e]) : ValT(0);
                    p[e] = Widen<CompT>(v[u].v[e]) * Widen<CompT>(xv);
                }
                *reinterpret_cast<int4 *>(sProd + 4 * q) = *reinterpret_cast<const int4 *>(p);
            }
        }
    } else {
        for (int idx = j0 + tid; idx < j1; idx += kTileThreads) {
            const int cidx = a.colInd[idx];
            sProd[idx - base] = Widen<CompT>(a.val[idx]) * Widen<CompT>(__ldg(a.x + cidx));
        }
    }
    __syncthreads();

    // ---- phase 2: every thread walks kItemsPerThread consecutive merge items -----------
    // Local merge coordinates: row ends sRow[k + 1] - j0 (k < R) against non-zero indices 0..nn-1.
    const int items = R + nn;
    const int dBeg = tid * kItemsPerThread < items ? tid * kItemsPerThread : items;
    const int dEnd = dBeg + kItemsPerThread < items ? dBeg + kItemsPerThread : items;
    int rowIdx, nzIdx;
    {
        int lo = dBeg - nn > 0 ? dBeg - nn : 0;
        int hi = dBeg < R ? dBeg : R;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (sRow[mid + 1] - j0 <= dBeg - mid - 1) lo = mid + 1;
            else hi = mid;
        }
        rowIdx = lo;
        nzIdx = dBeg - lo;
    }
    const CompT *prod = sProd + (j0 - base);
    int rowEnd = rowIdx < R ? sRow[rowIdx + 1] - j0 : 0x7fffffff;
    CompT running = CompT(0);
    int firstEnded = -1;  // first row this thread finishes: it may have begun in an earlier thread
#pragma unroll
    for (int it = 0; it < kItemsPerThread; ++it) {
        if (dBeg + it < dEnd) {
            if (nzIdx < rowEnd) {
                running += prod[nzIdx];
                ++nzIdx;
            } else {
                sRowSum[rowIdx] = running;
                if (firstEnded < 0) firstEnded = rowIdx;
                running = CompT(0);
                ++rowIdx;
                rowEnd = rowIdx < R ? sRow[rowIdx + 1] - j0 : 0x7fffffff;
            }
        }
    }

    // Segmented inclusive scan of the (row, partial) carries over the threads of the CTA: after
    // it, thread u holds the sum of the pieces of its last row held by threads <= u.
    CompT scan = running;
    const int key = rowIdx;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const CompT v2 = __shfl_up_sync(0xffffffffu, scan, off);
        const int k2 = __shfl_up_sync(0xffffffffu, key, off);
        if (lane >= off && k2 == key) scan += v2;
    }
    if (lane == 0) sWarpKeyFirst[warp] = key;
    if (lane == 31) {
        sWarpKeyLast[warp] = key;
        sWarpValLast[warp] = scan;
    }
    __syncthreads();
    if (__shfl_sync(0xffffffffu, key, 0) == key) {  // this thread's run reaches the start of its warp
        for (int w = warp - 1; w >= 0; --w) {
            if (sWarpKeyLast[w] != key) break;
            scan += sWarpValLast[w];
            if (sWarpKeyFirst[w] != key) break;
        }
    }
    sScan[tid] = scan;
    __syncthreads();
    if (firstEnded >= 0 && tid > 0) sRowSum[firstEnded] += sScan[tid - 1];
    __syncthreads();

    // ---- phase 3: coalesced epilogue ---------------------------------------------------
    const CompT alpha = a.sc.Alpha();
    const CompT beta = a.sc.Beta();
    auto storeRow = [&](int r, CompT sum) {
        CompT z = alpha * sum;
        if (beta != CompT(0)) z += beta * Widen<CompT>(a.y[r]);
        a.y[r] = Narrow<OutT>(z);
    };
    // Arrival protocol for a row r cut by tile boundaries; t1 is the tile where r ends.
    auto arrive = [&](int r, int t1) {
        __threadfence();
        const int tFirst = (int)(((long long)r + a.rowPtr[r]) / kTileItems);
        const int expected = t1 - tFirst;  // arrivals that precede the last one
        const int old = atomicAdd(a.counters + t1, 1);
        if (old == expected) {
            a.counters[t1] = 0;  // ready for the next launch
            __threadfence();
            CompT s = CompT(0);
            for (int u = tFirst; u < t1; ++u) s += __ldcg(a.partTail + u);
            s += __ldcg(a.partHead + t1);
            storeRow(r, s);
        }
    };
    const bool headContinues = R > 0 && sRow[0] < j0;  // row i0 began in an earlier tile
    for (int k = tid; k < R; k += kTileThreads) {
        if (k == 0 && headContinues) {
            a.partHead[t] = sRowSum[0];
            arrive(i0, t);
        } else {
            storeRow(i0 + k, sRowSum[k]);
        }
    }
    // Piece of the row after the last complete one, if this tile holds any of it.
    if (tid == kTileThreads - 1) {
        const int tailStart = sRow[R] > j0 ? sRow[R] : j0;
        if (i1 < a.rows && j1 > tailStart) {
            a.partTail[t] = scan;  // key == R here: the run of carries that ends the tile
            const int t1 = (int)(((long long)i1 + a.rowPtr[i1 + 1]) / kTileItems);
            arrive(i1, t1);
        }
    }
}

// ---------------------------------------------------------------- workspace-free kernel

// G lanes per row (G a power of two <= 32 chosen from nnz / rows), grid-stride over rows.
template <typename CompT, typename ValT, typename OutT>
__global__ void __launch_bounds__(256) SpmvRowGroupKernel(const int32_t *__restrict__ rowPtr,
                                                           const int32_t *__restrict__ colInd,
                                                           const ValT *__restrict__ val,
                                                           const ValT *__restrict__ x, OutT *__restrict__ y,
                                                           int rows, Scalars<CompT> sc, int G)
{
    const CompT alpha = sc.Alpha();
    const CompT beta = sc.Beta();
    const int lane = threadIdx.x & (G - 1);
    const long long groupsTotal = (long long)gridDim.x * blockDim.x / G;
    const long long first = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const long long rowsPadded = ((long long)rows + groupsTotal - 1) / groupsTotal * groupsTotal;
    for (long long r = first; r < rowsPadded; r += groupsTotal) {
        CompT sum = CompT(0);
        if (r < rows) {
            const int s = rowPtr[r];
            const int e = rowPtr[r + 1];
            for (int p = s + lane; p < e; p += G)
                sum += Widen<CompT>(__ldcs(val + p)) * Widen<CompT>(__ldg(x + __ldcs(colInd + p)));
        }
        sum = GroupSum(sum, G);
        if (r < rows && lane == 0) {
            CompT z = alpha * sum;
            if (beta != CompT(0)) z += beta * Widen<CompT>(y[r]);
            y[r] = Narrow<OutT>(z);
        }
    }
}

// ---------------------------------------------------------------- transpose kernels

// acc[j] = beta * y[j]  (AccT is the output type itself, or float for 16-bit outputs)
template <typename CompT, typename OutT, typename AccT>
__global__ void SpmvTransScaleKernel(const OutT *y, AccT *acc, int n, Scalars<CompT> sc)  // y may alias acc
{
    const CompT beta = sc.Beta();
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x)
        acc[j] = (beta == CompT(0)) ? AccT(0) : static_cast<AccT>(beta * Widen<CompT>(y[j]));
}

// acc[col] += (alpha * x[i]) * a_ij, G lanes per row, atomics on the accumulator.
template <typename CompT, typename ValT, typename AccT>
__global__ void __launch_bounds__(256) SpmvTransScatterKernel(const int32_t *__restrict__ rowPtr,
                                                               const int32_t *__restrict__ colInd,
                                                               const ValT *__restrict__ val,
                                                               const ValT *__restrict__ x, AccT *__restrict__ acc,
                                                               int rows, Scalars<CompT> sc, int G)
{
    const CompT alpha = sc.Alpha();
    const int lane = threadIdx.x & (G - 1);
    const long long groupsTotal = (long long)gridDim.x * blockDim.x / G;
    for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G; r < rows; r += groupsTotal) {
        const CompT xv = alpha * Widen<CompT>(x[r]);
        if (xv == CompT(0)) continue;
        const int s = rowPtr[r];
        const int e = rowPtr[r + 1];
        for (int p = s + lane; p < e; p += G)
            atomicAdd(acc + colInd[p], static_cast<AccT>(xv * Widen<CompT>(val[p])));
    }
}

template <typename OutT>
__global__ void SpmvTransNarrowKernel(const float *__restrict__ acc, OutT *__restrict__ y, int n)
{
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x)
        y[j] = Narrow<OutT>(acc[j]);
}

// ---------------------------------------------------------------- host dispatch

template <typename CompT>
Scalars<CompT> MakeScalars(const b200spScalars *s);
template <>
Scalars<float> MakeScalars<float>(const b200spScalars *s)
{
    return {s->alpha_f, s->beta_f, static_cast<const float *>(s->alpha_dev), static_cast<const float *>(s->beta_dev)};
}
template <>
Scalars<int32_t> MakeScalars<int32_t>(const b200spScalars *s)
{
    return {s->alpha_i, s->beta_i, static_cast<const int32_t *>(s->alpha_dev),
            static_cast<const int32_t *>(s->beta_dev)};
}

int GroupWidthFor(int64_t rows, int64_t nnz)
{
    const int64_t avg = rows > 0 ? nnz / rows : 0;
    int G = 1;
    while (G < 32 && G < avg) G <<= 1;
    return G;
}

template <typename CompT, typename ValT, typename OutT>
int LaunchTyped(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, void *y, int64_t rows,
                int64_t nnz, const b200spScalars *s, void *plan, cudaStream_t stream)
{
    const Scalars<CompT> sc = MakeScalars<CompT>(s);
    if (plan != nullptr) {
        const PlanLayout L = LayoutFor(rows, nnz);
        if (L.ntiles == 0) return 0;
        char *p = static_cast<char *>(plan);
        TileArgs<CompT, ValT, OutT> a;
        a.rowPtr = rowPtr;
        a.colInd = colInd;
        a.val = static_cast<const ValT *>(val);
        a.x = static_cast<const ValT *>(x);
        a.y = static_cast<OutT *>(y);
        a.rows = (int)rows;
        a.nnz = (int)nnz;
        a.sc = sc;
        a.tileRow = reinterpret_cast<const int32_t *>(p + L.offTileRow);
        a.counters = reinterpret_cast<int32_t *>(p + L.offCounters);
        a.partHead = reinterpret_cast<CompT *>(p + L.offHead);
        a.partTail = reinterpret_cast<CompT *>(p + L.offTail);
        const bool vec = (reinterpret_cast<uintptr_t>(colInd) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(val) % (4 * sizeof(ValT)) == 0);
        if (vec) SpmvTileKernel<CompT, ValT, OutT, true><<<(unsigned)L.ntiles, kTileThreads, 0, stream>>>(a);
        else SpmvTileKernel<CompT, ValT, OutT, false><<<(unsigned)L.ntiles, kTileThreads, 0, stream>>>(a);
        return (int)cudaGetLastError();
    }
    if (rows == 0) return 0;
    const int G = GroupWidthFor(rows, nnz);
    const int64_t wantBlocks = (rows * G + 255) / 256;
    const int64_t maxBlocks = (int64_t)b200sp_sm_count() * 32;
    const unsigned blocks = (unsigned)(wantBlocks < maxBlocks ? wantBlocks : maxBlocks);
    SpmvRowGroupKernel<CompT, ValT, OutT><<<blocks, 256, 0, stream>>>(
        rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), static_cast<OutT *>(y),
        (int)rows, sc, G);
    return (int)cudaGetLastError();
}

template <typename CompT, typename ValT, typename OutT>
int LaunchTransTyped(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, void *y,
                     int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *s, void *scratch,
                     size_t scratchBytes, cudaStream_t stream)
{
    const Scalars<CompT> sc = MakeScalars<CompT>(s);
    if (cols == 0) return 0;
    const int sms = b200sp_sm_count();
    const unsigned eltBlocks = (unsigned)((cols + 255) / 256 < (int64_t)sms * 16 ? (cols + 255) / 256 : sms * 16);
    const int G = GroupWidthFor(rows, nnz);
    const int64_t want = rows > 0 ? (rows * G + 255) / 256 : 1;
    const unsigned rowBlocks = (unsigned)(want < (int64_t)sms * 32 ? want : sms * 32);
    constexpr bool kNarrowOut = sizeof(OutT) == 2;
    if constexpr (kNarrowOut) {
        if (scratch == nullptr || scratchBytes < sizeof(float) * (size_t)cols) return (int)cudaErrorInvalidValue;
        float *acc = static_cast<float *>(scratch);
        SpmvTransScaleKernel<CompT, OutT, float><<<eltBlocks, 256, 0, stream>>>(static_cast<const OutT *>(y), acc,
                                                                                 (int)cols, sc);
        if (rows > 0)
            SpmvTransScatterKernel<CompT, ValT, float><<<rowBlocks, 256, 0, stream>>>(
                rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), acc, (int)rows, sc, G);
        SpmvTransNarrowKernel<OutT><<<eltBlocks, 256, 0, stream>>>(acc, static_cast<OutT *>(y), (int)cols);
    } else {
        OutT *acc = static_cast<OutT *>(y);
        SpmvTransScaleKernel<CompT, OutT, OutT><<<eltBlocks, 256, 0, stream>>>(acc, acc, (int)cols, sc);
        if (rows > 0)
            SpmvTransScatterKernel<CompT, ValT, OutT><<<rowBlocks, 256, 0, stream>>>(
                rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), acc, (int)rows, sc, G);
    }
    return (int)cudaGetLastError();
}

// Calls f.template operator()<CompT, ValT, OutT>() for a supported type triple, or returns -1.
template <typename F>
int DispatchTypes(int comp, int val, int out, F &&f)
{
    if (comp == B200SP_I32) {
        if (val == B200SP_I32 && out == B200SP_I32) return f.template operator()<int32_t, int32_t, int32_t>();
        return -1;
    }
    if (comp != B200SP_F32) return -1;
    if (val == B200SP_F32 && out == B200SP_F32) return f.template operator()<float, float, float>();
    if (val == B200SP_F16 && out == B200SP_F32) return f.template operator()<float, __half, float>();
    if (val == B200SP_F16 && out == B200SP_F16) return f.template operator()<float, __half, __half>();
    if (val == B200SP_BF16 && out == B200SP_F32) return f.template operator()<float, __nv_bfloat16, float>();
    if (val == B200SP_BF16 && out == B200SP_BF16) return f.template operator()<float, __nv_bfloat16, __nv_bfloat16>();
    if (val == B200SP_I32 && out == B200SP_F32) return f.template operator()<float, int32_t, float>();
    return -1;
}

}  // namespace

extern "C" {

int b200sp_sm_count(void)
{
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            cached = n;
        else
            return 148;
    }
    return cached;
}

size_t b200sp_spmv_plan_bytes(int64_t rows, int64_t nnz) { return LayoutFor(rows, nnz).total; }

int b200sp_spmv_analyze(const int32_t *row_ptr, int64_t rows, int64_t nnz, void *plan, size_t plan_bytes,
                        void *stream)
{
    const PlanLayout L = LayoutFor(rows, nnz);
    if (plan == nullptr || plan_bytes < L.total) return (int)cudaErrorInvalidValue;
    if (L.ntiles == 0) return 0;
    char *p = static_cast<char *>(plan);
    const unsigned blocks = (unsigned)((L.ntiles + 1 + 255) / 256);
    SpmvTileSearchKernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        row_ptr, (int)rows, (int)nnz, (int)L.ntiles, reinterpret_cast<int32_t *>(p + L.offTileRow),
        reinterpret_cast<int32_t *>(p + L.offCounters));
    return (int)cudaGetLastError();
}

int b200sp_spmv_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x, void *y,
                       int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars, int comp_type,
                       int val_type, int out_type, void *plan, void *stream)
{
    (void)cols;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rc = DispatchTypes(comp_type, val_type, out_type, [&]<typename C, typename V, typename O>() {
        return LaunchTyped<C, V, O>(row_ptr, col_ind, val, x, y, rows, nnz, scalars, plan, st);
    });
    return rc < 0 ? (int)cudaErrorInvalidValue : rc;
}

int b200sp_spmv_trans_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x,
                             void *y, int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars,
                             int comp_type, int val_type, int out_type, void *scratch, size_t scratch_bytes,
                             void *stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rc = DispatchTypes(comp_type, val_type, out_type, [&]<typename C, typename V, typename O>() {
        return LaunchTransTyped<C, V, O>(row_ptr, col_ind, val, x, y, rows, cols, nnz, scalars, scratch,
                                         scratch_bytes, st);
    });
    return rc < 0 ? (int)cudaErrorInvalidValue : rc;
}

}  // extern "C"

// ---------------------------------------------------------------- entry point without allocation

namespace {

// Scratch for b200sp_spmv_f32_noalloc: the tile table, arrival counters and partial sums that
// b200sp_spmv_analyze would otherwise write into a caller-allocated workspace.  Every GPU that
// loads the library carries this array until the process exits.
constexpr int64_t kNoAllocMaxItems = B200SP_NOALLOC_MAX_ITEMS;
constexpr size_t kNoAllocBytes = 16 * ((size_t)(kNoAllocMaxItems / kTileItems) + 2) + 4 * 256;
static __device__ __align__(256) unsigned char gNoAllocScratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
void *gNoAllocAddr[kMaxDevices] = {};  // device address of gNoAllocScratch, per device ordinal

// In host code `gNoAllocScratch` is only a handle for the runtime, not an address a kernel can
// use; the device address has to be asked for, once per device, with that device current.
int NoAllocScratchAddress(void **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    if (gNoAllocAddr[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, gNoAllocScratch);
        if (e != cudaSuccess) return (int)e;
        gNoAllocAddr[dev] = p;
    }
    *out = gNoAllocAddr[dev];
    return 0;
}

}  // namespace

extern "C" int b200sp_spmv_f32_noalloc(const int32_t *row_ptr, const int32_t *col_ind, const float *val,
                                       const float *x, float *y, int64_t rows, int64_t cols, int64_t nnz,
                                       float alpha, float beta, void *stream)
{
    (void)cols;
    if (rows < 0 || nnz < 0 || rows > INT32_MAX || nnz > INT32_MAX) return (int)cudaErrorInvalidValue;
    const PlanLayout L = LayoutFor(rows, nnz);
    if (rows + nnz > kNoAllocMaxItems || L.total > kNoAllocBytes) {
        std::fprintf(stderr,
                     "b200sp_spmv_f32_noalloc: rows + nnz = %lld exceeds B200SP_NOALLOC_MAX_ITEMS = %lld; "
                     "use aclsparseSpMV with a caller-provided buffer for a matrix of this size\n",
                     (long long)(rows + nnz), (long long)kNoAllocMaxItems);
        return (int)cudaErrorInvalidValue;
    }
    void *scratch = nullptr;
    const int rc = NoAllocScratchAddress(&scratch);
    if (rc != 0) return rc;
    if (L.ntiles == 0) return 0;
    // The analysis rewrites the tile table and zeroes the arrival counters, so nothing a previous
    // call left in the array is read.
    const int an = b200sp_spmv_analyze(row_ptr, rows, nnz, scratch, kNoAllocBytes, stream);
    if (an != 0) return an;
    b200spScalars sc{};
    sc.alpha_f = alpha;
    sc.beta_f = beta;
    return LaunchTyped<float, float, float>(row_ptr, col_ind, val, x, y, rows, nnz, &sc, scratch,
                                            static_cast<cudaStream_t>(stream));
}
