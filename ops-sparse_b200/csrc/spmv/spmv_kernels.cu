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

// Tuning knobs (compile-time; the defaults are the measured best on B200, see profiles/).
#ifndef B200SP_SPMV_THREADS
#define B200SP_SPMV_THREADS 256
#endif
#ifndef B200SP_SPMV_ITEMS_PER_THREAD
#define B200SP_SPMV_ITEMS_PER_THREAD 15
#endif
#ifndef B200SP_SPMV_MIN_BLOCKS
#define B200SP_SPMV_MIN_BLOCKS 5
#endif
constexpr int kTileThreads = B200SP_SPMV_THREADS;
constexpr int kItemsPerThread = B200SP_SPMV_ITEMS_PER_THREAD;  // odd: neighbouring threads start in different banks
constexpr int kTileItems = kTileThreads * kItemsPerThread;  // merge items (row ends + non-zeros) per tile
constexpr int kSmemWords = kTileItems + 12;                 // row offsets + products, with alignment slack
constexpr int kVecPerThread = (kTileItems + 6 + 4 * kTileThreads - 1) / (4 * kTileThreads);

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Long rows: rows of at least kLongLen entries are taken out of the tiles and summed by
// SpmvLongRowKernel, which stages x in shared memory one block of kXBlockBytes at a time.
#ifndef B200SP_SPMV_LONG_LEN
#define B200SP_SPMV_LONG_LEN 1024
#endif
#ifndef B200SP_SPMV_PIECE_LANES
#define B200SP_SPMV_PIECE_LANES 8  // lanes that share one (long row, x block) piece
#endif
constexpr int kLongLen = B200SP_SPMV_LONG_LEN;
constexpr int kNoLongRows = 0x7fffffff;
constexpr int kXBlockBytes = 128 * 1024;    // x slice resident in shared memory per CTA
constexpr int kMaxXBlocks = 64;             // wider matrices keep every row in the tiles
constexpr int kLongThreads = 1024;
constexpr int kMaxSkip = kTileItems / kLongLen + 3;  // long-row pieces that can meet one tile
static_assert(kLongLen >= 256, "long-row threshold too small for the per-tile skip list");

struct LongHeader {  // first 256 bytes of the long-row part of the plan
    int32_t count;     // rows routed to the long-row kernel
    int32_t unsorted;  // set when such a row has descending column indices (path is then not used)
};

struct PlanLayout {
    int64_t ntiles;
    int64_t capLong;   // 0 when the long-row path cannot be used for this shape
    int32_t xBlocks;   // column blocks of x
    int32_t xBlockElems;
    size_t offTileRow, offCounters, offHead, offTail, offFlags;
    size_t offLongHeader, offLongRows, offSegStart, offLongCounters, offLongPartials, offSkip, total;
};

// cols == 0 gives the tile-only layout (no long-row part).
inline PlanLayout LayoutFor(int64_t rows, int64_t nnz, int64_t cols = 0, int valBytes = 4)
{
    PlanLayout L;
    L.ntiles = (rows + nnz + kTileItems - 1) / kTileItems;
    L.offTileRow = 0;
    L.offCounters = AlignUp(L.offTileRow + sizeof(int32_t) * (size_t)(L.ntiles + 1), 256);
    L.offHead = AlignUp(L.offCounters + sizeof(int32_t) * (size_t)L.ntiles, 256);
    L.offTail = AlignUp(L.offHead + 4 * (size_t)L.ntiles, 256);
    L.offFlags = AlignUp(L.offTail + 4 * (size_t)L.ntiles, 256);
    L.offLongHeader = AlignUp(L.offFlags + sizeof(int32_t) * (size_t)L.ntiles, 256);
    L.xBlockElems = kXBlockBytes / valBytes;
    const int64_t xb = cols > 0 ? (cols + L.xBlockElems - 1) / L.xBlockElems : 0;
    L.xBlocks = (xb >= 1 && xb <= kMaxXBlocks) ? (int32_t)xb : 0;
    L.capLong = (L.xBlocks > 0 && nnz >= kLongLen) ? nnz / kLongLen : 0;
    L.offLongRows = L.offLongHeader + 256;
    L.offSegStart = AlignUp(L.offLongRows + sizeof(int32_t) * (size_t)L.capLong, 256);
    L.offLongCounters = AlignUp(L.offSegStart + sizeof(int32_t) * (size_t)L.capLong * (L.xBlocks + 1), 256);
    L.offLongPartials = AlignUp(L.offLongCounters + sizeof(int32_t) * (size_t)L.capLong, 256);
    L.offSkip = AlignUp(L.offLongPartials + 4 * (size_t)L.capLong * L.xBlocks, 256);
    // per tile: up to kMaxSkip [lo, hi) ranges of entries that belong to long rows
    L.total = AlignUp(L.offSkip + (L.capLong > 0 ? sizeof(int32_t) * 2 * kMaxSkip * (size_t)L.ntiles : 0), 256);
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
                                     int32_t *__restrict__ tileRow, int32_t *__restrict__ counters,
                                     int32_t *__restrict__ flags)
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
    if (t < ntiles) {
        counters[t] = 0;
        flags[t] = 0;
    }
}

// Appends every row of at least kLongLen entries to the long-row list (slot order is arbitrary;
// no result depends on it).
__global__ void SpmvFindLongRowsKernel(const int32_t *__restrict__ rowPtr, int rows, LongHeader *hdr,
                                       int32_t *__restrict__ longRows, int32_t *__restrict__ longCounters)
{
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
         r += (long long)gridDim.x * blockDim.x) {
        if (rowPtr[r + 1] - rowPtr[r] >= kLongLen) {
            const int slot = atomicAdd(&hdr->count, 1);
            longRows[slot] = (int32_t)r;
            longCounters[slot] = 0;
        }
    }
}

// One warp per long row: checks that its column indices ascend (the column-block cut below is a
// binary search) and records, for every tile the row meets, which of the tile's entries are its:
// flags[t] counts the ranges stored in skip[t][..] (a tile can meet at most kMaxSkip long rows).
__global__ void SpmvMarkLongRowsKernel(const int32_t *__restrict__ rowPtr, const int32_t *__restrict__ colInd,
                                       LongHeader *hdr, const int32_t *__restrict__ longRows,
                                       const int32_t *__restrict__ tileRow, int32_t *__restrict__ flags,
                                       int32_t *__restrict__ skip, long long totalItems)
{
    const int lane = threadIdx.x & 31;
    const int warpsTotal = gridDim.x * (blockDim.x >> 5);
    const int n = hdr->count;
    for (int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); slot < n; slot += warpsTotal) {
        const int r = longRows[slot];
        const int s = rowPtr[r], e = rowPtr[r + 1];
        bool bad = false;
        for (int p = s + lane; p + 1 < e; p += 32) bad |= colInd[p] > colInd[p + 1];
        if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(&hdr->unsorted, 1);
        const int tFirst = (int)(((long long)r + s) / kTileItems);
        const int tLast = (int)(((long long)r + e) / kTileItems);
        for (int t = tFirst + lane; t <= tLast; t += 32) {
            const long long d0 = (long long)t * kTileItems;
            const long long d1 = d0 + kTileItems < totalItems ? d0 + kTileItems : totalItems;
            const int j0 = (int)(d0 - tileRow[t]);
            const int j1 = (int)(d1 - tileRow[t + 1]);
            const int lo = s > j0 ? s : j0;
            const int hi = e < j1 ? e : j1;
            if (hi > lo) {
                const int k = atomicAdd(&flags[t], 1);
                if (k < kMaxSkip) {
                    skip[(long long)t * 2 * kMaxSkip + 2 * k] = lo;
                    skip[(long long)t * 2 * kMaxSkip + 2 * k + 1] = hi;
                }
            }
        }
    }
}

// segStart[slot * (xBlocks + 1) + b] = first entry of the row whose column is >= b * xBlockElems.
__global__ void SpmvLongSegmentsKernel(const int32_t *__restrict__ rowPtr, const int32_t *__restrict__ colInd,
                                       const LongHeader *hdr, const int32_t *__restrict__ longRows,
                                       int32_t *__restrict__ segStart, int xBlocks, int xBlockElems)
{
    const long long total = (long long)hdr->count * (xBlocks + 1);
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (long long)gridDim.x * blockDim.x) {
        const int slot = (int)(w / (xBlocks + 1));
        const int b = (int)(w - (long long)slot * (xBlocks + 1));
        const int r = longRows[slot];
        int lo = rowPtr[r], hi = rowPtr[r + 1];
        if (b == xBlocks) lo = hi;
        const long long bound = (long long)b * xBlockElems;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (colInd[mid] < bound) lo = mid + 1;
            else hi = mid;
        }
        segStart[w] = lo;
    }
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
    const int32_t *tileFlags;  // how many long rows meet this tile
    const int32_t *tileSkip;   // [tile][kMaxSkip][2]: entry ranges of those rows inside the tile
    int longLen;               // rows at least this long belong to SpmvLongRowKernel; kNoLongRows = none
};

template <typename CompT, typename ValT, typename OutT, bool kVec>
__global__ void __launch_bounds__(kTileThreads, B200SP_SPMV_MIN_BLOCKS) SpmvTileKernel(const TileArgs<CompT, ValT, OutT> a)
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

    // Entry ranges of this tile that belong to long rows (SpmvLongRowKernel sums those rows); the
    // analysis stored them per tile, so nothing here waits for the row offsets.
    int nSkip = 0;
    int skLo[kMaxSkip], skHi[kMaxSkip];
    if (a.longLen != kNoLongRows) {
        nSkip = a.tileFlags[t];
        nSkip = nSkip < kMaxSkip ? nSkip : kMaxSkip;
        const int32_t *sk = a.tileSkip + (long long)t * 2 * kMaxSkip;
#pragma unroll
        for (int i = 0; i < kMaxSkip; ++i) {
            skLo[i] = i < nSkip ? sk[2 * i] : 0;
            skHi[i] = i < nSkip ? sk[2 * i + 1] : 0;
        }
    }
    const bool flagged = nSkip > 0;  // same for the whole CTA
    // the whole tile lies inside one long row: nothing to do here
    if (R == 0 && nSkip == 1 && skLo[0] <= j0 && skHi[0] >= j1) return;
    // true when entries [lo, hi) all belong to long rows
    auto skipped = [&](int lo, int hi) {
        bool in = false;
#pragma unroll
        for (int i = 0; i < kMaxSkip; ++i) in |= (i < nSkip) && skLo[i] <= lo && hi <= skHi[i];
        return in;
    };

    // y of the first rows that end here, fetched now so that the epilogue does not wait for it
    const CompT betaEarly = a.sc.Beta();
    CompT yEarly = CompT(0);
    if (betaEarly != CompT(0) && tid < R) yEarly = Widen<CompT>(a.y[i0 + tid]);

    for (int k = tid; k <= R; k += kTileThreads) sRow[k] = a.rowPtr[i0 + k];

    // ---- phase 1: stream the tile's non-zeros, gather x, store products -------------
    if (kVec) {
        const int nvec = (j1 - base + 3) >> 2;  // <= kVecPerThread * kTileThreads
        int4 c[kVecPerThread];
        Quad<ValT> v[kVecPerThread];
        bool dead[kVecPerThread];  // quad outside the tile's vectors, or wholly inside a long row
#pragma unroll
        for (int u = 0; u < kVecPerThread; ++u) {
            const int q = tid + u * kTileThreads;
            const int idx = base + 4 * q;
            dead[u] = q >= nvec || (flagged && skipped(idx, idx + 4));
            c[u] = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[u].v[e] = ValT(0);
            if (!dead[u]) {
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
                    // so were quads skipped as part of a long row: no gather for either.
                    const bool live = idx + e < a.nnz && !dead[u];
                    const ValT xv = live ? __ldg(a.x + cc[e]) : ValT(0);
                    p[e] = Widen<CompT>(v[u].v[e]) * Widen<CompT>(xv);
                }
                *reinterpret_cast<int4 *>(sProd + 4 * q) = *reinterpret_cast<const int4 *>(p);
            }
        }
    } else {
        for (int idx = j0 + tid; idx < j1; idx += kTileThreads) {
            if (flagged && skipped(idx, idx + 1)) {
                sProd[idx - base] = CompT(0);
                continue;
            }
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
        if (a.longLen != kNoLongRows && sRow[k + 1] - sRow[k] >= a.longLen) continue;  // SpmvLongRowKernel writes it
        if (k == 0 && headContinues) {
            a.partHead[t] = sRowSum[0];
            arrive(i0, t);
        } else if (k == tid) {  // y of this row was fetched at the start of the kernel
            CompT z = alpha * sRowSum[k];
            if (beta != CompT(0)) z += beta * yEarly;
            a.y[i0 + k] = Narrow<OutT>(z);
        } else {
            storeRow(i0 + k, sRowSum[k]);
        }
    }
    // Piece of the row after the last complete one, if this tile holds any of it.
    if (tid == kTileThreads - 1) {
        const int tailStart = sRow[R] > j0 ? sRow[R] : j0;
        if (i1 < a.rows && j1 > tailStart) {
            const int tailEnd = a.rowPtr[i1 + 1];
            if (a.longLen == kNoLongRows || tailEnd - sRow[R] < a.longLen) {
                a.partTail[t] = scan;  // key == R here: the run of carries that ends the tile
                arrive(i1, (int)(((long long)i1 + tailEnd) / kTileItems));
            }
        }
    }
}

// ---------------------------------------------------------------- long-row kernel

template <typename CompT, typename ValT, typename OutT>
struct LongArgs {
    const int32_t *colInd;
    const ValT *val;
    const ValT *x;
    OutT *y;
    int cols;
    int nnz;
    Scalars<CompT> sc;
    const LongHeader *hdr;
    const int32_t *longRows;
    const int32_t *segStart;   // [slot][xBlocks + 1]
    int32_t *counters;         // [group], arrivals of the group's column-block CTAs
    CompT *partials;           // [slot][xBlocks]
    int xBlocks;
    int xBlockElems;
    int groups;                // CTAs per column block
};

// CTA (b, g) keeps block b of x (kXBlockBytes) in shared memory and sums, for every long row of
// its group, the entries whose column falls in that block -- a contiguous piece of the row,
// because column indices ascend.  One warp per piece; x comes from shared memory, so the only
// global traffic is the col_ind / values stream.  Eight lanes share a piece.  The last CTA of a
// row group to finish adds each row's partial sums in block order and writes y.
template <typename CompT, typename ValT, typename OutT, bool kVec>
__global__ void __launch_bounds__(kLongThreads) SpmvLongRowKernel(const LongArgs<CompT, ValT, OutT> a)
{
    extern __shared__ __align__(16) unsigned char sRaw[];
    ValT *xs = reinterpret_cast<ValT *>(sRaw);
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int b = blockIdx.x % a.xBlocks;
    const int g = blockIdx.x / a.xBlocks;
    const int nLong = a.hdr->count;
    const int x0 = b * a.xBlockElems;
    const int xn = a.cols - x0 < a.xBlockElems ? a.cols - x0 : a.xBlockElems;

    // stage the x block
    constexpr int kPer16 = 16 / (int)sizeof(ValT);
    if (reinterpret_cast<uintptr_t>(a.x) % 16 == 0) {
        const int nv = xn / kPer16;
        const int4 *src = reinterpret_cast<const int4 *>(a.x + x0);
        int4 *dst = reinterpret_cast<int4 *>(xs);
        for (int i = tid; i < nv; i += kLongThreads) dst[i] = __ldg(src + i);
        for (int i = nv * kPer16 + tid; i < xn; i += kLongThreads) xs[i] = a.x[x0 + i];
    } else {
        for (int i = tid; i < xn; i += kLongThreads) xs[i] = a.x[x0 + i];
    }
    __syncthreads();

    const ValT *xrel = xs - x0;  // xrel[col] is x[col] for the columns of this block
    // kPieceLanes lanes share one piece, so a warp has 32 / kPieceLanes pieces in flight.
    constexpr int kPieceLanes = B200SP_SPMV_PIECE_LANES;
    constexpr int kUnroll = 4;  // quads in flight per lane
    constexpr int kPiecesPerCta = kLongThreads / kPieceLanes;
    const int pl = tid & (kPieceLanes - 1);
    const int piece = tid / kPieceLanes;
    const int stride = a.groups * kPiecesPerCta;
    const int first = g * kPiecesPerCta + piece;
    const int trips = nLong > g * kPiecesPerCta ? (nLong - g * kPiecesPerCta + stride - 1) / stride : 0;  // CTA-uniform
    // piece bounds are fetched one trip ahead so that a trip starts with its loads, not a wait
    auto loadBounds = [&](int slot, int &s, int &e) {
        s = 0;
        e = 0;
        if (slot < nLong) {
            const int32_t *seg = a.segStart + (long long)slot * (a.xBlocks + 1) + b;
            s = seg[0];
            e = seg[1];
        }
    };
    int sCur, eCur, sNext, eNext;
    loadBounds(first, sCur, eCur);
    for (int it = 0; it < trips; ++it) {
        const int slot = first + it * stride;
        loadBounds(slot + stride, sNext, eNext);
        const int s = sCur, e = eCur;
        CompT sum = CompT(0);
        if (e > s) {
            if (kVec) {
                // whole aligned quads [vs, ve) in the middle, up to three single entries at either end;
                // the single entries are requested first and used last
                const int vs = (s + 3) >> 2;
                const int ve = e >> 2;
                const int headEnd = 4 * vs < e ? 4 * vs : e;
                const int ph = s + pl;
                const int pt = 4 * ve + pl;
                const bool doHead = pl < 4 && ph < headEnd;
                const bool doTail = pl < 4 && ve >= vs && pt < e;
                const int ch = doHead ? a.colInd[ph] : x0, ct = doTail ? a.colInd[pt] : x0;
                const ValT vh = doHead ? a.val[ph] : ValT(0), vt = doTail ? a.val[pt] : ValT(0);
                for (int v = vs + pl; v < ve; v += kUnroll * kPieceLanes) {
                    int4 c[kUnroll];
                    Quad<ValT> q[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int vv = v + kPieceLanes * u;
                        if (vv < ve) {
                            c[u] = __ldcs(reinterpret_cast<const int4 *>(a.colInd) + vv);
                            q[u] = LoadQuad(a.val + 4 * vv);
                        } else {
                            c[u] = make_int4(x0, x0, x0, x0);
#pragma unroll
                            for (int k = 0; k < 4; ++k) q[u].v[k] = ValT(0);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        sum += Widen<CompT>(q[u].v[0]) * Widen<CompT>(xrel[c[u].x]);
                        sum += Widen<CompT>(q[u].v[1]) * Widen<CompT>(xrel[c[u].y]);
                        sum += Widen<CompT>(q[u].v[2]) * Widen<CompT>(xrel[c[u].z]);
                        sum += Widen<CompT>(q[u].v[3]) * Widen<CompT>(xrel[c[u].w]);
                    }
                }
                sum += Widen<CompT>(vh) * Widen<CompT>(xrel[ch]) + Widen<CompT>(vt) * Widen<CompT>(xrel[ct]);
            } else {
                for (int p = s + pl; p < e; p += kPieceLanes)
                    sum += Widen<CompT>(a.val[p]) * Widen<CompT>(xrel[a.colInd[p]]);
            }
        }
        sCur = sNext;
        eCur = eNext;
        sum = GroupSum(sum, kPieceLanes);
        if (pl == 0 && slot < nLong) a.partials[(long long)slot * a.xBlocks + b] = sum;
    }

    // The CTAs (0..xBlocks-1, g) share the rows of group g: the last of them to get here adds
    // each row's partial sums in block order and writes y.
    __shared__ int sLast;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(a.counters + g, 1);
        sLast = (old == a.xBlocks - 1);
        if (sLast) a.counters[g] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sLast) return;
    __threadfence();
    const CompT alpha = a.sc.Alpha();
    const CompT beta = a.sc.Beta();
    for (int i = tid; i < trips * kPiecesPerCta; i += kLongThreads) {
        const int slot = g * kPiecesPerCta + (i % kPiecesPerCta) + (i / kPiecesPerCta) * stride;
        if (slot >= nLong) continue;
        CompT total = CompT(0);
        const CompT *part = a.partials + (long long)slot * a.xBlocks;
        for (int bb = 0; bb < a.xBlocks; bb += 8) {  // eight loads in flight, added in block order
            CompT pv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pv[k] = bb + k < a.xBlocks ? __ldcg(part + bb + k) : CompT(0);
#pragma unroll
            for (int k = 0; k < 8; ++k) total += pv[k];
        }
        const int r = a.longRows[slot];
        CompT z = alpha * total;
        if (beta != CompT(0)) z += beta * Widen<CompT>(a.y[r]);
        a.y[r] = Narrow<OutT>(z);
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

// A second stream (and the two events that fork it from / join it to the caller's stream) per
// device, created at first use.  Holds no device memory.
struct SideLane {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};

SideLane *GetSideLane()
{
    static SideLane lanes[64];
    static bool ready[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ready[dev]) {
        SideLane &l = lanes[dev];
        if (cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&l.join, cudaEventDisableTiming) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;  // fall back to one stream
        }
        ready[dev] = true;
    }
    return &lanes[dev];
}

template <typename CompT, typename ValT, typename OutT, bool kVec>
int LaunchLong(const LongArgs<CompT, ValT, OutT> &la, int blocks, cudaStream_t stream)
{
    static bool configured = false;  // this instantiation may use kXBlockBytes of dynamic shared memory
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(SpmvLongRowKernel<CompT, ValT, OutT, kVec>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kXBlockBytes);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    SpmvLongRowKernel<CompT, ValT, OutT, kVec><<<(unsigned)blocks, kLongThreads, kXBlockBytes, stream>>>(la);
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

template <typename CompT, typename ValT, typename OutT>
int LaunchTyped(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, void *y, int64_t rows,
                int64_t nnz, const b200spScalars *s, void *plan, cudaStream_t stream, int64_t cols = 0,
                int32_t longRows = 0)
{
    const Scalars<CompT> sc = MakeScalars<CompT>(s);
    if (plan != nullptr) {
        const PlanLayout L = LayoutFor(rows, nnz, cols, (int)sizeof(ValT));
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
        a.tileFlags = reinterpret_cast<const int32_t *>(p + L.offFlags);
        a.tileSkip = reinterpret_cast<const int32_t *>(p + L.offSkip);
        const bool useLong = longRows > 0 && L.capLong > 0;
        a.longLen = useLong ? kLongLen : kNoLongRows;
        const bool vec = (reinterpret_cast<uintptr_t>(colInd) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(val) % (4 * sizeof(ValT)) == 0);
        auto launchTiles = [&]() {
            if (vec) SpmvTileKernel<CompT, ValT, OutT, true><<<(unsigned)L.ntiles, kTileThreads, 0, stream>>>(a);
            else SpmvTileKernel<CompT, ValT, OutT, false><<<(unsigned)L.ntiles, kTileThreads, 0, stream>>>(a);
            b200sp_note_launches(1);
            return (int)cudaGetLastError();
        };
        if (!useLong) return launchTiles();

        LongArgs<CompT, ValT, OutT> la;
        la.colInd = colInd;
        la.val = static_cast<const ValT *>(val);
        la.x = static_cast<const ValT *>(x);
        la.y = static_cast<OutT *>(y);
        la.cols = (int)cols;
        la.nnz = (int)nnz;
        la.sc = sc;
        la.hdr = reinterpret_cast<const LongHeader *>(p + L.offLongHeader);
        la.longRows = reinterpret_cast<const int32_t *>(p + L.offLongRows);
        la.segStart = reinterpret_cast<const int32_t *>(p + L.offSegStart);
        la.counters = reinterpret_cast<int32_t *>(p + L.offLongCounters);
        la.partials = reinterpret_cast<CompT *>(p + L.offLongPartials);
        la.xBlocks = L.xBlocks;
        la.xBlockElems = L.xBlockElems;
        const int sms = b200sp_sm_count();
        int groups = sms / L.xBlocks;  // one wave: every CTA holds 128 KB of shared memory
        const int maxGroups = (longRows + kLongThreads / B200SP_SPMV_PIECE_LANES - 1) / (kLongThreads / B200SP_SPMV_PIECE_LANES);
        if (groups > maxGroups) groups = maxGroups;
        if (groups < 1) groups = 1;
        la.groups = groups;
        // The two kernels write disjoint rows of y: the long-row kernel runs on a side stream
        // forked from and joined back into the caller's stream, so they share the SMs.
        SideLane *lane = GetSideLane();
        cudaStream_t longStream = stream;
        if (lane != nullptr) {
            cudaError_t e = cudaEventRecord(lane->fork, stream);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(lane->stream, lane->fork, 0);
            if (e != cudaSuccess) return (int)e;
            longStream = lane->stream;
        }
        int rc = vec ? LaunchLong<CompT, ValT, OutT, true>(la, groups * L.xBlocks, longStream)
                     : LaunchLong<CompT, ValT, OutT, false>(la, groups * L.xBlocks, longStream);
        if (rc != 0) return rc;
        if (lane != nullptr) {
            const cudaError_t e = cudaEventRecord(lane->join, lane->stream);
            if (e != cudaSuccess) return (int)e;
        }
        rc = launchTiles();
        if (rc != 0) return rc;
        if (lane != nullptr) return (int)cudaStreamWaitEvent(stream, lane->join, 0);
        return 0;
    }
    if (rows == 0) return 0;
    const int G = GroupWidthFor(rows, nnz);
    const int64_t wantBlocks = (rows * G + 255) / 256;
    const int64_t maxBlocks = (int64_t)b200sp_sm_count() * 32;
    const unsigned blocks = (unsigned)(wantBlocks < maxBlocks ? wantBlocks : maxBlocks);
    SpmvRowGroupKernel<CompT, ValT, OutT><<<blocks, 256, 0, stream>>>(
        rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), static_cast<OutT *>(y),
        (int)rows, sc, G);
    b200sp_note_launches(1);
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
        b200sp_note_launches(1);
        if (rows > 0) {
            SpmvTransScatterKernel<CompT, ValT, float><<<rowBlocks, 256, 0, stream>>>(
                rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), acc, (int)rows, sc, G);
            b200sp_note_launches(1);
        }
        SpmvTransNarrowKernel<OutT><<<eltBlocks, 256, 0, stream>>>(acc, static_cast<OutT *>(y), (int)cols);
        b200sp_note_launches(1);
    } else {
        OutT *acc = static_cast<OutT *>(y);
        SpmvTransScaleKernel<CompT, OutT, OutT><<<eltBlocks, 256, 0, stream>>>(acc, acc, (int)cols, sc);
        b200sp_note_launches(1);
        if (rows > 0) {
            SpmvTransScatterKernel<CompT, ValT, OutT><<<rowBlocks, 256, 0, stream>>>(
                rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), acc, (int)rows, sc, G);
            b200sp_note_launches(1);
        }
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

namespace {
int ValueBytes(int valType)
{
    switch (valType) {
        case B200SP_F16: case B200SP_BF16: return 2;
        case B200SP_I8: return 1;
        default: return 4;
    }
}
}  // namespace

size_t b200sp_spmv_plan_bytes(int64_t rows, int64_t cols, int64_t nnz, int val_type)
{
    return LayoutFor(rows, nnz, cols, ValueBytes(val_type)).total;
}

int b200sp_spmv_analyze(const int32_t *row_ptr, const int32_t *col_ind, int64_t rows, int64_t cols, int64_t nnz,
                        int val_type, void *plan, size_t plan_bytes, int32_t *long_rows, void *stream)
{
    // Without a place to report the long-row count the tile-only layout is used (cols = 0).
    const PlanLayout L = LayoutFor(rows, nnz, long_rows != nullptr ? cols : 0, ValueBytes(val_type));
    if (long_rows != nullptr) *long_rows = 0;
    if (plan == nullptr || plan_bytes < L.total) return (int)cudaErrorInvalidValue;
    if (L.ntiles == 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *p = static_cast<char *>(plan);
    const unsigned blocks = (unsigned)((L.ntiles + 1 + 255) / 256);
    SpmvTileSearchKernel<<<blocks, 256, 0, st>>>(row_ptr, (int)rows, (int)nnz, (int)L.ntiles,
                                                 reinterpret_cast<int32_t *>(p + L.offTileRow),
                                                 reinterpret_cast<int32_t *>(p + L.offCounters),
                                                 reinterpret_cast<int32_t *>(p + L.offFlags));
    b200sp_note_launches(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || long_rows == nullptr || L.capLong == 0 || col_ind == nullptr) return (int)e;

    // Long-row part: list the rows, check their column order, cut them at the x-block borders.
    auto *hdr = reinterpret_cast<LongHeader *>(p + L.offLongHeader);
    auto *rowsList = reinterpret_cast<int32_t *>(p + L.offLongRows);
    e = cudaMemsetAsync(hdr, 0, 256, st);
    if (e != cudaSuccess) return (int)e;
    const int sms = b200sp_sm_count();
    const long long want = (rows + 255) / 256;
    SpmvFindLongRowsKernel<<<(unsigned)(want < sms * 16LL ? want : sms * 16LL), 256, 0, st>>>(
        row_ptr, (int)rows, hdr, rowsList, reinterpret_cast<int32_t *>(p + L.offLongCounters));
    b200sp_note_launches(1);
    SpmvMarkLongRowsKernel<<<(unsigned)(sms * 4), 256, 0, st>>>(
        row_ptr, col_ind, hdr, rowsList, reinterpret_cast<const int32_t *>(p + L.offTileRow),
        reinterpret_cast<int32_t *>(p + L.offFlags), reinterpret_cast<int32_t *>(p + L.offSkip), rows + nnz);
    b200sp_note_launches(1);
    SpmvLongSegmentsKernel<<<(unsigned)(sms * 8), 256, 0, st>>>(row_ptr, col_ind, hdr, rowsList,
                                                                reinterpret_cast<int32_t *>(p + L.offSegStart),
                                                                L.xBlocks, L.xBlockElems);
    b200sp_note_launches(1);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    LongHeader host{};
    e = cudaMemcpyAsync(&host, hdr, sizeof(host), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    *long_rows = host.unsorted ? 0 : host.count;  // unsorted long rows stay in the tiles
    return 0;
}

int b200sp_spmv_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x, void *y,
                       int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars, int comp_type,
                       int val_type, int out_type, void *plan, int32_t long_rows, void *stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rc = DispatchTypes(comp_type, val_type, out_type, [&]<typename C, typename V, typename O>() {
        // the tile arrays sit at the same offsets whether or not the plan has a long-row part
        return LaunchTyped<C, V, O>(row_ptr, col_ind, val, x, y, rows, nnz, scalars, plan, st,
                                    long_rows > 0 ? cols : 0, long_rows);
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
constexpr size_t kNoAllocBytes = 20 * ((size_t)(kNoAllocMaxItems / kTileItems) + 2) + 6 * 256 + 256;
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
    const int an = b200sp_spmv_analyze(row_ptr, nullptr, rows, 0, nnz, B200SP_F32, scratch, kNoAllocBytes, nullptr, stream);
    if (an != 0) return an;
    b200spScalars sc{};
    sc.alpha_f = alpha;
    sc.beta_f = beta;
    return LaunchTyped<float, float, float>(row_ptr, col_ind, val, x, y, rows, nnz, &sc, scratch,
                                            static_cast<cudaStream_t>(stream));
}
