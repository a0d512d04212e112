// CSR SpMV kernels for sm_100a and their extern "C" launchers.
//
// The reference's device code for this operator (sparse/spmv/arch22/kernels/spmv_kernel.h:
// 27-310 non-transpose, 321-640 transpose) gives every core an equal count of rows and
// walks them one at a time.  Two designs replace it here, chosen by what the caller set up.
//
// Binned path (a buffer analysed once by aclsparseSpMVPreprocess / b200sp_spmv_analyze with
// plan_info).  The analysis lists the rows of 33..1023 entries ("medium") and of >= 1024
// entries ("long", ordered by descending length) as {row, start, end}; a product is then two
// launches over disjoint rows of y, the first forked onto a side stream so that they share
// the SMs:
//   SpmvLongBlockKernel     (enough long rows -- 48 per block of x --, ascending columns, at most 2 M columns)
//                           x is cut into blocks of 32768 columns; a CTA keeps one block in
//                           shared memory and sums the pieces of all long rows that fall into
//                           it, so the gathers of more than half of the non-zeros of a
//                           power-law matrix never leave the SM.  The last CTA to finish a group
//                           of rows adds their per-block partial sums in block order.
//   SpmvAllBinsKernel       (otherwise) one grid for all bins: a CTA per listed long row with 128-bit
//                           loads first, then the medium and short rows as below; no side stream.
//   SpmvMediumShortKernel   one grid: first a warp per listed medium row, then every row gets
//                           a group of G = 2 or 4 lanes (rows longer than 32 entries are
//                           skipped).  SpmvShortRowsKernel alone when no row is medium.
// Gathers of x from scattered columns cost one L2 sector request each, and an SM issues one
// request per clock: many light warps, each with a few independent gathers in flight, keep
// that port busy for the medium and short rows, and the long rows stay off it altogether.
//
// Tile path (no analysed buffer: the tile table is rebuilt into the handle workspace on every
// call, no host synchronisation; also the entry point that allocates nothing).  The work is
// cut by *merge path*: the rows' end markers and the non-zeros form one merged sequence of
// rows + nnz items and every CTA takes an equal slice (a tile) of it, whatever the row
// lengths are.  A tile
//   1. streams its slice of col_ind / values with 128-bit evict-first loads, gathers x
//      through the read-only path and parks the products in shared memory;
//   2. lets every thread walk 15 consecutive merge items (add a product, or close a row),
//      then joins rows that span threads with a segmented scan over the threads' carries;
//   3. writes y with one coalesced pass (alpha * sum + beta * y).
// A row cut by a tile boundary is finished without a second kernel and without waiting:
// every tile that holds a piece stores its partial sum, then bumps an arrival counter owned
// by the tile in which the row ends; whichever tile arrives last adds the pieces in tile
// order (so the result does not depend on scheduling) and writes y.
//
// Numerics follow the reference golden SpmvCpu (test/spmv/arch22/spmv_test.cpp:156-173):
// values and x are widened to the compute type before the multiply, sums are kept in the
// compute type, the result is alpha*sum + beta*y rounded once to the output type.
// beta == 0 never reads y.
#include <atomic>
#include <cstdint>
#include <cstdio>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "../common/side_stream.h"

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

// Rows of at least kLongLen entries form the "long" bin of the binned path (see below).  Measured on the
// 1,048,576-row power-law matrix (us per product): 1024: 95.0, 768: 94.5, 512: 90.6, 384: 104.2.
#ifndef B200SP_SPMV_LONG_LEN
#define B200SP_SPMV_LONG_LEN 512
#endif
constexpr int kLongLen = B200SP_SPMV_LONG_LEN;

// Long rows that keep CTAs of their own (the list path) are cut into segments of kSegLen entries, a CTA each: a
// 16384-entry row is then eight CTAs working side by side instead of one CTA making eight round trips to memory,
// which is what bounded a product on a small shard.  A row of several segments is finished by whichever of its
// CTAs arrives last: it adds the segments' partial sums in segment order (no wait, fixed order).
// One eighth of the power-law matrix (131,081 rows, 978 long ones, 3.8 M entries), whole product: segments of
// 2048 / 4096 / 8192 entries 22.6 / 21.9 / 20.6 us; one sixteenth: 14.4 / 14.0 / 14.4.
#ifndef B200SP_SPMV_SEG_LEN
#define B200SP_SPMV_SEG_LEN 8192
#endif
constexpr int kSegLen = B200SP_SPMV_SEG_LEN;


struct PlanLayout {  // tile plan: what SpmvTileKernel needs
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
            a.partTail[t] = scan;  // key == R here: the run of carries that ends the tile
            arrive(i1, (int)(((long long)i1 + a.rowPtr[i1 + 1]) / kTileItems));
        }
    }
}

// ---------------------------------------------------------------- binned path

// Rows are binned by length by the analysis pass and each bin has its own code:
//   short  (<= kShortMax entries)   ShortRowsBody : G = 2 or 4 lanes per row (8 compiles, for experiments), all rows scanned
//   medium (<  kLongLen entries)    MediumRowsBody: one warp per listed row
//   long   (>= kLongLen entries)    SpmvLongBlockKernel (x blocks in shared memory) or LongRowBody (a CTA per row)
// Short and medium rows share one grid; the long rows run beside it on a side stream.
#ifndef B200SP_SPMV_SHORT_MAX
#define B200SP_SPMV_SHORT_MAX 32
#endif
constexpr int kShortMax = B200SP_SPMV_SHORT_MAX;
#ifndef B200SP_SPMV_LONG_UNROLL
#define B200SP_SPMV_LONG_UNROLL 4
#endif
constexpr int kLongUnroll = B200SP_SPMV_LONG_UNROLL;  // quads in flight per thread of the long-row kernel

struct BinHeader {  // first 256 bytes of the binned plan
    int32_t medium;           // rows in the medium list
    int32_t longs;            // rows in the long list
    unsigned long long shortNnz;  // entries in short rows (picks the lane-group width)
    int32_t shortRows;
    int32_t unsorted;         // set when a long row has descending column indices
    int32_t segments;         // segments the long rows were cut into
};

// Long rows, second form: x is cut into blocks of kXBlockElems columns and every CTA of
// SpmvLongBlockKernel keeps one block in shared memory, so the gathers of the long rows never
// leave the SM (the other bins keep the L1 -> L2 request path to themselves).
#ifndef B200SP_SPMV_XBLOCK_ELEMS
#define B200SP_SPMV_XBLOCK_ELEMS 32768
#endif
#ifndef B200SP_SPMV_LONG_BLOCK_THREADS
#define B200SP_SPMV_LONG_BLOCK_THREADS 1024
#endif
#ifndef B200SP_SPMV_LONG_BLOCK_UNROLL
#define B200SP_SPMV_LONG_BLOCK_UNROLL 2
#endif
constexpr int kXBlockElems = B200SP_SPMV_XBLOCK_ELEMS;  // 128 KB of fp32 x, 64 KB of 16-bit x
constexpr int kMaxXBlocks = 64;      // wider matrices use SpmvLongListKernel
constexpr int kMaxLongGroups = 64;   // CTAs per column block
constexpr int kLongBlockThreads = B200SP_SPMV_LONG_BLOCK_THREADS;
#ifndef B200SP_SPMV_PIECE_LANES
#define B200SP_SPMV_PIECE_LANES 8    // lanes that share one (long row, x block) piece
#endif
#ifndef B200SP_SPMV_FUSE_LIST
#define B200SP_SPMV_FUSE_LIST 1      // long rows that keep a CTA each share one grid with the other bins
#endif
#ifndef B200SP_SPMV_MIN_LONG_BLOCKED
#define B200SP_SPMV_MIN_LONG_BLOCKED 64  // fewer long rows than this: not worth staging x
#endif

__global__ void SpmvBinRowsKernel(const int32_t *__restrict__ rowPtr, int rows, BinHeader *hdr,
                                  int4 *__restrict__ listM, int4 *__restrict__ listL)
{
    const int lane = threadIdx.x & 31;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long rowsPadded = ((long long)rows + stride - 1) / stride * stride;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rowsPadded; r += stride) {
        int shortLen = 0, isShort = 0;
        if (r < rows) {
            const int rs = rowPtr[r], re = rowPtr[r + 1];
            const int len = re - rs;
            // a list entry carries the row's bounds, so its kernel starts on col_ind / values at once
            if (len >= kLongLen) listL[atomicAdd(&hdr->longs, 1)] = make_int4((int)r, rs, re, 0);
            else if (len > kShortMax) listM[atomicAdd(&hdr->medium, 1)] = make_int4((int)r, rs, re, 0);
            else {
                shortLen = len;
                isShort = 1;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            shortLen += __shfl_xor_sync(0xffffffffu, shortLen, off);
            isShort += __shfl_xor_sync(0xffffffffu, isShort, off);
        }
        if (lane == 0 && isShort) {
            atomicAdd(&hdr->shortNnz, (unsigned long long)shortLen);
            atomicAdd(&hdr->shortRows, isShort);
        }
    }
}

// Orders a list of {row, start, end} entries by descending row length (in classes of an
// eighth of an octave; the order inside a class is arbitrary and no result depends on it), so
// that the longest rows start first and the rows that share a warp or a CTA are alike.
// One CTA: the lists hold thousands of rows, not millions.
__global__ void __launch_bounds__(1024) SpmvSortByLengthKernel(const int32_t *__restrict__ count,
                                                                const int4 *__restrict__ in, int4 *__restrict__ out)
{
    __shared__ int sHist[256];
    const int tid = threadIdx.x;
    const int n = *count;
    auto lengthClass = [](int4 ent) {
        const int len = ent.z - ent.y;             // >= 33 for every listed row
        const int k = 31 - __clz(len);             // floor(log2(len)) >= 5
        const int key = k * 8 + ((len >> (k - 3)) & 7);
        return 255 - key;                          // descending
    };
    if (tid < 256) sHist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += 1024) atomicAdd(&sHist[lengthClass(in[i])], 1);
    __syncthreads();
    if (tid == 0) {
        int running = 0;
        for (int d = 0; d < 256; ++d) {
            const int c = sHist[d];
            sHist[d] = running;
            running += c;
        }
    }
    __syncthreads();
    for (int i = tid; i < n; i += 1024) {
        const int4 ent = in[i];
        out[atomicAdd(&sHist[lengthClass(ent)], 1)] = ent;
    }
}

// One CTA: segment table of the ordered long list.  Slot i (row r, entries [s, e)) gets ceil(len / kSegLen)
// consecutive entries {r, segment start, segment end, i} of `segs`, rowSeg[i] = {first partial slot, segments}, and
// a zeroed arrival counter; the order of `segs` is the order of the list (longest rows first).
__global__ void __launch_bounds__(1024) SpmvCutSegmentsKernel(BinHeader *hdr, const int4 *__restrict__ listL,
                                                               int4 *__restrict__ segs, int2 *__restrict__ rowSeg,
                                                               int32_t *__restrict__ counters)
{
    __shared__ int sWarp[32];
    __shared__ int sCarry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = hdr->longs;
    if (tid == 0) sCarry = 0;
    __syncthreads();
    for (int i0 = 0; i0 < n; i0 += 1024) {
        const int i = i0 + tid;
        int4 ent = make_int4(0, 0, 0, 0);
        int nseg = 0;
        if (i < n) {
            ent = listL[i];
            nseg = (ent.z - ent.y + kSegLen - 1) / kSegLen;
        }
        int incl = nseg;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) sWarp[warp] = incl;
        __syncthreads();
        int before = sCarry;
        for (int w = 0; w < warp; ++w) before += sWarp[w];
        const int first = before + incl - nseg;
        if (i < n) {
            rowSeg[i] = make_int2(first, nseg);
            counters[i] = 0;
            for (int k = 0; k < nseg; ++k) {
                const int a = ent.y + k * kSegLen;
                segs[first + k] = make_int4(ent.x, a, a + kSegLen < ent.z ? a + kSegLen : ent.z, i);
            }
        }
        __syncthreads();
        if (tid == 1023) sCarry = before + incl;
        __syncthreads();
    }
    if (tid == 0) hdr->segments = sCarry;
}

// One warp per listed long row: checks that its column indices ascend, then cuts it at the x
// block boundaries by binary search: segStart[slot * (xBlocks + 1) + b] = first entry of the row
// whose column is >= b * kXBlockElems.
__global__ void SpmvLongSegmentsKernel(const int32_t *__restrict__ colInd, BinHeader *hdr,
                                       const int4 *__restrict__ listL, int32_t *__restrict__ segStart,
                                       int xBlocks)
{
    const int lane = threadIdx.x & 31;
    const int warpsTotal = gridDim.x * (blockDim.x >> 5);
    const int n = hdr->longs;
    for (int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); slot < n; slot += warpsTotal) {
        const int4 ent = listL[slot];
        const int s = ent.y, e = ent.z;
        bool bad = false;
        for (int p = s + lane; p + 1 < e; p += 32) bad |= colInd[p] > colInd[p + 1];
        if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(&hdr->unsorted, 1);
        for (int b = lane; b <= xBlocks; b += 32) {
            int lo = s, hi = e;
            if (b == xBlocks) lo = hi;
            const long long bound = (long long)b * kXBlockElems;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (colInd[mid] < bound) lo = mid + 1;
                else hi = mid;
            }
            segStart[(long long)slot * (xBlocks + 1) + b] = lo;
        }
    }
}

template <typename CompT, typename ValT, typename OutT>
struct LongBlockArgs {
    const int32_t *colInd;
    const ValT *val;
    const ValT *x;
    OutT *y;
    int cols;
    Scalars<CompT> sc;
    const int4 *list;          // {row, start, end, 0} per long row
    const int32_t *segStart;   // [slot][xBlocks + 1]
    int32_t *counters;         // [group], arrivals of the group's column-block CTAs
    CompT *partials;           // [slot][xBlocks]
    int nLong;
    int xBlocks;
    int groups;                // CTAs per column block
};

// CTA (b, g) keeps block b of x in shared memory and sums, for every long row of its group,
// the entries whose column falls in that block -- a contiguous piece of the row, because the
// column indices ascend.  kPieceLanes lanes share a piece; x comes from shared memory, so the
// only global traffic is the col_ind / values stream.  The last CTA of a row group to finish
// adds each row's partial sums in block order (no wait, fixed order) and writes y.
// Registers are capped at 48 (not at the 64 a 1024-thread CTA could have): while this kernel holds an SM, the
// CTAs of the medium / short grid get what is left of the register file, and both grids are bound by latency x
// occupancy.  Timestamps taken inside the kernels on the power-law matrix: these CTAs run 30-43 us, all done 47 us
// after the first started; the medium rows beside them finish at 68 us instead of 35 alone, the short rows at
// 91.  Product time with 56 / 46 / 40 registers here: 90.2 / 86.4 / 89.2 us.
template <typename CompT, typename ValT, typename OutT, bool kVec>
__global__ void __maxnreg__(48) SpmvLongBlockKernel(const LongBlockArgs<CompT, ValT, OutT> a)
{
    extern __shared__ __align__(16) unsigned char sRaw[];
    ValT *xs = reinterpret_cast<ValT *>(sRaw);
    const int tid = threadIdx.x;
    const int b = blockIdx.x % a.xBlocks;
    const int g = blockIdx.x / a.xBlocks;
    const int nLong = a.nLong;
    const int x0 = b * kXBlockElems;
    const int xn = a.cols - x0 < kXBlockElems ? a.cols - x0 : kXBlockElems;

    // stage the x block
    constexpr int kPer16 = 16 / (int)sizeof(ValT);
    if (reinterpret_cast<uintptr_t>(a.x) % 16 == 0) {
        const int nv = xn / kPer16;
        const int4 *src = reinterpret_cast<const int4 *>(a.x + x0);  // x0 * sizeof(ValT) is a multiple of 16
        int4 *dst = reinterpret_cast<int4 *>(xs);
        for (int i = tid; i < nv; i += kLongBlockThreads) dst[i] = __ldg(src + i);
        for (int i = nv * kPer16 + tid; i < xn; i += kLongBlockThreads) xs[i] = a.x[x0 + i];
    } else {
        for (int i = tid; i < xn; i += kLongBlockThreads) xs[i] = a.x[x0 + i];
    }
    __syncthreads();

    const ValT *xrel = xs - x0;  // xrel[col] is x[col] for the columns of this block
    constexpr int kPieceLanes = B200SP_SPMV_PIECE_LANES;
    constexpr int kUnroll = B200SP_SPMV_LONG_BLOCK_UNROLL;  // quads in flight per lane
    constexpr int kPiecesPerCta = kLongBlockThreads / kPieceLanes;
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
    for (int i = tid; i < trips * kPiecesPerCta; i += kLongBlockThreads) {
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
        const int r = a.list[slot].x;
        CompT z = alpha * total;
        if (beta != CompT(0)) z += beta * Widen<CompT>(a.y[r]);
        a.y[r] = Narrow<OutT>(z);
    }
}

// The three bins as device functions of a block index `bid`.  (One fused grid with a role per
// block range was measured: no faster than three kernels on forked streams on the power-law
// matrix, 6-12 % slower on the banded one, so each bin is a kernel of its own.)
template <typename CompT, typename ValT, typename OutT, int G>
__device__ __forceinline__ void ShortRowsBody(unsigned bid, const int32_t *__restrict__ rowPtr,
                                              const int32_t *__restrict__ colInd, const ValT *__restrict__ val,
                                              const ValT *__restrict__ x, OutT *__restrict__ y, int rows,
                                              const Scalars<CompT> &sc)
{
    const int lane = threadIdx.x & (G - 1);
    const long long r = ((long long)bid * blockDim.x + threadIdx.x) / G;
    int s = 0, e = 0;
    if (r < rows) {
        s = rowPtr[r];
        e = rowPtr[r + 1];
    }
    const bool mine = r < rows && e - s <= kShortMax;  // longer rows belong to the other kernels
    if (!mine) e = s;
    const CompT beta = sc.Beta();
    CompT yOld = CompT(0);
    if (mine && lane == 0 && beta != CompT(0)) yOld = Widen<CompT>(y[r]);  // requested now, used at the end
    CompT sum = CompT(0);
    // up to four entries per lane in flight
    for (int p = s + lane; p < e; p += 4 * G) {
        int c[4];
        ValT v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool in = p + u * G < e;
            c[u] = in ? __ldcs(colInd + p + u * G) : 0;
            v[u] = in ? __ldcs(val + p + u * G) : ValT(0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const ValT xv = p + u * G < e ? __ldg(x + c[u]) : ValT(0);
            sum += Widen<CompT>(v[u]) * Widen<CompT>(xv);
        }
    }
    sum = GroupSum(sum, G);
    if (mine && lane == 0) {
        CompT z = sc.Alpha() * sum;
        if (beta != CompT(0)) z += beta * yOld;
        y[r] = Narrow<OutT>(z);
    }
}

template <typename CompT, typename ValT, typename OutT>
__device__ __forceinline__ void MediumRowsBody(unsigned bid, const int32_t *__restrict__ colInd,
                                               const ValT *__restrict__ val, const ValT *__restrict__ x,
                                               OutT *__restrict__ y, const int4 *__restrict__ list, int count,
                                               const Scalars<CompT> &sc)
{
    const int lane = threadIdx.x & 31;
    const int i = (int)bid * (int)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= count) return;  // whole warps leave together
    const int4 ent = __ldg(list + i);
    const int r = ent.x, s = ent.y, e = ent.z;
    const CompT beta = sc.Beta();
    CompT yOld = CompT(0);
    if (lane == 0 && beta != CompT(0)) yOld = Widen<CompT>(y[r]);  // requested now, used at the end
    CompT sum = CompT(0);
    for (int p = s + lane; p < e; p += 4 * 32) {
        int c[4];
        ValT v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool in = p + u * 32 < e;
            c[u] = in ? __ldcs(colInd + p + u * 32) : 0;
            v[u] = in ? __ldcs(val + p + u * 32) : ValT(0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const ValT xv = p + u * 32 < e ? __ldg(x + c[u]) : ValT(0);
            sum += Widen<CompT>(v[u]) * Widen<CompT>(xv);
        }
    }
    sum = GroupSum(sum, 32);
    if (lane == 0) {
        CompT z = sc.Alpha() * sum;
        if (beta != CompT(0)) z += beta * yOld;
        y[r] = Narrow<OutT>(z);
    }
}

struct LongSegs {             // the long rows cut into segments (see SpmvCutSegmentsKernel)
    const int4 *segs;         // {row, start, end, slot}
    const int4 *list;         // {row, row start, row end, 0} per slot
    const int2 *rowSeg;       // {first partial slot, segments} per slot
    int32_t *counters;        // arrivals per slot
    void *partials;           // one compute-type value per segment
};

template <typename CompT, typename ValT, typename OutT, bool kVec, int kUnrollQ = kLongUnroll>
__device__ __forceinline__ void LongRowBody(unsigned bid, const int32_t *__restrict__ colInd,
                                            const ValT *__restrict__ val, const ValT *__restrict__ x,
                                            OutT *__restrict__ y, const LongSegs &ls, const Scalars<CompT> &sc,
                                            CompT *sWarp)
{
    const int tid = threadIdx.x;
    const int4 ent = __ldg(ls.segs + bid);
    const int r = ent.x, s = ent.y, e = ent.z, slot = ent.w;
    const int2 rs = __ldg(ls.rowSeg + slot);  // {first partial slot, segments of this row}
    const CompT beta = sc.Beta();
    CompT yOld = CompT(0);
    if (tid == 0 && rs.y == 1 && beta != CompT(0)) yOld = Widen<CompT>(y[r]);  // requested now, used at the end
    CompT sum = CompT(0);
    if (kVec) {
        // whole aligned quads [vs, ve); up to three single entries before and after them
        const int vs = (s + 3) >> 2, ve = e >> 2;
        const int headEnd = 4 * vs < e ? 4 * vs : e;
        const int ph = s + tid, pt = 4 * ve + (tid - 4);
        const bool doHead = tid < 4 && ph < headEnd;
        const bool doTail = tid >= 4 && tid < 8 && ve >= vs && pt < e;
        const int pe = doHead ? ph : pt;
        const int ce = (doHead || doTail) ? colInd[pe] : 0;
        const ValT vE = (doHead || doTail) ? val[pe] : ValT(0);
        for (int v = vs + tid; v < ve; v += kUnrollQ * 256) {
            int4 c[kUnrollQ];
            Quad<ValT> q[kUnrollQ];
#pragma unroll
            for (int u = 0; u < kUnrollQ; ++u) {
                const int vv = v + 256 * u;
                if (vv < ve) {
                    c[u] = __ldcs(reinterpret_cast<const int4 *>(colInd) + vv);
                    q[u] = LoadQuad(val + 4 * vv);
                } else {
                    c[u] = make_int4(0, 0, 0, 0);
#pragma unroll
                    for (int k = 0; k < 4; ++k) q[u].v[k] = ValT(0);
                }
            }
#pragma unroll
            for (int u = 0; u < kUnrollQ; ++u) {
                if (v + 256 * u < ve) {
                    sum += Widen<CompT>(q[u].v[0]) * Widen<CompT>(__ldg(x + c[u].x));
                    sum += Widen<CompT>(q[u].v[1]) * Widen<CompT>(__ldg(x + c[u].y));
                    sum += Widen<CompT>(q[u].v[2]) * Widen<CompT>(__ldg(x + c[u].z));
                    sum += Widen<CompT>(q[u].v[3]) * Widen<CompT>(__ldg(x + c[u].w));
                }
            }
        }
        if (doHead || doTail) sum += Widen<CompT>(vE) * Widen<CompT>(__ldg(x + ce));
    } else {
        for (int p = s + tid; p < e; p += 256) sum += Widen<CompT>(val[p]) * Widen<CompT>(__ldg(x + colInd[p]));
    }
    sum = GroupSum(sum, 32);
    if ((tid & 31) == 0) sWarp[tid >> 5] = sum;
    __syncthreads();
    if (tid == 0) {
        CompT tot = CompT(0);
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += sWarp[w];
        if (rs.y > 1) {
            // one of several segments: leave the partial sum, and finish the row if this CTA is the last to arrive
            CompT *part = static_cast<CompT *>(ls.partials) + rs.x;
            const int rowStart = __ldg(ls.list + slot).y;
            part[(s - rowStart) / kSegLen] = tot;
            __threadfence();
            const int old = atomicAdd(ls.counters + slot, 1);
            if (old != rs.y - 1) return;
            ls.counters[slot] = 0;  // ready for the next launch
            __threadfence();
            tot = CompT(0);
            for (int k = 0; k < rs.y; ++k) tot += __ldcg(part + k);  // segment order: the sum does not depend on timing
            if (beta != CompT(0)) yOld = Widen<CompT>(y[r]);
        }
        CompT z = sc.Alpha() * tot;
        if (beta != CompT(0)) z += beta * yOld;
        y[r] = Narrow<OutT>(z);
    }
}

template <typename CompT, typename ValT, typename OutT, int G>
__global__ void __launch_bounds__(256) SpmvShortRowsKernel(const int32_t *__restrict__ rowPtr,
                                                            const int32_t *__restrict__ colInd,
                                                            const ValT *__restrict__ val,
                                                            const ValT *__restrict__ x, OutT *__restrict__ y,
                                                            int rows, Scalars<CompT> sc)
{
    ShortRowsBody<CompT, ValT, OutT, G>(blockIdx.x, rowPtr, colInd, val, x, y, rows, sc);
}

// Medium and short rows in one grid: blocks [0, ceil(nM / 8)) take eight listed medium rows
// each (the longer pieces of work start first), the rest sweep all rows for the short ones.
// One launch instead of two streams: whether two large grids on different streams really
// overlap depends on how the driver maps streams to hardware queues, which a library cannot see.
template <typename CompT, typename ValT, typename OutT, int G>
__global__ void __launch_bounds__(256) SpmvMediumShortKernel(const int32_t *__restrict__ rowPtr,
                                                              const int32_t *__restrict__ colInd,
                                                              const ValT *__restrict__ val,
                                                              const ValT *__restrict__ x, OutT *__restrict__ y,
                                                              const int4 *__restrict__ listM, int nM, int rows,
                                                              Scalars<CompT> sc)
{
    const unsigned wpc = blockDim.x >> 5;
    const unsigned mediumBlocks = ((unsigned)nM + wpc - 1u) / wpc;
    if (blockIdx.x < mediumBlocks) MediumRowsBody<CompT, ValT, OutT>(blockIdx.x, colInd, val, x, y, listM, nM, sc);
    else ShortRowsBody<CompT, ValT, OutT, G>(blockIdx.x - mediumBlocks, rowPtr, colInd, val, x, y, rows, sc);
}

template <typename CompT, typename ValT, typename OutT, bool kVec>
__global__ void __launch_bounds__(256) SpmvLongListKernel(const int32_t *__restrict__ colInd,
                                                           const ValT *__restrict__ val,
                                                           const ValT *__restrict__ x, OutT *__restrict__ y,
                                                           LongSegs ls, Scalars<CompT> sc)
{
    __shared__ CompT sWarp[8];
    LongRowBody<CompT, ValT, OutT, kVec>(blockIdx.x, colInd, val, x, y, ls, sc, sWarp);
}

// All three bins in one grid, for matrices whose long rows keep a CTA each: blocks [0, nL) take one long
// row, the next ceil(nM / 8) eight medium rows, the rest sweep the short rows.  Blocks are handed out in
// index order, so the longest pieces of work start first.  One launch and no fork / join: on a
// 131,000-row shard the two-stream form spent more time between its kernels than in them.
template <typename CompT, typename ValT, typename OutT, int G, bool kVec>
__global__ void __launch_bounds__(256, 6) SpmvAllBinsKernel(const int32_t *__restrict__ rowPtr,
                                                             const int32_t *__restrict__ colInd,
                                                             const ValT *__restrict__ val, const ValT *__restrict__ x,
                                                             OutT *__restrict__ y, const int4 *__restrict__ listM,
                                                             LongSegs ls, int nM, int nL, int rows,
                                                             Scalars<CompT> sc)
{
    __shared__ CompT sWarp[8];
    unsigned b = blockIdx.x;
    if (b < (unsigned)nL) {  // nL counts segments here
        LongRowBody<CompT, ValT, OutT, kVec, 2>(b, colInd, val, x, y, ls, sc, sWarp);
        return;
    }
    b -= (unsigned)nL;
    const unsigned mediumBlocks = ((unsigned)nM + 7u) >> 3;
    if (b < mediumBlocks) MediumRowsBody<CompT, ValT, OutT>(b, colInd, val, x, y, listM, nM, sc);
    else ShortRowsBody<CompT, ValT, OutT, G>(b - mediumBlocks, rowPtr, colInd, val, x, y, rows, sc);
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

__global__ void SpmvMaxRowLengthKernel(const int32_t *__restrict__ rowPtr, int rows, int32_t *__restrict__ out)
{
    int best = 0;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
         r += (long long)gridDim.x * blockDim.x) {
        const int len = rowPtr[r + 1] - rowPtr[r];
        best = len > best ? len : best;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const int o = __shfl_xor_sync(0xffffffffu, best, off);
        best = o > best ? o : best;
    }
    if ((threadIdx.x & 31) == 0 && best > 0) atomicMax(out, best);
}

// The same scatter cut by non-zeros instead of rows: a warp takes kTransChunk consecutive entries,
// whatever rows they belong to, and every lane finds the row of its entry by a binary search among
// the rows the chunk touches.  A scatter needs no per-row reduction, so a row of 16384 entries is
// simply spread over 64 warps; with a lane group per row it is one warp's 512 sequential trips.
constexpr int kTransChunk = 256;
template <typename CompT, typename ValT, typename AccT>
__global__ void __launch_bounds__(256) SpmvTransScatterNnzKernel(const int32_t *__restrict__ rowPtr,
                                                                  const int32_t *__restrict__ colInd,
                                                                  const ValT *__restrict__ val,
                                                                  const ValT *__restrict__ x,
                                                                  AccT *__restrict__ acc, int rows, int nnz,
                                                                  Scalars<CompT> sc)
{
    const CompT alpha = sc.Alpha();
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    const long long chunks = ((long long)nnz + kTransChunk - 1) / kTransChunk;
    auto rowOf = [&](int p, int lo, int hi) {  // largest r in [lo, hi] with rowPtr[r] <= p
        while (lo < hi) {
            const int mid = lo + ((hi - lo + 1) >> 1);
            if (__ldg(rowPtr + mid) <= p) lo = mid;
            else hi = mid - 1;
        }
        return lo;
    };
    // The same for a p that all lanes share: 32 probes per round instead of one (rowPtr[lo] <= p is given).
    auto warpRowOf = [&](int p, int lo, int hi) {
        while (hi > lo) {
            const long long span = (long long)hi - lo;
            if (span <= 32) {
                const int cand = lo + 1 + lane;
                const bool ok = cand <= hi && __ldg(rowPtr + cand) <= p;
                lo += __popc(__ballot_sync(0xffffffffu, ok));  // the probes are monotone
                break;
            }
            const int cand = lo + (int)((lane + 1) * span / 32);  // lane 31 probes hi
            const bool ok = __ldg(rowPtr + cand) <= p;
            const int k = __popc(__ballot_sync(0xffffffffu, ok));
            const int newLo = k == 0 ? lo : lo + (int)((long long)k * span / 32);
            const int newHi = k == 32 ? hi : lo + (int)((long long)(k + 1) * span / 32) - 1;
            lo = newLo;
            hi = newHi;
        }
        return lo;
    };
    for (long long c = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < chunks; c += warpsTotal) {
        const int c0 = (int)(c * kTransChunk);
        const int c1 = c0 + kTransChunk < nnz ? c0 + kTransChunk : nnz;
        const int rFirst = warpRowOf(c0, 0, rows - 1);
        const int rLast = warpRowOf(c1 - 1, rFirst, rows - 1);
        for (int p = c0 + lane; p < c1; p += 32) {
            const int r = rowOf(p, rFirst, rLast);
            const CompT xv = alpha * Widen<CompT>(__ldg(x + r));
            if (xv == CompT(0)) continue;
            atomicAdd(acc + __ldcs(colInd + p), static_cast<AccT>(xv * Widen<CompT>(__ldcs(val + p))));
        }
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
#ifdef B200SP_SPMV_FORCE_G
    return B200SP_SPMV_FORCE_G;
#endif
    const int64_t avg = rows > 0 ? nnz / rows : 0;
    int G = 1;
    while (G < 32 && G < avg) G <<= 1;
    return G;
}

// Binned plan in the caller's buffer: header, list of medium rows, list of long rows and, when
// the matrix is narrow enough for the blocked long-row kernel, that kernel's tables.
struct BinLayout {
    int64_t capM, capL, capS;
    int32_t xBlocks;  // column blocks of x; 0 = the blocked long-row kernel is not available
    size_t offHeader, offListM, offListL, offTmpL, offSegStart, offLongCounters, offPartials, offSegs, offRowSeg,
        offSegCounters, offSegPartials, total;
};

inline BinLayout BinLayoutFor(int64_t rows, int64_t cols, int64_t nnz)
{
    BinLayout L;
    const int64_t byNnz = nnz / (kShortMax + 1);
    L.capM = (byNnz < rows ? byNnz : rows) + 1;
    L.capL = nnz / kLongLen + 1;
    const int64_t xb = (cols + kXBlockElems - 1) / kXBlockElems;
    L.xBlocks = (xb >= 1 && xb <= kMaxXBlocks && nnz / kLongLen >= B200SP_SPMV_MIN_LONG_BLOCKED) ? (int32_t)xb : 0;
    L.offHeader = 0;
    L.offListM = 256;
    L.offListL = AlignUp(L.offListM + sizeof(int4) * (size_t)L.capM, 256);
    L.offTmpL = AlignUp(L.offListL + sizeof(int4) * (size_t)L.capL, 256);  // long rows as found, before ordering
    L.offSegStart = AlignUp(L.offTmpL + sizeof(int4) * (size_t)L.capL, 256);
    L.offLongCounters = AlignUp(L.offSegStart + sizeof(int32_t) * (size_t)L.capL * (L.xBlocks > 0 ? L.xBlocks + 1 : 0), 256);
    L.offPartials = AlignUp(L.offLongCounters + sizeof(int32_t) * kMaxLongGroups, 256);
    L.capS = nnz / kSegLen + L.capL;  // a row of len entries has at most len / kSegLen + 1 segments
    L.offSegs = AlignUp(L.offPartials + 4 * (size_t)L.capL * L.xBlocks, 256);
    L.offRowSeg = AlignUp(L.offSegs + sizeof(int4) * (size_t)L.capS, 256);
    L.offSegCounters = AlignUp(L.offRowSeg + sizeof(int2) * (size_t)L.capL, 256);
    L.offSegPartials = AlignUp(L.offSegCounters + sizeof(int32_t) * (size_t)L.capL, 256);
    L.total = AlignUp(L.offSegPartials + 4 * (size_t)L.capS, 256);
    return L;
}

// plan_info layout shared with the host layer (see b200sp_kernels.h)
enum { kInfoKind = 0, kInfoMedium = 1, kInfoLong = 2, kInfoGroup = 3, kInfoXBlocks = 4, kInfoBlockElems = 5, kInfoLongLen = 6,
       kInfoSegments = 7 };
enum { kPlanTiles = 0, kPlanBinned = 1, kPlanBinnedBlocked = 2 };  // blocked: long rows go to SpmvLongBlockKernel

template <typename CompT, typename ValT, typename OutT, bool kVec>
int LaunchLongBlock(const LongBlockArgs<CompT, ValT, OutT> &la, int blocks, cudaStream_t stream)
{
    constexpr int kSmem = kXBlockElems * (int)sizeof(ValT);
    static bool configured[b200sp::kMaxDevices] = {};  // per device: this instantiation may use kSmem bytes
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= b200sp::kMaxDevices) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(SpmvLongBlockKernel<CompT, ValT, OutT, kVec>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    SpmvLongBlockKernel<CompT, ValT, OutT, kVec><<<(unsigned)blocks, kLongBlockThreads, kSmem, stream>>>(la);
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

template <typename CompT, typename ValT, typename OutT>
int LaunchBinned(const int32_t *rowPtr, const int32_t *colInd, const ValT *val, const ValT *x, OutT *y, int64_t rows,
                 int64_t cols, int64_t nnz, const Scalars<CompT> &sc, void *plan, const int32_t *info,
                 cudaStream_t stream)
{
    const BinLayout L = BinLayoutFor(rows, cols, nnz);
    char *p = static_cast<char *>(plan);
    const int4 *listM = reinterpret_cast<const int4 *>(p + L.offListM);
    const int4 *listL = reinterpret_cast<const int4 *>(p + L.offListL);
    const int nM = info[kInfoMedium], nL = info[kInfoLong], G = info[kInfoGroup], nS = info[kInfoSegments];
    LongSegs ls;
    ls.segs = reinterpret_cast<const int4 *>(p + L.offSegs);
    ls.list = listL;
    ls.rowSeg = reinterpret_cast<const int2 *>(p + L.offRowSeg);
    ls.counters = reinterpret_cast<int32_t *>(p + L.offSegCounters);
    ls.partials = p + L.offSegPartials;
    const bool vec = (reinterpret_cast<uintptr_t>(colInd) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(val) % (4 * sizeof(ValT)) == 0);
#if B200SP_SPMV_FUSE_LIST
    // Only for small products (up to 4 M entries): there the fork / join costs more than it buys.  Larger ones
    // keep two kernels on forked streams -- equal in isolation (36.9 us either way on 7.6 M entries), but four
    // such products pipelined on three streams with their host copies took 329 us fused against 287 us forked.
    if (nL > 0 && nnz <= (4ll << 20) && !(info[kInfoKind] == kPlanBinnedBlocked && L.xBlocks > 0)) {
        const unsigned blocks = (unsigned)nS + (unsigned)((nM + 7) / 8) + (unsigned)((rows * G + 255) / 256);
        auto launch = [&]<int GG>() {
            if (vec) SpmvAllBinsKernel<CompT, ValT, OutT, GG, true><<<blocks, 256, 0, stream>>>(
                rowPtr, colInd, val, x, y, listM, ls, nM, nS, (int)rows, sc);
            else SpmvAllBinsKernel<CompT, ValT, OutT, GG, false><<<blocks, 256, 0, stream>>>(
                rowPtr, colInd, val, x, y, listM, ls, nM, nS, (int)rows, sc);
        };
        switch (G) {
            case 2: launch.template operator()<2>(); break;
            case 8: launch.template operator()<8>(); break;
            default: launch.template operator()<4>(); break;
        }
        b200sp_note_launches(1);
        return (int)cudaGetLastError();
    }
#endif
    // The kernels write disjoint rows of y.  The long rows go first, to a side stream forked from
    // and joined back into the caller's stream; medium and short rows follow in one grid.
    b200sp::SideLanes *lanes = nL > 0 ? b200sp::GetSideLanes() : nullptr;
    cudaStream_t sL = stream;
    if (lanes != nullptr) {
        cudaError_t e = cudaEventRecord(lanes->fork, stream);
        if (e != cudaSuccess) return (int)e;
        sL = lanes->stream[0];
    }
    if (nL > 0) {
        if (lanes != nullptr && cudaStreamWaitEvent(sL, lanes->fork, 0) != cudaSuccess) return (int)cudaGetLastError();
        if (info[kInfoKind] == kPlanBinnedBlocked && L.xBlocks > 0) {
            LongBlockArgs<CompT, ValT, OutT> la;
            la.colInd = colInd;
            la.val = val;
            la.x = x;
            la.y = y;
            la.cols = (int)cols;
            la.sc = sc;
            la.list = listL;
            la.segStart = reinterpret_cast<const int32_t *>(p + L.offSegStart);
            la.counters = reinterpret_cast<int32_t *>(p + L.offLongCounters);
            la.partials = reinterpret_cast<CompT *>(p + L.offPartials);
            la.nLong = nL;
            la.xBlocks = L.xBlocks;
            // one CTA per SM at most (it holds half of the SM's threads and a block of x)
            constexpr int kPiecesPerCta = kLongBlockThreads / B200SP_SPMV_PIECE_LANES;
            int groups = b200sp_sm_count() / L.xBlocks;
            const int useful = (nL + kPiecesPerCta - 1) / kPiecesPerCta;
            if (groups > useful) groups = useful;
            if (groups > kMaxLongGroups) groups = kMaxLongGroups;
            if (groups < 1) groups = 1;
            la.groups = groups;
            const int rcL = vec ? LaunchLongBlock<CompT, ValT, OutT, true>(la, L.xBlocks * groups, sL)
                                : LaunchLongBlock<CompT, ValT, OutT, false>(la, L.xBlocks * groups, sL);
            if (rcL != 0) return rcL;
        } else {
            if (vec) SpmvLongListKernel<CompT, ValT, OutT, true><<<(unsigned)nS, 256, 0, sL>>>(colInd, val, x, y, ls, sc);
            else SpmvLongListKernel<CompT, ValT, OutT, false><<<(unsigned)nS, 256, 0, sL>>>(colInd, val, x, y, ls, sc);
            b200sp_note_launches(1);
        }
        if (lanes != nullptr) cudaEventRecord(lanes->join[0], sL);
    }
    if (rows > 0) {
        // CTAs of kMsThreads threads: a CTA's slot is recycled when its slowest warp is done, and rows of one
        // CTA differ in length (128 threads: 90.4 us on the power-law matrix, 256: 91.3, 64: 91.8).
        constexpr int kMsThreads = 128;
        constexpr int kWpc = kMsThreads / 32;
        const unsigned shortBlocks = (unsigned)((rows * G + kMsThreads - 1) / kMsThreads);
        if (nM > 0) {
            const unsigned blocks = (unsigned)((nM + kWpc - 1) / kWpc) + shortBlocks;
            switch (G) {
                case 2: SpmvMediumShortKernel<CompT, ValT, OutT, 2><<<blocks, kMsThreads, 0, stream>>>(rowPtr, colInd, val, x, y, listM, nM, (int)rows, sc); break;
                case 8: SpmvMediumShortKernel<CompT, ValT, OutT, 8><<<blocks, kMsThreads, 0, stream>>>(rowPtr, colInd, val, x, y, listM, nM, (int)rows, sc); break;
                default: SpmvMediumShortKernel<CompT, ValT, OutT, 4><<<blocks, kMsThreads, 0, stream>>>(rowPtr, colInd, val, x, y, listM, nM, (int)rows, sc); break;
            }
        } else {
            switch (G) {
                case 2: SpmvShortRowsKernel<CompT, ValT, OutT, 2><<<shortBlocks, kMsThreads, 0, stream>>>(rowPtr, colInd, val, x, y, (int)rows, sc); break;
                case 8: SpmvShortRowsKernel<CompT, ValT, OutT, 8><<<shortBlocks, kMsThreads, 0, stream>>>(rowPtr, colInd, val, x, y, (int)rows, sc); break;
                default: SpmvShortRowsKernel<CompT, ValT, OutT, 4><<<shortBlocks, kMsThreads, 0, stream>>>(rowPtr, colInd, val, x, y, (int)rows, sc); break;
            }
        }
        b200sp_note_launches(1);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (lanes != nullptr) e = cudaStreamWaitEvent(stream, lanes->join[0], 0);
    return (int)e;
}

template <typename CompT, typename ValT, typename OutT>
int LaunchTyped(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, void *y, int64_t rows,
                int64_t cols, int64_t nnz, const b200spScalars *s, void *plan, const int32_t *info,
                cudaStream_t stream)
{
    const Scalars<CompT> sc = MakeScalars<CompT>(s);
    if (plan != nullptr && info != nullptr && info[kInfoKind] != kPlanTiles)
        return LaunchBinned<CompT, ValT, OutT>(rowPtr, colInd, static_cast<const ValT *>(val),
                                               static_cast<const ValT *>(x), static_cast<OutT *>(y), rows, cols, nnz,
                                               sc, plan, info, stream);
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
        b200sp_note_launches(1);
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
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

template <typename CompT, typename ValT, typename OutT>
int LaunchTransTyped(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, void *y,
                     int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *s, void *scratch,
                     size_t scratchBytes, bool byNnz, cudaStream_t stream)
{
    const Scalars<CompT> sc = MakeScalars<CompT>(s);
    if (cols == 0) return 0;
    const int sms = b200sp_sm_count();
    const unsigned eltBlocks = (unsigned)((cols + 255) / 256 < (int64_t)sms * 16 ? (cols + 255) / 256 : sms * 16);
    const int G = GroupWidthFor(rows, nnz);
    const int64_t want = rows > 0 ? (rows * G + 255) / 256 : 1;
    const unsigned rowBlocks = (unsigned)(want < (int64_t)sms * 32 ? want : sms * 32);
    const int64_t wantNnz = (nnz + 8 * kTransChunk - 1) / (8 * kTransChunk);  // eight warps, one chunk each
    const unsigned nnzBlocks = (unsigned)(wantNnz < (int64_t)sms * 32 ? (wantNnz > 0 ? wantNnz : 1) : sms * 32);
    constexpr bool kNarrowOut = sizeof(OutT) == 2;
    if constexpr (kNarrowOut) {
        if (scratch == nullptr || scratchBytes < sizeof(float) * (size_t)cols) return (int)cudaErrorInvalidValue;
        float *acc = static_cast<float *>(scratch);
        SpmvTransScaleKernel<CompT, OutT, float><<<eltBlocks, 256, 0, stream>>>(static_cast<const OutT *>(y), acc,
                                                                                 (int)cols, sc);
        b200sp_note_launches(1);
        if (rows > 0) {
            if (byNnz && nnz > 0)
                SpmvTransScatterNnzKernel<CompT, ValT, float><<<nnzBlocks, 256, 0, stream>>>(
                    rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), acc, (int)rows,
                    (int)nnz, sc);
            else
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
            if (byNnz && nnz > 0)
                SpmvTransScatterNnzKernel<CompT, ValT, OutT><<<nnzBlocks, 256, 0, stream>>>(
                    rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(x), acc, (int)rows,
                    (int)nnz, sc);
            else
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
    // one cached value per device ordinal: the GPUs of a process need not be alike
    static std::atomic<int> cached[b200sp::kMaxDevices] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    const bool slot = dev >= 0 && dev < b200sp::kMaxDevices;
    if (slot) {
        n = cached[dev].load(std::memory_order_relaxed);
        if (n > 0) return n;
    }
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    if (slot) cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

size_t b200sp_spmv_tile_plan_bytes(int64_t rows, int64_t nnz) { return LayoutFor(rows, nnz).total; }

size_t b200sp_spmv_plan_bytes(int64_t rows, int64_t cols, int64_t nnz)
{
    const size_t tiles = LayoutFor(rows, nnz).total;
    const size_t bins = BinLayoutFor(rows, cols, nnz).total;
    return tiles > bins ? tiles : bins;  // one buffer serves either plan
}

int b200sp_spmv_analyze(const int32_t *row_ptr, const int32_t *col_ind, int64_t rows, int64_t cols, int64_t nnz,
                        void *plan, size_t plan_bytes, int32_t *plan_info, void *stream)
{
    const size_t need = plan_info == nullptr ? LayoutFor(rows, nnz).total : BinLayoutFor(rows, cols, nnz).total;
    if (plan == nullptr || plan_bytes < need) return (int)cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *p = static_cast<char *>(plan);
    if (plan_info == nullptr) {
        // Tile plan: nothing to read back, so nothing synchronises.
        const PlanLayout L = LayoutFor(rows, nnz);
        if (L.ntiles == 0) return 0;
        const unsigned blocks = (unsigned)((L.ntiles + 1 + 255) / 256);
        SpmvTileSearchKernel<<<blocks, 256, 0, st>>>(row_ptr, (int)rows, (int)nnz, (int)L.ntiles,
                                                     reinterpret_cast<int32_t *>(p + L.offTileRow),
                                                     reinterpret_cast<int32_t *>(p + L.offCounters));
        b200sp_note_launches(1);
        return (int)cudaGetLastError();
    }
    // Binned plan: list the medium and the long rows, then read the counts back (one sync).
    const BinLayout L = BinLayoutFor(rows, cols, nnz);
    auto *hdr = reinterpret_cast<BinHeader *>(p + L.offHeader);
    cudaError_t e = cudaMemsetAsync(hdr, 0, 256, st);
    if (e != cudaSuccess) return (int)e;
    const bool blocked = L.xBlocks > 0 && col_ind != nullptr;
    if (blocked) {
        e = cudaMemsetAsync(p + L.offLongCounters, 0, sizeof(int32_t) * kMaxLongGroups, st);
        if (e != cudaSuccess) return (int)e;
    }
    if (rows > 0) {
        const long long want = (rows + 255) / 256;
        const long long cap = (long long)b200sp_sm_count() * 16;
        SpmvBinRowsKernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
            row_ptr, (int)rows, hdr, reinterpret_cast<int4 *>(p + L.offListM),
            reinterpret_cast<int4 *>(p + L.offTmpL));
        SpmvSortByLengthKernel<<<1, 1024, 0, st>>>(&hdr->longs, reinterpret_cast<const int4 *>(p + L.offTmpL),
                                                   reinterpret_cast<int4 *>(p + L.offListL));
        SpmvCutSegmentsKernel<<<1, 1024, 0, st>>>(hdr, reinterpret_cast<const int4 *>(p + L.offListL),
                                                  reinterpret_cast<int4 *>(p + L.offSegs),
                                                  reinterpret_cast<int2 *>(p + L.offRowSeg),
                                                  reinterpret_cast<int32_t *>(p + L.offSegCounters));
        b200sp_note_launches(3);
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    if (blocked && rows > 0) {
        // Cut every long row at the x block boundaries (the count of long rows is still on the device).
        SpmvLongSegmentsKernel<<<(unsigned)(b200sp_sm_count() * 4), 256, 0, st>>>(
            col_ind, hdr, reinterpret_cast<const int4 *>(p + L.offListL),
            reinterpret_cast<int32_t *>(p + L.offSegStart), L.xBlocks);
        b200sp_note_launches(1);
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    BinHeader host{};
    e = cudaMemcpyAsync(&host, hdr, sizeof(host), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    const double avgShort = host.shortRows > 0 ? (double)host.shortNnz / host.shortRows : 0.0;
    // Staging x costs every one of the xBlocks x groups CTAs the same whatever the number of long rows:
    // on shards of the power-law matrix the blocked kernel won with 2155 long rows (51 vs 70 us) and 4299
    // (95 vs 133 us), lost with 1070 (44 vs 37 us), tied with 517 -- 32 column blocks each time.
    const int minLong = B200SP_SPMV_MIN_LONG_BLOCKED > 48 * L.xBlocks ? B200SP_SPMV_MIN_LONG_BLOCKED : 48 * L.xBlocks;
    const bool useBlocked = blocked && host.unsorted == 0 && host.longs >= minLong;
    plan_info[kInfoKind] = useBlocked ? kPlanBinnedBlocked : kPlanBinned;
    plan_info[kInfoXBlocks] = useBlocked ? L.xBlocks : 0;
    plan_info[kInfoBlockElems] = useBlocked ? kXBlockElems : 0;
    plan_info[kInfoLongLen] = kLongLen;
    plan_info[kInfoSegments] = host.segments;
    plan_info[kInfoMedium] = host.medium;
    plan_info[kInfoLong] = host.longs;
#ifdef B200SP_SPMV_FORCE_SHORT_G
    plan_info[kInfoGroup] = B200SP_SPMV_FORCE_SHORT_G;
#else
    // measured: 27-entry stencil rows run 92 us with 2 or 4 lanes per row, 107 us with 8, 141 us with 16;
    // power-law rows (3.3 entries on average) 96 us with 2 lanes, 115 us with 4
    plan_info[kInfoGroup] = avgShort < 6.0 ? 2 : 4;
#endif
    return 0;
}

int b200sp_spmv_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x, void *y,
                       int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars, int comp_type,
                       int val_type, int out_type, void *plan, const int32_t *plan_info, void *stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rc = DispatchTypes(comp_type, val_type, out_type, [&]<typename C, typename V, typename O>() {
        return LaunchTyped<C, V, O>(row_ptr, col_ind, val, x, y, rows, cols, nnz, scalars, plan, plan_info, st);
    });
    return rc < 0 ? (int)cudaErrorInvalidValue : rc;
}

int b200sp_spmv_max_row_length(const int32_t *row_ptr, int64_t rows, void *scratch4, int32_t *max_len, void *stream)
{
    if (max_len == nullptr || scratch4 == nullptr) return (int)cudaErrorInvalidValue;
    *max_len = 0;
    if (rows <= 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(scratch4, 0, sizeof(int32_t), st);
    if (e != cudaSuccess) return (int)e;
    const long long want = (rows + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 16;
    SpmvMaxRowLengthKernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(row_ptr, (int)rows,
                                                                             static_cast<int32_t *>(scratch4));
    b200sp_note_launches(1);
    e = cudaMemcpyAsync(max_len, scratch4, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaStreamSynchronize(st);
}

int b200sp_spmv_trans_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x,
                             void *y, int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars,
                             int comp_type, int val_type, int out_type, void *scratch, size_t scratch_bytes,
                             int by_nnz, void *stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rc = DispatchTypes(comp_type, val_type, out_type, [&]<typename C, typename V, typename O>() {
        return LaunchTransTyped<C, V, O>(row_ptr, col_ind, val, x, y, rows, cols, nnz, scalars, scratch,
                                         scratch_bytes, by_nnz != 0, st);
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
// Device address of gNoAllocScratch, per device ordinal.  Host threads may race to fill a slot; they all
// store the same address, and the atomic keeps that race defined.
std::atomic<void *> gNoAllocAddr[kMaxDevices] = {};

// In host code `gNoAllocScratch` is only a handle for the runtime, not an address a kernel can
// use; the device address has to be asked for, once per device, with that device current.
int NoAllocScratchAddress(void **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    void *p = gNoAllocAddr[dev].load(std::memory_order_relaxed);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, gNoAllocScratch);
        if (e != cudaSuccess) return (int)e;
        gNoAllocAddr[dev].store(p, std::memory_order_relaxed);
    }
    *out = p;
    return 0;
}

}  // namespace

extern "C" int b200sp_spmv_f32_noalloc(const int32_t *row_ptr, const int32_t *col_ind, const float *val,
                                       const float *x, float *y, int64_t rows, int64_t cols, int64_t nnz,
                                       float alpha, float beta, void *stream)
{
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
    const int an = b200sp_spmv_analyze(row_ptr, nullptr, rows, cols, nnz, scratch, kNoAllocBytes, nullptr, stream);
    if (an != 0) return an;
    b200spScalars sc{};
    sc.alpha_f = alpha;
    sc.beta_f = beta;
    return LaunchTyped<float, float, float>(row_ptr, col_ind, val, x, y, rows, cols, nnz, &sc, scratch, nullptr,
                                            static_cast<cudaStream_t>(stream));
}
