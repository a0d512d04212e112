// CSR SpMM kernels for sm_100a and their extern "C" launchers.
//
// The reference computes one (row, 8-column chunk) per SIMT thread and re-reads the row's
// col_ind / values once per chunk (sparse/spmm/arch35/spmm_kernel.cpp:88-268).  Here a group
// of lanes owns a row: the lanes sit side by side on a row of B, 16 bytes each (so every B
// row is fetched with 128-bit coalesced loads), the row's col_ind / values are read once,
// one per lane, and handed round the group by shuffle.  A group is as wide as a B row needs
// (N * sizeof / 16 lanes, a power of two up to 32), so one warp carries 1 to 32 rows of A.
// Each output keeps one fp32 accumulator that takes its products in CSR order with separate
// multiply and add, exactly as the golden does: for rows of up to 1024 entries the result is
// bit-identical to the golden.
//
// Row-length routing (the analysis pass fills the workspace):
//     rows <= 1024 non-zeros            -> one lane group per row;
//     longer rows                       -> cut into segments of 4096 non-zeros, one CTA
//                                          (4 warps) per segment.  A row of several
//                                          segments is completed by whichever segment CTA
//                                          finishes last: it adds the stored partial rows in
//                                          segment order, so no CTA ever waits and the sum
//                                          order is fixed.
// Layouts other than "B rows contiguous, C row-major, 16-byte aligned", and the int8 path,
// go through a generic one-thread-per-output kernel that uses the reference's index
// formulas verbatim in meaning (spmm_kernel.cpp:156-168, 215-219).
//
// Numerics follow the golden SpmmCpuFp32 / SpmmCpuInt8 (test/spmm/arch35/spmm_test.cpp:
// 125-200): inputs widened to fp32 (int32), products accumulated in fp32 (int32),
// C = alpha*acc + beta*C with C not read when beta == 0; fp16 output is clamped to
// +-65504 before rounding; int32 output is computed in int64 and saturated.
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "../common/side_stream.h"

namespace {

#ifndef B200SP_SPMM_THREADS
#define B200SP_SPMM_THREADS 128
#endif
constexpr int kThreads = B200SP_SPMM_THREADS;  // warps of a CTA: one lane-group set each, or one long-row segment
constexpr int kWarps = kThreads / 32;
constexpr int kLongRow = 1024;          // rows longer than this are handled by segment CTAs
constexpr int kSegNnz = 4096;           // non-zeros per segment
constexpr int kWarpSegNnz = kSegNnz / kWarps;
constexpr int kMaxTileCols = 256;       // widest column tile one warp pass covers (32 lanes x 8)

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct SegEntry {
    int32_t row;
    int32_t seg;      // index of this segment inside its row
    int32_t longIdx;  // index into the long-row table
    int32_t pad;
};
struct LongRow {
    int32_t row;
    int32_t segBase;   // first entry of this row in the segment table
    int32_t nseg;
    int32_t partBase;  // first partial-row slot (rows of two or more segments only)
};

// Column blocking of the long rows (see SpmmLongBlockKernel): B is cut into at most kMaxBlocks blocks of
// consecutive rows, each small enough to stay in L2 while every long row of A sums its entries that fall into it.
constexpr int kMaxBlocks = 64;
#ifndef B200SP_SPMM_BLOCK_MB
#define B200SP_SPMM_BLOCK_MB 32
#endif
constexpr long long kBlockBytes = (long long)B200SP_SPMM_BLOCK_MB << 20;  // target size of one block of B rows
constexpr long long kBlockMinB = 96ll << 20;      // a B smaller than this is left to L2 as a whole
constexpr int kBlockMinRowBytes = 512;            // B rows narrower than a warp of 16-byte pieces keep the segment CTAs
#ifndef B200SP_SPMM_UNIT_NNZ
#define B200SP_SPMM_UNIT_NNZ 256
#endif
constexpr int kUnitNnz = B200SP_SPMM_UNIT_NNZ;   // a (row, block) piece longer than this is cut into several units

struct PlanLayout {
    int64_t capLong, capSegs, capBlockSlots;
    size_t offCounts, offLong, offSegs, offCounters, offPartials;
    size_t offCuts, offRowSlots, offBlockCounters, offBlockMeta, offUnits, offBlockPartials, total;
};

inline PlanLayout LayoutFor(int64_t rows, int64_t nnz, int64_t n)
{
    (void)rows;
    PlanLayout L;
    L.capLong = nnz / (kLongRow + 1) + 1;
    L.capSegs = nnz / kSegNnz + L.capLong + 1;
    L.offCounts = 0;
    L.offLong = 256;
    L.offSegs = AlignUp(L.offLong + sizeof(LongRow) * (size_t)L.capLong, 256);
    L.offCounters = AlignUp(L.offSegs + sizeof(SegEntry) * (size_t)L.capSegs, 256);
    L.offPartials = AlignUp(L.offCounters + sizeof(int32_t) * (size_t)L.capLong, 256);
    // Only rows of two or more segments store partial rows; those have > kSegNnz entries.
    const int64_t capPartialSegs = 2 * (nnz / kSegNnz) + 1;
    L.offCuts = AlignUp(L.offPartials + sizeof(float) * (size_t)capPartialSegs * (size_t)n, 256);
    // Column blocks: a cut table and a {first slot, slots} pair per long row, the unit table and one partial row
    // per unit, up to a budget of one unit per 128 non-zeros (rows of C at least 128 wide only: narrower ones
    // never take that path).
    L.capBlockSlots = n >= 128 ? nnz / 128 + kMaxBlocks : 0;
    const bool on = L.capBlockSlots > 0;
    L.offRowSlots = AlignUp(L.offCuts + (on ? sizeof(int32_t) * (size_t)L.capLong * (kMaxBlocks + 1) : 0), 256);
    L.offBlockCounters = AlignUp(L.offRowSlots + (on ? sizeof(int2) * (size_t)L.capLong : 0), 256);
    L.offBlockMeta = AlignUp(L.offBlockCounters + (on ? sizeof(int32_t) * (size_t)L.capLong : 0), 256);
    L.offUnits = AlignUp(L.offBlockMeta + (on ? sizeof(int32_t) * 3 * kMaxBlocks : 0), 256);
    L.offBlockPartials = AlignUp(L.offUnits + (on ? sizeof(int4) * (size_t)L.capBlockSlots : 0), 256);
    L.total = AlignUp(L.offBlockPartials + sizeof(float) * (size_t)L.capBlockSlots * (size_t)n, 256);
    return L;
}

// ---------------------------------------------------------------- element helpers

template <typename T> __device__ __forceinline__ float ToF32(T v);
template <> __device__ __forceinline__ float ToF32<float>(float v) { return v; }
template <> __device__ __forceinline__ float ToF32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ToF32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T FromF32(float v);
template <> __device__ __forceinline__ float FromF32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half FromF32<__half>(float v)
{
    // Saturate instead of producing inf (reference spmm_kernel.cpp:232-236).
    v = fminf(fmaxf(v, -65504.0f), 65504.0f);
    return __float2half_rn(v);
}
template <> __device__ __forceinline__ __nv_bfloat16 FromF32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct ScalarsF {
    float alpha, beta;
    const float *alphaDev, *betaDev;
    __device__ __forceinline__ float Alpha() const { return alphaDev ? *alphaDev : alpha; }
    __device__ __forceinline__ float Beta() const { return betaDev ? *betaDev : beta; }
};
struct ScalarsI {
    int32_t alpha, beta;
    const int32_t *alphaDev, *betaDev;
    __device__ __forceinline__ int32_t Alpha() const { return alphaDev ? *alphaDev : alpha; }
    __device__ __forceinline__ int32_t Beta() const { return betaDev ? *betaDev : beta; }
};

// How the rows of B are fetched.  B is the operand every row of A gathers from: when it fits in L2 (67 MB at
// 262,144 x 64 fp32) it should stay there while col_ind / values / C stream past it, so its loads carry an
// L2 evict-last policy (per instruction; nothing outlives the launch) and the streams are evict-first.
//   0: plain read-only loads   1: read-only loads with L2::evict_last   2: the same without allocating in L1
#ifndef B200SP_SPMM_B_POLICY
#define B200SP_SPMM_B_POLICY 1
#endif
__device__ __forceinline__ uint4 LoadB16(const void *p)
{
#if B200SP_SPMM_B_POLICY == 0
    return __ldg(reinterpret_cast<const uint4 *>(p));
#else
    uint64_t pol;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));  // hoisted out of loops by the compiler
    uint4 q;
#if B200SP_SPMM_B_POLICY == 1
    asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                 : "l"(p), "l"(pol));
#else
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                 : "l"(p), "l"(pol));
#endif
    return q;
#endif
}

// 16 bytes of a B row as fp32 values: 4 floats, or 8 half / bf16.
template <typename T> struct Pack;
template <> struct Pack<float> {
    static constexpr int kElems = 4;
    static __device__ __forceinline__ void Load(const float *p, float (&out)[4])
    {
        const uint4 q = LoadB16(p);
        out[0] = __uint_as_float(q.x); out[1] = __uint_as_float(q.y);
        out[2] = __uint_as_float(q.z); out[3] = __uint_as_float(q.w);
    }
};
template <> struct Pack<__half> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void Load(const __half *p, float (&out)[8])
    {
        const uint4 q = LoadB16(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
};
template <> struct Pack<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void Load(const __nv_bfloat16 *p, float (&out)[8])
    {
        const uint4 q = LoadB16(p);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// ---------------------------------------------------------------- analysis

__global__ void SpmmFindLongRowsKernel(const int32_t *__restrict__ rowPtr, int rows, int32_t *counts,
                                       LongRow *longRows, SegEntry *segs, int32_t *counters)
{
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
         r += (long long)gridDim.x * blockDim.x) {
        const int len = rowPtr[r + 1] - rowPtr[r];
        if (len <= kLongRow) continue;
        const int nseg = (len + kSegNnz - 1) / kSegNnz;
        const int li = atomicAdd(&counts[0], 1);
        const int sb = atomicAdd(&counts[1], nseg);
        const int pb = nseg > 1 ? atomicAdd(&counts[2], nseg) : 0;
        longRows[li] = {(int32_t)r, sb, nseg, pb};
        counters[li] = 0;
        for (int s = 0; s < nseg; ++s) segs[sb + s] = {(int32_t)r, s, li, 0};
    }
}

// A warp per long row: checks that its columns ascend, finds where it crosses the boundaries of the column
// blocks (cut[b] = first entry whose column is >= b * blockCols; cut[blocks] = the row's end) and counts the
// units (pieces of at most kUnitNnz entries inside one block) of the row and of every block.
__global__ void __launch_bounds__(256) SpmmCutBlocksKernel(const int32_t *__restrict__ rowPtr,
                                                           const int32_t *__restrict__ colInd,
                                                           const LongRow *__restrict__ longRows, int nLong,
                                                           long long blockCols, int blocks, int32_t *__restrict__ cuts,
                                                           int2 *__restrict__ rowSlots, int32_t *__restrict__ counters,
                                                           int32_t *__restrict__ blockUnits, int32_t *unsorted)
{
    const int lane = threadIdx.x & 31;
    const int li = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (li >= nLong) return;
    const int row = longRows[li].row;
    const int s = rowPtr[row], e = rowPtr[row + 1];
    bool bad = false;
    for (int p = s + lane; p + 1 < e; p += 32) bad |= colInd[p] > colInd[p + 1];
    if (__any_sync(0xffffffffu, bad)) {
        if (lane == 0) atomicExch(unsorted, 1);
    }
    int32_t *cut = cuts + (long long)li * (kMaxBlocks + 1);
    for (int b = lane; b <= blocks; b += 32) {
        int lo = s, hi = e;
        if (b == blocks) lo = e;
        const long long target = (long long)b * blockCols;
        while (lo < hi) {
            const int mid = lo + ((hi - lo) >> 1);
            if ((long long)colInd[mid] < target) lo = mid + 1;
            else hi = mid;
        }
        cut[b] = lo;
    }
    __syncwarp();
    int units = 0;
    for (int b = lane; b < blocks; b += 32) {
        const int len = cut[b + 1] - cut[b];
        const int u = len > 0 ? (len + kUnitNnz - 1) / kUnitNnz : 0;  // garbage-in (unsorted) can make len negative
        if (u > 0) atomicAdd(blockUnits + b, u);
        units += u;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) units += __shfl_xor_sync(0xffffffffu, units, off);
    if (lane == 0) {
        rowSlots[li] = make_int2(0, units);
        counters[li] = 0;
    }
}

// One CTA: first slot of every long row (exclusive scan of the rows' unit counts, in list order) and first unit
// of every block; the total goes to *total.
__global__ void __launch_bounds__(1024) SpmmBlockScanKernel(int2 *__restrict__ rowSlots, int nLong,
                                                            int32_t *__restrict__ blockMeta, int blocks, int32_t *total)
{
    __shared__ int sWarp[32];
    __shared__ int sCarry;
    if (threadIdx.x == 0) sCarry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < nLong; base += 1024) {
        const int i = base + threadIdx.x;
        const int n = i < nLong ? rowSlots[i].y : 0;
        int incl = n;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += t;
        }
        if (lane == 31) sWarp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = sWarp[lane];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, off);
                if (lane >= off) w += t;
            }
            sWarp[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int before = sCarry + (warp > 0 ? sWarp[warp - 1] : 0) + incl - n;
        if (i < nLong) rowSlots[i].x = before;
        __syncthreads();
        if (threadIdx.x == 1023) sCarry = before + n;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int run = 0;
        for (int b = 0; b < blocks; ++b) {  // blockMeta: [0..64) units of the block, [64..128) first unit, [128..192) filled
            blockMeta[kMaxBlocks + b] = run;
            blockMeta[2 * kMaxBlocks + b] = 0;
            run += blockMeta[b];
        }
        *total = sCarry;
    }
}

struct BlockUnit {
    int32_t start, end;  // entries of the row inside one column block
    int32_t longIdx;
    int32_t slot;        // partial row this unit writes
};

// A warp per long row: writes the row's units into the table, block by block (the table is ordered by block; the
// order inside a block is whatever the atomics give, the slot of a unit is fixed by its place in the row).
__global__ void __launch_bounds__(256) SpmmFillUnitsKernel(const int32_t *__restrict__ cuts, const int2 *__restrict__ rowSlots,
                                                           int nLong, int blocks, int32_t *__restrict__ blockMeta,
                                                           BlockUnit *__restrict__ units, int capUnits)
{
    const int lane = threadIdx.x & 31;
    const int li = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (li >= nLong) return;
    const int32_t *cut = cuts + (long long)li * (kMaxBlocks + 1);
    int slot = rowSlots[li].x;
    for (int b = 0; b < blocks; ++b) {
        const int s = cut[b], e = cut[b + 1];
        const int n = e > s ? (e - s + kUnitNnz - 1) / kUnitNnz : 0;
        if (n == 0) continue;
        int pos = 0;
        if (lane == 0) pos = blockMeta[kMaxBlocks + b] + atomicAdd(blockMeta + 2 * kMaxBlocks + b, n);
        pos = __shfl_sync(0xffffffffu, pos, 0);
        for (int i = lane; i < n; i += 32) {
            const int us = s + i * kUnitNnz;
            if (pos + i < capUnits)
                units[pos + i] = {us, us + kUnitNnz < e ? us + kUnitNnz : e, li, slot + i};
        }
        slot += n;
    }
}

// ---------------------------------------------------------------- fast path

template <typename ValT, typename OutT>
struct FastArgs {
    const int32_t *rowPtr;
    const int32_t *colInd;
    const ValT *val;
    const ValT *B;
    OutT *C;
    int m;
    int n;
    long long ldb;
    long long ldc;
    ScalarsF sc;
    int nsegs;
    const LongRow *longRows;
    const SegEntry *segs;
    int32_t *counters;
    float *partials;      // [partial slot][n]
};

// One accumulation step, in the golden's arithmetic: the product is rounded, then added
// (no fused multiply-add), so a row summed in CSR order reproduces the golden bit for bit.
template <bool kKahan>
__device__ __forceinline__ void Accumulate(float v, float b, float &acc, float &comp)
{
    const float prod = __fmul_rn(v, b);
    if (kKahan) {  // compensated summation, the reference's high-precision algorithm
        const float y = __fsub_rn(prod, comp);
        const float t = __fadd_rn(acc, y);
        comp = __fsub_rn(__fsub_rn(t, acc), y);
        acc = t;
    } else {
        acc = __fadd_rn(acc, prod);
    }
}

// Adds sum_{p in [s, e)} val[p] * B[col[p], slice] to acc, p ascending.  The kLanes lanes of a
// group call it together with the same s, e (groups of one warp may differ); `trips` is the
// warp-uniform number of kLanes-wide chunks to walk (>= this group's own need).
#ifndef B200SP_SPMM_BATCH
#define B200SP_SPMM_BATCH 4
#endif

template <typename ValT, bool kKahan, int kLanes>
__device__ __forceinline__ void RowDot(const int32_t *__restrict__ colInd, const ValT *__restrict__ val,
                                       const ValT *__restrict__ Bslice, long long ldb, int s, int e, int trips,
                                       bool colLive, bool allColsLive, float (&acc)[Pack<ValT>::kElems],
                                       float (&comp)[Pack<ValT>::kElems])
{
    constexpr int E = Pack<ValT>::kElems;
    constexpr int kBatch = kLanes < B200SP_SPMM_BATCH ? kLanes : B200SP_SPMM_BATCH;  // B rows in flight per lane
    const int li = threadIdx.x & (kLanes - 1);
    for (int chunk = 0; chunk < trips; ++chunk) {
        const int p0 = s + chunk * kLanes;
        const int rem = e - p0;  // entries of this group's row left; <= 0 once the row is done
        int myCol = 0;
        float myVal = 0.0f;
        if (li < rem) {
            myCol = __ldcs(colInd + p0 + li);
            myVal = ToF32(__ldcs(val + p0 + li));
        }
        // Whole warp on full chunks and live columns: straight-line code without predicates.
        if (allColsLive && __all_sync(0xffffffffu, rem >= kLanes)) {
#pragma unroll
            for (int q0 = 0; q0 < kLanes; q0 += kBatch) {
                float b[kBatch][E];
                float v[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int c = __shfl_sync(0xffffffffu, myCol, q0 + u, kLanes);
                    v[u] = __shfl_sync(0xffffffffu, myVal, q0 + u, kLanes);
                    Pack<ValT>::Load(Bslice + (long long)c * ldb, b[u]);
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
#pragma unroll
                    for (int i = 0; i < E; ++i) Accumulate<kKahan>(v[u], b[u][i], acc[i], comp[i]);
                }
            }
            continue;
        }
#pragma unroll
        for (int q0 = 0; q0 < kLanes; q0 += kBatch) {
            float b[kBatch][E];
            float v[kBatch];
            bool live[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int c = __shfl_sync(0xffffffffu, myCol, q0 + u, kLanes);
                v[u] = __shfl_sync(0xffffffffu, myVal, q0 + u, kLanes);
                live[u] = colLive && (q0 + u < rem);
                if (live[u]) {
                    Pack<ValT>::Load(Bslice + (long long)c * ldb, b[u]);
                } else {
#pragma unroll
                    for (int i = 0; i < E; ++i) b[u][i] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                if (live[u]) {
#pragma unroll
                    for (int i = 0; i < E; ++i) Accumulate<kKahan>(v[u], b[u][i], acc[i], comp[i]);
                }
            }
        }
    }
}

#ifndef B200SP_SPMM_C_STREAMED
#define B200SP_SPMM_C_STREAMED 1
#endif
#if B200SP_SPMM_C_STREAMED
#define B200SP_SPMM_C_LOAD(p) __ldcs(p)
#define B200SP_SPMM_C_STORE(p, v) __stcs(p, v)
#else
#define B200SP_SPMM_C_LOAD(p) (*(p))
#define B200SP_SPMM_C_STORE(p, v) (*(p) = (v))
#endif
template <typename OutT, int E>
__device__ __forceinline__ void StoreRowSlice(OutT *dst, const float (&acc)[E], float alpha, float beta)
{
    // C is read at most once and written once per product: streamed, so that it does not displace B in L2.
    float z[E];
    if (beta != 0.0f) {
        constexpr int kVecs = E * (int)sizeof(OutT) / 16;
        alignas(16) OutT old[E];
#pragma unroll
        for (int i = 0; i < kVecs; ++i)
            reinterpret_cast<uint4 *>(old)[i] = B200SP_SPMM_C_LOAD(reinterpret_cast<const uint4 *>(dst) + i);
#pragma unroll
        for (int i = 0; i < E; ++i) z[i] = __fadd_rn(__fmul_rn(alpha, acc[i]), __fmul_rn(beta, ToF32(old[i])));
    } else {
#pragma unroll
        for (int i = 0; i < E; ++i) z[i] = __fmul_rn(alpha, acc[i]);
    }
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
        for (int i = 0; i < E; i += 4)
            B200SP_SPMM_C_STORE(reinterpret_cast<float4 *>(dst + i), make_float4(z[i], z[i + 1], z[i + 2], z[i + 3]));
    } else {
        static_assert(E == 8, "16-bit output slices are 8 wide");
        alignas(16) OutT o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = FromF32<OutT>(z[i]);
        B200SP_SPMM_C_STORE(reinterpret_cast<uint4 *>(dst), *reinterpret_cast<const uint4 *>(o));
    }
}

// kLanes lanes lie side by side on one row of B (16 bytes each); a warp therefore carries
// 32 / kLanes rows of A at once.  Rows of up to kLongRow entries are summed by their group in
// CSR order; longer rows belong to the segment CTAs at the front of the grid.
template <typename ValT, typename OutT, bool kKahan, int kLanes>
__global__ void __launch_bounds__(kThreads) SpmmFastKernel(const FastArgs<ValT, OutT> a)
{
    constexpr int E = Pack<ValT>::kElems;
    constexpr int kRowsPerWarp = 32 / kLanes;
    constexpr int kTileCols = kLanes * E;
    __shared__ float sAcc[kWarps][kMaxTileCols];
    __shared__ int sLast;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int li = lane & (kLanes - 1);
    const float alpha = a.sc.Alpha();
    const float beta = a.sc.Beta();

    if ((int)blockIdx.x >= a.nsegs) {
        // ---- one lane group per row ----
        const long long row = ((long long)(blockIdx.x - a.nsegs) * kWarps + warp) * kRowsPerWarp + lane / kLanes;
        int s = 0, e = 0;
        if (row < a.m) {
            s = a.rowPtr[row];
            e = a.rowPtr[row + 1];
            if (e - s > kLongRow) e = s;  // owned by segment CTAs
        }
        int trips = (e - s + kLanes - 1) / kLanes;
#pragma unroll
        for (int off = kLanes; off < 32; off <<= 1) {
            const int other = __shfl_xor_sync(0xffffffffu, trips, off);
            trips = other > trips ? other : trips;
        }
        const bool skip = row >= a.m || (a.rowPtr[row + 1] - a.rowPtr[row] > kLongRow);
        for (int col0 = 0; col0 < a.n; col0 += kTileCols) {
            const int col = col0 + li * E;
            const bool colLive = col < a.n;
            const bool allLive = col0 + kTileCols <= a.n;
            float acc[E], comp[E];
#pragma unroll
            for (int i = 0; i < E; ++i) acc[i] = comp[i] = 0.0f;
            RowDot<ValT, kKahan, kLanes>(a.colInd, a.val, a.B + col, a.ldb, s, e, trips, colLive, allLive, acc, comp);
            if (kKahan) {
#pragma unroll
                for (int i = 0; i < E; ++i) acc[i] -= comp[i];
            }
            if (!skip && colLive) StoreRowSlice<OutT, E>(a.C + row * a.ldc + col, acc, alpha, beta);
        }
        return;
    }

    // ---- one CTA per long-row segment: the four warps take a quarter each ----
    const SegEntry seg = a.segs[blockIdx.x];
    const LongRow lr = a.longRows[seg.longIdx];
    const int rowStart = a.rowPtr[seg.row];
    const int rowEnd = a.rowPtr[seg.row + 1];
    const int segStart = rowStart + seg.seg * kSegNnz;
    const int segEnd = segStart + kSegNnz < rowEnd ? segStart + kSegNnz : rowEnd;
    // inside a warp the lane groups take interleaved kLanes-wide chunks of the warp's quarter
    int ws = segStart + warp * kWarpSegNnz;
    int we = ws + kWarpSegNnz;
    if (ws > segEnd) ws = segEnd;
    if (we > segEnd) we = segEnd;
    const int g = lane / kLanes;
    float *partial = a.partials + (long long)(lr.partBase + seg.seg) * a.n;

    for (int col0 = 0; col0 < a.n; col0 += kTileCols) {
        const int col = col0 + li * E;
        const bool colLive = col < a.n;
        const bool allLive = col0 + kTileCols <= a.n;
        float acc[E], comp[E];
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = comp[i] = 0.0f;
        // group g walks chunks g, g + kRowsPerWarp, ... of [ws, we)
        const int nChunks = (we - ws + kLanes - 1) / kLanes;
        for (int ch0 = 0; ch0 < nChunks; ch0 += kRowsPerWarp) {  // same trip count in every group
            const int ch = ch0 + g;
            const int cs = ws + ch * kLanes < we ? ws + ch * kLanes : we;
            const int ce = cs + kLanes < we ? cs + kLanes : we;
            RowDot<ValT, kKahan, kLanes>(a.colInd, a.val, a.B + col, a.ldb, cs, ce, 1, colLive, allLive, acc, comp);
        }
#pragma unroll
        for (int i = 0; i < E; ++i) {
            if (kKahan) acc[i] -= comp[i];
#pragma unroll
            for (int off = kLanes; off < 32; off <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
        }
        if (lane < kLanes) {
#pragma unroll
            for (int i = 0; i < E; ++i) sAcc[warp][li * E + i] = acc[i];
        }
        __syncthreads();
        // warp 0 adds the four warps' slices in warp order
        if (warp == 0 && lane < kLanes && colLive) {
            float tot[E];
#pragma unroll
            for (int i = 0; i < E; ++i) {
                tot[i] = sAcc[0][li * E + i];
#pragma unroll
                for (int w = 1; w < kWarps; ++w) tot[i] += sAcc[w][li * E + i];
            }
            if (lr.nseg == 1) {
                StoreRowSlice<OutT, E>(a.C + (long long)seg.row * a.ldc + col, tot, alpha, beta);
            } else {
#pragma unroll
                for (int i = 0; i < E; ++i) partial[col + i] = tot[i];
            }
        }
        __syncthreads();
    }
    if (lr.nseg == 1) return;

    // Arrival: the segment that comes last sums all partial rows in segment order.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(a.counters + seg.longIdx, 1);
        sLast = (old == lr.nseg - 1);
        if (sLast) a.counters[seg.longIdx] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sLast) return;
    __threadfence();
    const float *first = a.partials + (long long)lr.partBase * a.n;
    for (int col = threadIdx.x * E; col < a.n; col += kThreads * E) {
        float tot[E];
#pragma unroll
        for (int i = 0; i < E; ++i) tot[i] = 0.0f;
        for (int sgi = 0; sgi < lr.nseg; ++sgi) {
#pragma unroll
            for (int i = 0; i < E; ++i) tot[i] += __ldcg(first + (long long)sgi * a.n + col + i);
        }
        StoreRowSlice<OutT, E>(a.C + (long long)seg.row * a.ldc + col, tot, alpha, beta);
    }
}

// ---------------------------------------------------------------- long rows by column blocks

// When B is much larger than L2, a long row of A gathers every one of its B rows from DRAM.  Rows of more than
// kLongRow entries are few and hold a large share of the non-zeros (a graph's hubs); with ascending columns the
// entries of such a row that fall into one block of consecutive B rows are contiguous in col_ind.  So B is cut
// into blocks of about kBlockBytes and the grid walks the pieces (row, block) block by block: while one block
// is being worked on, every long row gathers from the same few megabytes, which the first touch brings into L2
// and the evict-last policy of the B loads keeps there.  Pieces are cut into units of at most kUnitNnz entries so
// that all units take about the same time and the grid stays inside a window of one or two blocks.  A warp sums
// one unit in CSR order into one partial row; the warp that completes a row adds its partial rows in column
// order (fixed order: the same bits every run) and applies the epilogue.
struct BlockArgs {
    int nUnits;
    const BlockUnit *units;   // ordered by column block
    const int2 *rowSlots;     // [long row] {first partial slot, slots}
    int32_t *counters;        // [long row] arrivals
    float *partials;          // [slot][n]
};

// Packed fp32 arithmetic of sm_100: one instruction, two fused multiply-adds.  The long rows are not bound to the
// golden's separate multiply and add (their sums are regrouped by block anyway), and this kernel, fed from L2,
// is limited by instruction issue rather than by DRAM.
__device__ __forceinline__ void Fma2(float2 &acc, float x, float y, float v)
{
    unsigned long long a, bq, c;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(x), "f"(y));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bq) : "f"(v));
    asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(acc.x), "f"(acc.y));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(bq));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(acc.x), "=f"(acc.y) : "l"(c));
}

// acc[0 .. E/2) += v * (the E values of 16 bytes of a B row)
template <typename ValT> struct FusedRow;
template <> struct FusedRow<float> {
    static __device__ __forceinline__ void Add(const uint4 &q, float v, float2 (&acc)[2])
    {
        Fma2(acc[0], __uint_as_float(q.x), __uint_as_float(q.y), v);
        Fma2(acc[1], __uint_as_float(q.z), __uint_as_float(q.w), v);
    }
};
template <> struct FusedRow<__nv_bfloat16> {
    static __device__ __forceinline__ void Add(const uint4 &q, float v, float2 (&acc)[4])
    {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            Fma2(acc[i], __uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u), v);
    }
};
template <> struct FusedRow<__half> {
    static __device__ __forceinline__ void Add(const uint4 &q, float v, float2 (&acc)[4])
    {
        const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            Fma2(acc[i], f.x, f.y, v);
        }
    }
};

// Measured on the 2 M x 2 M graph matrix with 512-byte rows of B (2,767 long rows, 14.0 M entries), this kernel
// alone, microseconds: the segment CTAs it replaces 1067 (DRAM-bound: every B row fetched from DRAM);
// blocks of 16 / 24 / 32 / 48 / 64 MB 848 / 729 / 727 / 715 / 725; units of 128 / 256 / 512 entries
// 851 / 727 / 813; 2 / 4 / 8 / 16 rows in flight per lane 879 / 727 / 752 / 857; a fixed grid of 4 CTAs per SM
// walking the units with a stride 1739 (its warps drift apart and the window of blocks in use outgrows L2).
// At 714 us: 1.9 GB of DRAM traffic instead of 7.2, issue slots 54 % busy (28 warp instructions per B row).
#ifndef B200SP_SPMM_BLOCK_BATCH
#define B200SP_SPMM_BLOCK_BATCH 4   // B rows a lane has in flight
#endif
#ifndef B200SP_SPMM_BLOCK_CTAS
#define B200SP_SPMM_BLOCK_CTAS 0    // > 0: a fixed grid of that many CTAs per SM walks the units; 0: a CTA per 4 units
#endif

template <typename ValT, typename OutT>
__global__ void __launch_bounds__(kThreads) SpmmLongBlockKernel(const FastArgs<ValT, OutT> a, const BlockArgs b)
{
    constexpr int E = Pack<ValT>::kElems;
    constexpr int kTileCols = 32 * E;
    constexpr int kBatch = B200SP_SPMM_BLOCK_BATCH;
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * kWarps;
    for (long long unit = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5); unit < b.nUnits; unit += warpsTotal) {
        const int4 raw = __ldg(reinterpret_cast<const int4 *>(b.units) + unit);
        const int s = raw.x, e = raw.y, li = raw.z, slot = raw.w;
        float *partial = b.partials + (long long)slot * a.n;
        for (int col0 = 0; col0 < a.n; col0 += kTileCols) {
            const int col = col0 + lane * E;
            const bool colLive = col < a.n;
            const ValT *Bs = a.B + (colLive ? col : 0);
            float2 acc[E / 2];
#pragma unroll
            for (int i = 0; i < E / 2; ++i) acc[i] = make_float2(0.0f, 0.0f);
            for (int p0 = s; p0 < e; p0 += 32) {
                const int cnt = e - p0 < 32 ? e - p0 : 32;
                int myCol = 0;
                float myVal = 0.0f;
                if (lane < cnt) {
                    myCol = __ldcs(a.colInd + p0 + lane);
                    myVal = ToF32(__ldcs(a.val + p0 + lane));
                }
                int j = 0;
                for (; j + kBatch <= cnt; j += kBatch) {  // cnt is the same in every lane
                    uint4 q[kBatch];
                    float v[kBatch];
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        const int c = __shfl_sync(0xffffffffu, myCol, j + u);
                        v[u] = __shfl_sync(0xffffffffu, myVal, j + u);
                        q[u] = LoadB16(Bs + (long long)c * a.ldb);
                    }
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) FusedRow<ValT>::Add(q[u], v[u], acc);
                }
                for (; j < cnt; ++j) {
                    const int c = __shfl_sync(0xffffffffu, myCol, j);
                    const float v = __shfl_sync(0xffffffffu, myVal, j);
                    const uint4 q = LoadB16(Bs + (long long)c * a.ldb);
                    FusedRow<ValT>::Add(q, v, acc);
                }
            }
            if (colLive) {
#pragma unroll
                for (int i = 0; i < E / 2; i += 2)
                    __stcg(reinterpret_cast<float4 *>(partial + col + 2 * i),
                           make_float4(acc[i].x, acc[i].y, acc[i + 1].x, acc[i + 1].y));
            }
        }
        // Arrival: the unit that comes last adds the row's partial rows in slot (= column) order.
        const int2 rs = __ldg(b.rowSlots + li);
        __threadfence();
        int last = 0;
        if (lane == 0) {
            const int old = atomicAdd(b.counters + li, 1);
            last = old == rs.y - 1;
            if (last) b.counters[li] = 0;  // ready for the next launch
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) continue;
        __threadfence();
        const float alpha = a.sc.Alpha();
        const float beta = a.sc.Beta();
        const int row = a.longRows[li].row;
        const float *first = b.partials + (long long)rs.x * a.n;
        for (int col = lane * E; col < a.n; col += kTileCols) {
            float tot[E];
#pragma unroll
            for (int i = 0; i < E; ++i) tot[i] = 0.0f;
#pragma unroll 4
            for (int sl = 0; sl < rs.y; ++sl) {
#pragma unroll
                for (int i = 0; i < E; i += 4) {
                    const float4 v = __ldcg(reinterpret_cast<const float4 *>(first + (long long)sl * a.n + col + i));
                    tot[i] += v.x; tot[i + 1] += v.y; tot[i + 2] += v.z; tot[i + 3] += v.w;
                }
            }
            StoreRowSlice<OutT, E>(a.C + (long long)row * a.ldc + col, tot, alpha, beta);
        }
    }
}

// ---------------------------------------------------------------- row-stream path

// For B rows of 512 or 1024 bytes.  A warp owns 32 consecutive rows of A and walks their
// non-zeros as one stream, in CSR order, across the row boundaries; the B row of every entry
// is brought into shared memory by the copy engine (cp.async.bulk, one row per copy, completion
// counted on an mbarrier) several batches ahead of its use, so the chain row_ptr -> col_ind ->
// B row -> C row that bounds a row-at-a-time kernel on matrices full of one- and two-entry
// rows is paid once per warp, not once per row, and no registers hold data in flight.
// Every lane owns kRowBytes / 32 bytes of the row; each output keeps one fp32 accumulator
// that takes its products in CSR order with separate multiply and add, as in the kernel above,
// so the results are the same bits.  Rows above kLongRow entries are left to the segment CTAs
// of SpmmFastKernel.
// Measured on the 2 M x 2 M graph matrix with 512-byte rows (ms per product, segment CTAs included):
// 3 buffers x 16 rows x 4 warps per CTA 5.28; 2 x 16 x 4 3.97; 2 x 8 x 4 3.29; 2 x 4 x 4 3.38;
// 2 x 8 x 2 2.99; 2 x 8 x 1 2.91.  Less shared memory per warp means more warps per SM, and
// one warp per CTA gives the memory of a finished warp back at once.
#ifndef B200SP_SPMM_STREAM_BUFFERS
#define B200SP_SPMM_STREAM_BUFFERS 2
#endif
#ifndef B200SP_SPMM_STREAM_BATCH_BYTES
#define B200SP_SPMM_STREAM_BATCH_BYTES 4096
#endif
#ifndef B200SP_SPMM_STREAM_WARPS
#define B200SP_SPMM_STREAM_WARPS 1
#endif
constexpr int kStreamBuffers = B200SP_SPMM_STREAM_BUFFERS;  // batches of B rows per warp: one in use, the rest in flight
constexpr int kStreamWarps = B200SP_SPMM_STREAM_WARPS;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStreamRows = 32;                              // rows of A per warp
constexpr long long kStreamWaitCycles = 1ll << 31;           // SM clocks (about a second) to wait on one barrier before giving up
// What the next launches pass to the kernel as its wait limit and as bytes to expect beyond those it copies
// (b200sp_spmm_stream_wait_test: a test makes a wait run out without any fault by expecting bytes nobody sends).
long long gHostStreamWaitCycles = kStreamWaitCycles;
unsigned gHostStreamExtraTx = 0;

__device__ int gStreamError;  // set when a wait ran out (never observed; the kernel then stops writing C)

__device__ __forceinline__ uint32_t SmemAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void MbarInit(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Polls with a time limit; false when the limit was reached.
__device__ __forceinline__ bool MbarWait(uint64_t *bar, uint32_t parity, long long limit)
{
    if (MbarTryWait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!MbarTryWait(bar, parity)) {
        if (clock64() - t0 > limit) return false;
    }
    return true;
}
// One row: global -> shared through the copy engine; both addresses 16-byte aligned, bytes a multiple of 16.
// B200SP_SPMM_STREAM_B_POLICY 1: the copies carry an L2 evict-first policy, so that the rows this kernel streams
// through L2 once do not displace the block of B rows that SpmmLongBlockKernel, running beside it, keeps there.
// Measured: the row-stream kernel alone slows from 1.90 to 2.01 ms with it and the pair gains nothing; off.
#ifndef B200SP_SPMM_STREAM_B_POLICY
#define B200SP_SPMM_STREAM_B_POLICY 0
#endif
__device__ __forceinline__ void BulkLoadRow(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
#if B200SP_SPMM_STREAM_B_POLICY == 1
    uint64_t pol;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            SmemAddr(dst)),
        "l"(src), "r"(bytes), "r"(SmemAddr(bar)), "l"(pol)
        : "memory");
#else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     SmemAddr(dst)),
                 "l"(src), "r"(bytes), "r"(SmemAddr(bar))
                 : "memory");
#endif
}

template <int kBytes> struct LaneWords {  // kBytes of shared memory as 32-bit words
    static constexpr int kWords = kBytes / 4;
    static __device__ __forceinline__ void Load(const unsigned char *p, uint32_t (&w)[kWords])
    {
        if constexpr (kBytes == 4) {
            w[0] = *reinterpret_cast<const uint32_t *>(p);
        } else if constexpr (kBytes == 8) {
            const uint2 q = *reinterpret_cast<const uint2 *>(p);
            w[0] = q.x; w[1] = q.y;
        } else {
            static_assert(kBytes % 16 == 0, "a lane owns 4, 8 or a multiple of 16 bytes of a B row");
#pragma unroll
            for (int i = 0; i < kBytes / 16; ++i) {
                const uint4 q = reinterpret_cast<const uint4 *>(p)[i];
                w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
            }
        }
    }
};

template <typename ValT, int kWords> struct WordsToF32;
template <int kWords> struct WordsToF32<float, kWords> {
    static constexpr int kElems = kWords;
    static __device__ __forceinline__ void Convert(const uint32_t (&w)[kWords], float (&out)[kElems])
    {
#pragma unroll
        for (int i = 0; i < kWords; ++i) out[i] = __uint_as_float(w[i]);
    }
};
template <int kWords> struct WordsToF32<__half, kWords> {
    static constexpr int kElems = 2 * kWords;
    static __device__ __forceinline__ void Convert(const uint32_t (&w)[kWords], float (&out)[kElems])
    {
#pragma unroll
        for (int i = 0; i < kWords; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
};
template <int kWords> struct WordsToF32<__nv_bfloat16, kWords> {
    static constexpr int kElems = 2 * kWords;
    static __device__ __forceinline__ void Convert(const uint32_t (&w)[kWords], float (&out)[kElems])
    {
#pragma unroll
        for (int i = 0; i < kWords; ++i) {  // bf16 -> fp32 is a 16-bit shift
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// E consecutive outputs of one lane: z = alpha * acc + beta * old, stored with the widest aligned vector.
template <typename OutT, int E>
__device__ __forceinline__ void LoadOld(const OutT *src, float (&old)[E])
{
#pragma unroll
    for (int i = 0; i < E; ++i) old[i] = ToF32(src[i]);  // contiguous: the compiler merges these into vector loads
}
template <typename OutT, int E>
__device__ __forceinline__ void StoreSlice(OutT *dst, const float (&acc)[E], const float (&old)[E], float alpha,
                                           float beta)
{
    float z[E];
#pragma unroll
    for (int i = 0; i < E; ++i)
        z[i] = beta != 0.0f ? __fadd_rn(__fmul_rn(alpha, acc[i]), __fmul_rn(beta, old[i])) : __fmul_rn(alpha, acc[i]);
    constexpr int kBytes = E * (int)sizeof(OutT);
    alignas(16) OutT o[E];
#pragma unroll
    for (int i = 0; i < E; ++i) o[i] = FromF32<OutT>(z[i]);
    if constexpr (kBytes % 16 == 0) {
#pragma unroll
        for (int i = 0; i < kBytes / 16; ++i)
            reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(o)[i];
    } else if constexpr (kBytes == 8) {
        *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(o);
    } else {
        static_assert(kBytes == 4, "a lane writes 4, 8 or a multiple of 16 bytes of a C row");
        *reinterpret_cast<uint32_t *>(dst) = *reinterpret_cast<const uint32_t *>(o);
    }
}

template <typename ValT, typename OutT>
struct StreamArgs {
    const int32_t *rowPtr;
    const int32_t *colInd;
    const ValT *val;
    const ValT *B;
    OutT *C;
    int m;
    long long ldb;
    long long ldc;
    ScalarsF sc;
    long long waitCycles;   // limit of every wait on a copy barrier, in SM clocks
    unsigned extraTx;       // bytes expected on every barrier beyond those copied (0 outside the wait test)
};

template <int kRowBytes> struct StreamShape {
    static constexpr int kBatch = B200SP_SPMM_STREAM_BATCH_BYTES / kRowBytes;  // B rows per batch
    static_assert(kBatch >= 1 && kBatch <= 32, "a lane issues at most one row copy per batch");
    static constexpr int kWarpBytes = kStreamBuffers * (kBatch * kRowBytes + kBatch * 8) + 64;  // data, val, meta, barriers
    static constexpr int kCtaBytes = kStreamWarps * kWarpBytes;
};

template <typename ValT, typename OutT, int kRowBytes>
__global__ void __launch_bounds__(kStreamThreads) SpmmRowStreamKernel(const StreamArgs<ValT, OutT> a)
{
    using Shape = StreamShape<kRowBytes>;
    constexpr int kBatch = Shape::kBatch;
    constexpr int kLaneBytes = kRowBytes / 32;
    constexpr int kWords = kLaneBytes / 4;
    constexpr int E = WordsToF32<ValT, kWords>::kElems;
    extern __shared__ __align__(128) unsigned char sRaw[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    unsigned char *base = sRaw + (size_t)warp * Shape::kWarpBytes;
    unsigned char *sData = base;                                                          // [buffers][kBatch][kRowBytes]
    float *sVal = reinterpret_cast<float *>(base + kStreamBuffers * kBatch * kRowBytes);  // [buffers][kBatch]
    int *sMeta = reinterpret_cast<int *>(sVal + kStreamBuffers * kBatch);                 // [buffers][kBatch]
    uint64_t *sBar = reinterpret_cast<uint64_t *>(sMeta + kStreamBuffers * kBatch);       // [buffers]

    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < kStreamBuffers; ++i) MbarInit(sBar + i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const float alpha = a.sc.Alpha();
    const float beta = a.sc.Beta();
    const long long r0 = ((long long)blockIdx.x * kStreamWarps + warp) * kStreamRows;
    if (r0 >= a.m) return;

    // This lane's row: bounds, length, and where its entries start in the warp's stream.
    const long long myRow = r0 + lane;
    int s = 0, len = 0;
    bool mine = false;
    if (myRow < a.m) {
        s = a.rowPtr[myRow];
        len = a.rowPtr[myRow + 1] - s;
        mine = len <= kLongRow;  // longer rows are written by the segment CTAs
        if (!mine) len = 0;
    }
    int off = len;  // inclusive scan over the lanes, then made exclusive
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, off, d);
        if (lane >= d) off += t;
    }
    const int total = __shfl_sync(0xffffffffu, off, 31);
    off -= len;

    OutT *cRow0 = a.C + r0 * a.ldc + lane * E;
    // Rows without entries: C = beta * C.
    unsigned emptyMask = __ballot_sync(0xffffffffu, mine && len == 0);
    while (emptyMask != 0) {
        const int l = __ffs(emptyMask) - 1;
        emptyMask &= emptyMask - 1;
        float zero[E], old[E];
#pragma unroll
        for (int i = 0; i < E; ++i) zero[i] = old[i] = 0.0f;
        OutT *dst = cRow0 + (long long)l * a.ldc;
        if (beta != 0.0f) LoadOld<OutT, E>(dst, old);
        StoreSlice<OutT, E>(dst, zero, old, alpha, beta);
    }
    if (total == 0) return;
    const unsigned liveMask = __ballot_sync(0xffffffffu, len > 0);

    const int nBatches = (total + kBatch - 1) / kBatch;
    // Entry q of the stream (held by lane q % kBatch of its batch): column, value, and which row it
    // belongs to / whether it ends that row.
    int eCol = 0, eMeta = 0;
    float eVal = 0.0f;
    auto fetchEntries = [&](int k) {
        const int q = k * kBatch + lane;
        // last lane whose stream offset is <= q: the row that holds entry q
        int lo = 0;
#pragma unroll
        for (int step = 16; step > 0; step >>= 1) {
            const int cand = lo + step;
            const int offC = __shfl_sync(0xffffffffu, off, cand & 31);
            if (cand < 32 && offC <= q) lo = cand;
        }
        const int sL = __shfl_sync(0xffffffffu, s, lo);
        const int offL = __shfl_sync(0xffffffffu, off, lo);
        const int lenL = __shfl_sync(0xffffffffu, len, lo);
        if (lane < kBatch && q < total) {
            const int p = sL + (q - offL);
            eCol = __ldcs(a.colInd + p);
            eVal = ToF32(__ldcs(a.val + p));
            eMeta = lo | ((q - offL == lenL - 1) ? 0x100 : 0);
        }
    };
    auto issueBatch = [&](int k) {
        const int buf = k % kStreamBuffers;
        const int live = total - k * kBatch < kBatch ? total - k * kBatch : kBatch;
        if (lane == 0) MbarExpectTx(sBar + buf, (uint32_t)live * kRowBytes + a.extraTx);
        __syncwarp();
        if (lane < live) {
            sVal[buf * kBatch + lane] = eVal;
            sMeta[buf * kBatch + lane] = eMeta;
            BulkLoadRow(sData + ((size_t)buf * kBatch + lane) * kRowBytes, a.B + (long long)eCol * a.ldb, kRowBytes,
                        sBar + buf);
        }
    };

    // prologue: all but one buffer in flight
    const int ahead = kStreamBuffers - 1;
    for (int k = 0; k < ahead && k < nBatches; ++k) {
        fetchEntries(k);
        issueBatch(k);
    }
    if (ahead < nBatches) fetchEntries(ahead);

    float acc[E], old[E];
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] = old[i] = 0.0f;
    // C of the row being summed is requested when the row before it is written (when the warp starts, for the first)
    if (beta != 0.0f) LoadOld<OutT, E>(cRow0 + (long long)(__ffs(liveMask) - 1) * a.ldc, old);

    int failedAt = -1;
    for (int k = 0; k < nBatches; ++k) {
        if (k + ahead < nBatches) issueBatch(k + ahead);           // uses the entries fetched one trip ago
        if (k + ahead + 1 < nBatches) fetchEntries(k + ahead + 1);  // lands while this batch is summed
        const int buf = k % kStreamBuffers;
        __syncwarp();
        if (!MbarWait(sBar + buf, (uint32_t)(k / kStreamBuffers) & 1u, a.waitCycles)) {
            failedAt = k;
            if (lane == 0) atomicExch(&gStreamError, 1);
            break;
        }
        const int live = total - k * kBatch < kBatch ? total - k * kBatch : kBatch;
        const unsigned char *rowData = sData + (size_t)buf * kBatch * kRowBytes + lane * kLaneBytes;
#pragma unroll 4
        for (int j = 0; j < live; ++j) {
            const int meta = sMeta[buf * kBatch + j];
            const float v = sVal[buf * kBatch + j];
            uint32_t w[kWords];
            LaneWords<kLaneBytes>::Load(rowData + (size_t)j * kRowBytes, w);
            float b[E];
            WordsToF32<ValT, kWords>::Convert(w, b);
#pragma unroll
            for (int i = 0; i < E; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(v, b[i]));
            if (meta & 0x100) {  // last entry of its row (warp-uniform)
                const int l = meta & 0xff;
                StoreSlice<OutT, E>(cRow0 + (long long)l * a.ldc, acc, old, alpha, beta);
#pragma unroll
                for (int i = 0; i < E; ++i) acc[i] = 0.0f;
                const unsigned rest = l < 31 ? liveMask & (0xfffffffeu << l) : 0u;
                if (beta != 0.0f && rest != 0) LoadOld<OutT, E>(cRow0 + (long long)(__ffs(rest) - 1) * a.ldc, old);
            }
        }
        __syncwarp();  // every lane is done with this buffer before a later batch is copied into it
    }
    if (failedAt >= 0) {
        // A wait ran out: this warp writes no more of C.  Give the copies still in flight (batches
        // failedAt .. failedAt + ahead) a bounded chance to land before the shared memory they
        // target is released.
        for (int k = failedAt; k <= failedAt + ahead && k < nBatches; ++k)
            (void)MbarWait(sBar + k % kStreamBuffers, (uint32_t)(k / kStreamBuffers) & 1u, a.waitCycles);
    }
}

// ---------------------------------------------------------------- generic path

struct GenericShape {
    long long m, n, ldb, ldc;
    int bRowMajor, cRowMajor, opB, kahan;
};

__device__ __forceinline__ long long BIndex(const GenericShape &g, long long c, long long j)
{
    // op(B)(c, j): same four cases as the golden SpmmCpuFp32 (spmm_test.cpp:142-151).
    if (!g.opB) return g.bRowMajor ? c * g.ldb + j : j * g.ldb + c;
    return g.bRowMajor ? j * g.ldb + c : c * g.ldb + j;
}

template <typename ValT, typename OutT>
__global__ void __launch_bounds__(256) SpmmGenericFloatKernel(const int32_t *__restrict__ rowPtr,
                                                               const int32_t *__restrict__ colInd,
                                                               const ValT *__restrict__ val,
                                                               const ValT *__restrict__ B, OutT *__restrict__ C,
                                                               GenericShape g, ScalarsF sc)
{
    const float alpha = sc.Alpha();
    const float beta = sc.Beta();
    const long long total = g.m * g.n;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (long long)gridDim.x * blockDim.x) {
        const long long r = w / g.n;
        const long long j = w - r * g.n;
        float acc = 0.0f, comp = 0.0f;
        const int e = rowPtr[r + 1];
        for (int p = rowPtr[r]; p < e; ++p) {
            const float b = ToF32(B[BIndex(g, colInd[p], j)]);
            if (g.kahan) Accumulate<true>(ToF32(val[p]), b, acc, comp);
            else Accumulate<false>(ToF32(val[p]), b, acc, comp);
        }
        if (g.kahan) acc -= comp;
        const long long ci = g.cRowMajor ? r * g.ldc + j : j * g.ldc + r;
        float z = __fmul_rn(alpha, acc);
        if (beta != 0.0f) z = __fadd_rn(z, __fmul_rn(beta, ToF32(C[ci])));
        C[ci] = FromF32<OutT>(z);
    }
}

__global__ void __launch_bounds__(256) SpmmGenericInt8Kernel(const int32_t *__restrict__ rowPtr,
                                                              const int32_t *__restrict__ colInd,
                                                              const int8_t *__restrict__ val,
                                                              const int8_t *__restrict__ B, int32_t *__restrict__ C,
                                                              GenericShape g, ScalarsI sc)
{
    const int32_t alpha = sc.Alpha();
    const int32_t beta = sc.Beta();
    const long long total = g.m * g.n;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (long long)gridDim.x * blockDim.x) {
        const long long r = w / g.n;
        const long long j = w - r * g.n;
        int32_t acc = 0;
        const int e = rowPtr[r + 1];
        for (int p = rowPtr[r]; p < e; ++p)
            acc += (int32_t)val[p] * (int32_t)B[BIndex(g, colInd[p], j)];
        const long long ci = g.cRowMajor ? r * g.ldc + j : j * g.ldc + r;
        // int64 epilogue with saturation (reference spmm_kernel.cpp:251-266)
        long long wide = (long long)alpha * (long long)acc;
        if (beta != 0) wide += (long long)beta * (long long)C[ci];
        if (wide > 2147483647LL) wide = 2147483647LL;
        if (wide < -2147483648LL) wide = -2147483648LL;
        C[ci] = (int32_t)wide;
    }
}

// ---------------------------------------------------------------- host dispatch

ScalarsF MakeF(const b200spScalars *s)
{
    return {s->alpha_f, s->beta_f, static_cast<const float *>(s->alpha_dev), static_cast<const float *>(s->beta_dev)};
}
ScalarsI MakeI(const b200spScalars *s)
{
    return {s->alpha_i, s->beta_i, static_cast<const int32_t *>(s->alpha_dev),
            static_cast<const int32_t *>(s->beta_dev)};
}

bool Aligned16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

#ifndef B200SP_SPMM_USE_STREAM
#define B200SP_SPMM_USE_STREAM 1
#endif
// The copy engine of an SM starts about one row copy per 20 clocks (measured: 16.8 M copies of
// 256 bytes took 1.25 ms on 148 SMs), so rows shorter than 512 bytes move faster through plain
// 128-bit loads and stay with SpmmFastKernel (256-byte rows, 64 per row of A: 1249 us against 265 us).

template <typename ValT, typename OutT, int kRowBytes>
int LaunchRowStream(const StreamArgs<ValT, OutT> &sa, cudaStream_t stream)
{
    constexpr int kSmem = StreamShape<kRowBytes>::kCtaBytes;
    static bool configured[64] = {};  // per device: this instantiation uses kSmem bytes of dynamic shared memory
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(SpmmRowStreamKernel<ValT, OutT, kRowBytes>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    const long long rowsPerBlock = (long long)kStreamWarps * kStreamRows;
    const unsigned grid = (unsigned)((sa.m + rowsPerBlock - 1) / rowsPerBlock);
    SpmmRowStreamKernel<ValT, OutT, kRowBytes><<<grid, kStreamThreads, kSmem, stream>>>(sa);
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

template <typename ValT, typename OutT>
int LaunchFloat(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *B, void *C,
                const b200spSpmmShape *sh, const b200spScalars *s, void *plan, int32_t segments,
                cudaStream_t stream)
{
    constexpr int E = Pack<ValT>::kElems;
    // B rows contiguous in memory: (N, row-major) or (T, column-major).
    const bool bRowsContig = (sh->op_b == 0 && sh->order_b == 0) || (sh->op_b == 1 && sh->order_b == 1);
    const bool fast = plan != nullptr && bRowsContig && sh->order_c == 0 && sh->n % E == 0 && sh->ldb % E == 0 &&
                      sh->ldc % E == 0 && Aligned16(B) && Aligned16(C);
    if (fast) {
        const PlanLayout L = LayoutFor(sh->m, sh->nnz, sh->n);
        char *p = static_cast<char *>(plan);
        FastArgs<ValT, OutT> a;
        a.rowPtr = rowPtr;
        a.colInd = colInd;
        a.val = static_cast<const ValT *>(val);
        a.B = static_cast<const ValT *>(B);
        a.C = static_cast<OutT *>(C);
        a.m = (int)sh->m;
        a.n = (int)sh->n;
        a.ldb = sh->ldb;
        a.ldc = sh->ldc;
        a.sc = MakeF(s);
        a.longRows = reinterpret_cast<const LongRow *>(p + L.offLong);
        a.segs = reinterpret_cast<const SegEntry *>(p + L.offSegs);
        a.counters = reinterpret_cast<int32_t *>(p + L.offCounters);
        a.partials = reinterpret_cast<float *>(p + L.offPartials);
        int lanes_ = 1;  // lanes side by side on a row of B
        while (lanes_ < 32 && lanes_ * E < sh->n) lanes_ <<= 1;
        const long long rowsPerBlock = (long long)kWarps * (32 / lanes_);
        // B rows of 128 / 256 / 512 bytes: rows of up to kLongRow entries go to the row-stream kernel,
        // and SpmmFastKernel is launched for its segment CTAs only.
        const long long rowBytes = sh->n * (long long)sizeof(ValT);
        const bool stream_ = !sh->kahan && (rowBytes == 512 || rowBytes == 1024) && sh->m > 0 && B200SP_SPMM_USE_STREAM;
        // Long rows by column blocks of B (found applicable by b200sp_spmm_analyze_blocks) instead of by segments.
        const bool byBlocks = sh->block_units > 0 && sh->long_rows > 0 && !sh->kahan && rowBytes >= kBlockMinRowBytes &&
                              sh->block_units <= L.capBlockSlots;
        if (byBlocks) segments = 0;
        a.nsegs = segments;
        BlockArgs ba{};
        if (byBlocks) {
            ba.nUnits = sh->block_units;
            ba.units = reinterpret_cast<const BlockUnit *>(p + L.offUnits);
            ba.rowSlots = reinterpret_cast<const int2 *>(p + L.offRowSlots);
            ba.counters = reinterpret_cast<int32_t *>(p + L.offBlockCounters);
            ba.partials = reinterpret_cast<float *>(p + L.offBlockPartials);
        }
        const long long blockUnits = byBlocks ? (long long)ba.nUnits : 0;
        // With both kernels to run, the segment CTAs (the long rows: few CTAs, each with much work) are forked
        // onto the side stream first and the row-stream kernel shares the SMs with them.
        b200sp::SideLanes *lanes = nullptr;
        cudaStream_t segStream = stream;
#ifndef B200SP_SPMM_FORK_SEGMENTS
#define B200SP_SPMM_FORK_SEGMENTS 1
#endif
        if (B200SP_SPMM_FORK_SEGMENTS && ((stream_ && segments > 0) || byBlocks)) {
            lanes = b200sp::GetSideLanes();
            if (lanes != nullptr) {
                if (cudaEventRecord(lanes->fork, stream) != cudaSuccess ||
                    cudaStreamWaitEvent(lanes->stream[0], lanes->fork, 0) != cudaSuccess)
                    return (int)cudaGetLastError();
                segStream = lanes->stream[0];
            }
        }
        auto launchFast = [&](unsigned grid, cudaStream_t st) {
            auto launch = [&]<int kLanes>() {
                if (sh->kahan) SpmmFastKernel<ValT, OutT, true, kLanes><<<grid, kThreads, 0, st>>>(a);
                else SpmmFastKernel<ValT, OutT, false, kLanes><<<grid, kThreads, 0, st>>>(a);
                b200sp_note_launches(1);
            };
            switch (lanes_) {
                case 1: launch.template operator()<1>(); break;
                case 2: launch.template operator()<2>(); break;
                case 4: launch.template operator()<4>(); break;
                case 8: launch.template operator()<8>(); break;
                case 16: launch.template operator()<16>(); break;
                default: launch.template operator()<32>(); break;
            }
        };
        auto launchBlocks = [&](cudaStream_t st) {
            const long long want = (blockUnits + kWarps - 1) / kWarps;
            const long long fixed = B200SP_SPMM_BLOCK_CTAS > 0 ? (long long)b200sp_sm_count() * B200SP_SPMM_BLOCK_CTAS : want;
            SpmmLongBlockKernel<ValT, OutT><<<(unsigned)(want < fixed ? want : fixed), kThreads, 0, st>>>(a, ba);
            b200sp_note_launches(1);
        };
        if (lanes != nullptr) {
            if (byBlocks) launchBlocks(segStream);
            else launchFast((unsigned)segments, segStream);
            if (cudaGetLastError() != cudaSuccess || cudaEventRecord(lanes->join[0], segStream) != cudaSuccess)
                return (int)cudaErrorLaunchFailure;
        } else if (byBlocks) {
            launchBlocks(stream);
            if (cudaGetLastError() != cudaSuccess) return (int)cudaErrorLaunchFailure;
        }
        if (stream_) {
            StreamArgs<ValT, OutT> sa;
            sa.rowPtr = rowPtr;
            sa.colInd = colInd;
            sa.val = a.val;
            sa.B = a.B;
            sa.C = a.C;
            sa.m = a.m;
            sa.ldb = sh->ldb;
            sa.ldc = sh->ldc;
            sa.sc = a.sc;
            sa.waitCycles = gHostStreamWaitCycles;
            sa.extraTx = gHostStreamExtraTx;
            const int rc = rowBytes == 512 ? LaunchRowStream<ValT, OutT, 512>(sa, stream)
                                           : LaunchRowStream<ValT, OutT, 1024>(sa, stream);
            if (rc != 0) return rc;
        }
        // What is left for SpmmFastKernel on the caller's stream: the segment CTAs unless they were forked (or
        // replaced by the column-block kernel), and the rows of up to kLongRow entries unless the row-stream
        // kernel took them.
        const long long blocks = (lanes != nullptr ? 0 : (long long)segments) +
                                 (stream_ ? 0 : (sh->m + rowsPerBlock - 1) / rowsPerBlock);
        if (lanes != nullptr && !stream_) a.nsegs = 0;  // the forked launch had them; these CTAs are all row CTAs
        if (blocks > 0) {
            launchFast((unsigned)blocks, stream);
            if (cudaGetLastError() != cudaSuccess) return (int)cudaErrorLaunchFailure;
        }
        if (lanes != nullptr)  // the long rows are already running beside: join them
            return (int)cudaStreamWaitEvent(stream, lanes->join[0], 0);
        return 0;
    }
    GenericShape g{sh->m, sh->n, sh->ldb, sh->ldc, sh->order_b == 0, sh->order_c == 0, sh->op_b, sh->kahan};
    const long long total = sh->m * sh->n;
    if (total == 0) return 0;
    const long long want = (total + 255) / 256;
    const long long cap = (long long)b200sp_sm_count() * 32;
    SpmmGenericFloatKernel<ValT, OutT><<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(
        rowPtr, colInd, static_cast<const ValT *>(val), static_cast<const ValT *>(B), static_cast<OutT *>(C), g,
        MakeF(s));
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int b200sp_spmm_stream_error(void)
{
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, gStreamError, sizeof(flag)) != cudaSuccess) return -1;
    return flag;
}

int b200sp_spmm_stream_error_clear(void)
{
    const int zero = 0;
    return (int)cudaMemcpyToSymbol(gStreamError, &zero, sizeof(zero));
}

void b200sp_spmm_stream_wait_test(long long wait_cycles, unsigned extra_tx)
{
    gHostStreamWaitCycles = wait_cycles > 0 ? wait_cycles : kStreamWaitCycles;
    gHostStreamExtraTx = extra_tx;
}

size_t b200sp_spmm_plan_bytes(int64_t rows, int64_t nnz, int64_t n) { return LayoutFor(rows, nnz, n).total; }

int b200sp_spmm_analyze(const int32_t *row_ptr, int64_t rows, int64_t nnz, int64_t n, void *plan,
                        size_t plan_bytes, int32_t *segments, void *stream)
{
    const PlanLayout L = LayoutFor(rows, nnz, n);
    if (plan == nullptr || segments == nullptr || plan_bytes < L.total) return (int)cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *p = static_cast<char *>(plan);
    cudaError_t e = cudaMemsetAsync(p + L.offCounts, 0, 256, st);
    if (e != cudaSuccess) return (int)e;
    if (rows > 0) {
        const long long want = (rows + 255) / 256;
        const long long cap = (long long)b200sp_sm_count() * 16;
        SpmmFindLongRowsKernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
            row_ptr, (int)rows, reinterpret_cast<int32_t *>(p + L.offCounts),
            reinterpret_cast<LongRow *>(p + L.offLong), reinterpret_cast<SegEntry *>(p + L.offSegs),
            reinterpret_cast<int32_t *>(p + L.offCounters));
        b200sp_note_launches(1);
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    int32_t counts[2] = {0, 0};
    e = cudaMemcpyAsync(counts, p + L.offCounts, sizeof(counts), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    *segments = counts[1];
    return 0;
}

int b200sp_spmm_analyze_blocks(const int32_t *row_ptr, const int32_t *col_ind, int64_t rows, int64_t cols,
                               int64_t nnz, int64_t n, int64_t b_row_bytes, void *plan, size_t plan_bytes,
                               int32_t *block_units, int32_t *long_rows, void *stream)
{
    const PlanLayout L = LayoutFor(rows, nnz, n);
    if (plan == nullptr || block_units == nullptr || long_rows == nullptr || plan_bytes < L.total)
        return (int)cudaErrorInvalidValue;
    *block_units = 0;
    *long_rows = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *p = static_cast<char *>(plan);
    // counts: long rows, segments, partial slots of the segments, "a long row's columns do not ascend", units
    int32_t counts[5] = {0, 0, 0, 0, 0};
    cudaError_t e = cudaMemcpyAsync(counts, p + L.offCounts, sizeof(counts), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    const int nLong = counts[0];
    *long_rows = nLong;
    if (nLong <= 0 || col_ind == nullptr || L.capBlockSlots == 0 || b_row_bytes < kBlockMinRowBytes ||
        cols * b_row_bytes < kBlockMinB)
        return 0;
    long long blocks = (cols * b_row_bytes + kBlockBytes - 1) / kBlockBytes;
    if (blocks > kMaxBlocks) blocks = kMaxBlocks;
    if (blocks < 2) return 0;
    const long long blockCols = (cols + blocks - 1) / blocks;
    int32_t *countsDev = reinterpret_cast<int32_t *>(p + L.offCounts);
    int32_t *meta = reinterpret_cast<int32_t *>(p + L.offBlockMeta);
    int2 *rowSlots = reinterpret_cast<int2 *>(p + L.offRowSlots);
    int32_t *cuts = reinterpret_cast<int32_t *>(p + L.offCuts);
    e = cudaMemsetAsync(meta, 0, sizeof(int32_t) * 3 * kMaxBlocks, st);
    if (e != cudaSuccess) return (int)e;
    SpmmCutBlocksKernel<<<(unsigned)((nLong + 7) / 8), 256, 0, st>>>(
        row_ptr, col_ind, reinterpret_cast<const LongRow *>(p + L.offLong), nLong, blockCols, (int)blocks, cuts,
        rowSlots, reinterpret_cast<int32_t *>(p + L.offBlockCounters), meta, countsDev + 3);
    SpmmBlockScanKernel<<<1, 1024, 0, st>>>(rowSlots, nLong, meta, (int)blocks, countsDev + 4);
    SpmmFillUnitsKernel<<<(unsigned)((nLong + 7) / 8), 256, 0, st>>>(
        cuts, rowSlots, nLong, (int)blocks, meta, reinterpret_cast<BlockUnit *>(p + L.offUnits),
        (int)(L.capBlockSlots < INT32_MAX ? L.capBlockSlots : INT32_MAX));
    b200sp_note_launches(3);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(counts, countsDev, sizeof(counts), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    // Unsorted long rows, or more units than the plan has partial rows for: the segments stay in charge.
    if (counts[3] == 0 && counts[4] > 0 && counts[4] <= L.capBlockSlots) *block_units = counts[4];
    return 0;
}

int b200sp_spmm_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *B, void *C,
                       const b200spSpmmShape *shape, const b200spScalars *scalars, int val_type, int out_type,
                       void *plan, int32_t segments, void *stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (val_type == B200SP_F32 && out_type == B200SP_F32)
        return LaunchFloat<float, float>(row_ptr, col_ind, val, B, C, shape, scalars, plan, segments, st);
    if (val_type == B200SP_F16 && out_type == B200SP_F16)
        return LaunchFloat<__half, __half>(row_ptr, col_ind, val, B, C, shape, scalars, plan, segments, st);
    if (val_type == B200SP_BF16 && out_type == B200SP_BF16)
        return LaunchFloat<__nv_bfloat16, __nv_bfloat16>(row_ptr, col_ind, val, B, C, shape, scalars, plan,
                                                         segments, st);
    if (val_type == B200SP_BF16 && out_type == B200SP_F32)
        return LaunchFloat<__nv_bfloat16, float>(row_ptr, col_ind, val, B, C, shape, scalars, plan, segments, st);
    if (val_type == B200SP_I8 && out_type == B200SP_I32) {
        GenericShape g{shape->m, shape->n, shape->ldb, shape->ldc, shape->order_b == 0, shape->order_c == 0,
                       shape->op_b, 0};
        const long long total = shape->m * shape->n;
        if (total == 0) return 0;
        const long long want = (total + 255) / 256;
        const long long cap = (long long)b200sp_sm_count() * 32;
        SpmmGenericInt8Kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
            row_ptr, col_ind, static_cast<const int8_t *>(val), static_cast<const int8_t *>(B),
            static_cast<int32_t *>(C), g, MakeI(scalars));
        b200sp_note_launches(1);
        return (int)cudaGetLastError();
    }
    return (int)cudaErrorInvalidValue;
}

}  // extern "C"
