// Segmented sort of 64-bit keys, shared by aclsparseXcsrsort and aclsparseCsr2cscEx2.
//
// The reference ships device sorts of its own for both operators (sparse/csrsort/arch35/csrsort_host.cpp:146-222,
// sparse/csr2csc_ex2/arch35/csr2csc_ex2_host.cpp:539-640); these are the B200 ones.  Both callers make every key
// unique by packing what must be ordered into the high word and a tie-breaker into the low word
// (csrsort: column | position in the row; csr2csc: entry index | row), so any correct sort gives the stable
// order the goldens define, and one routine serves both:
//   segments of up to 256 keys   a warp per segment; every lane holds 1, 2, 4 or 8 keys in registers and the
//                                bitonic network runs over shuffles (partners in other lanes) and register pairs
//                                (partners in the same lane): no shared memory, no barrier;
//   up to kSegChunk = 2048 keys  a CTA per segment: its eight warps sort 256 keys each as above, then three
//                                merge rounds in shared memory (merge path: every thread finds its eight outputs
//                                by a binary search on a diagonal and merges them sequentially);
//   longer                       the same CTA sorts the segment chunk by chunk into the key array, then merges the
//                                sorted runs pairwise between the key array and a scratch array until one is left.
// The callers' own passes are folded into the sort through an `Io` policy: keys are formed while they are loaded
// (`Load(a, i)`: element i of the segment that starts at a) and split into the callers' outputs while they are
// stored (`Fetch(a, key)` reads what the stored element needs, for all elements of the segment, before
// `Commit(a, i, key, payload)` writes any of them, so a caller may sort in place; `Pack` / `Unpack` squeeze a
// payload into 32 bits for segments that park it in global memory).
// Nothing synchronises with the host: the first kernel appends the segments that are too long for a warp to a
// list in the workspace (those of more than kSegChunk keys at its far end) and the CTAs of the second take
// them from a shared cursor, the longest kind first, so that no CTA is left alone with several long segments.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"

namespace b200sp_segsort {

constexpr int kWarpMax = 256;             // keys a warp sorts in registers (8 per lane)
constexpr int kSegChunk = 2048;           // keys a CTA sorts in shared memory at once
constexpr int kSegThreads = 256;
constexpr int kPerThread = kSegChunk / kSegThreads;
constexpr unsigned long long kSentinel = ~0ull;  // sorts after every real key
// The list of segments too long for a warp: [0] segments of up to kSegChunk keys (entries from kListHead upwards),
// [1] longer ones (entries from the end of the list downwards), [2] the cursor the CTAs take work from.
constexpr int kListHead = 4;

// Bitonic sort of 32 * E keys held by one warp, element i = r * 32 + lane in v[r]; ascending in i.
template <int E>
__device__ __forceinline__ void WarpSort(unsigned long long (&v)[E], int lane)
{
#pragma unroll
    for (int k = 2; k <= 32 * E; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j >= 32) {  // partner in the same lane: registers r and r | (j / 32)
                const int jr = j >> 5;
#pragma unroll
                for (int r = 0; r < E; ++r) {
                    if ((r & jr) != 0) continue;
                    const bool up = ((r << 5) & k) == 0;  // k >= 64: decided by the register index alone
                    const unsigned long long x = v[r], y = v[r | jr];
                    const bool swap = (x > y) == up;
                    v[r] = swap ? y : x;
                    v[r | jr] = swap ? x : y;
                }
            } else {  // partner in lane ^ j, same register
#pragma unroll
                for (int r = 0; r < E; ++r) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v[r], j);
                    const bool up = (((r << 5) | lane) & k) == 0;
                    const bool lower = (lane & j) == 0;
                    const bool takeMin = lower == up;
                    v[r] = takeMin ? (v[r] < other ? v[r] : other) : (v[r] > other ? v[r] : other);
                }
            }
        }
    }
}

// One segment of up to 32 * E keys, by one warp, from load to store.
template <int E, class Io>
__device__ __forceinline__ void WarpSegment(const Io &io, int a, int len, int lane)
{
    unsigned long long v[E];
#pragma unroll
    for (int r = 0; r < E; ++r) {
        const int i = r * 32 + lane;
        v[r] = i < len ? io.Load(a, i) : kSentinel;
    }
    WarpSort<E>(v, lane);
    typename Io::Payload pay[E];
#pragma unroll
    for (int r = 0; r < E; ++r) {
        const int i = r * 32 + lane;
        pay[r] = i < len ? io.Fetch(a, v[r]) : typename Io::Payload{};
    }
    __syncwarp();  // orders every lane's fetches before any lane's commits (the caller may sort in place)
#pragma unroll
    for (int r = 0; r < E; ++r) {
        const int i = r * 32 + lane;
        if (i < len) io.Commit(a, i, v[r], pay[r]);
    }
}

// offsets[s] - base .. offsets[s + 1] - base delimit segment s.
template <class Io>
static __global__ void __launch_bounds__(256) SegSortWarpKernel(const int *__restrict__ offsets, int base, int segments,
                                                                Io io, int *__restrict__ longList)
{
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long s = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s < segments; s += warpsTotal) {
        const int a = offsets[s] - base;
        const int len = offsets[s + 1] - base - a;
        if (len <= 0) continue;
        if (len > kWarpMax) {
            if (lane == 0) {
                if (len > kSegChunk) longList[kListHead + segments - 1 - atomicAdd(longList + 1, 1)] = (int)s;
                else longList[kListHead + atomicAdd(longList, 1)] = (int)s;
            }
        } else if (len <= 32) {
            WarpSegment<1>(io, a, len, lane);  // also a single key: the caller's split must still happen
        } else if (len <= 64) {
            WarpSegment<2>(io, a, len, lane);
        } else if (len <= 128) {
            WarpSegment<4>(io, a, len, lane);
        } else {
            WarpSegment<8>(io, a, len, lane);
        }
    }
}

// The first d outputs of the merge of the sorted runs A[0, na) and B[0, nb) take `ai` keys of A: returns ai.
__device__ __forceinline__ int MergePathSplit(const unsigned long long *A, int na, const unsigned long long *B, int nb, int d)
{
    int l = d - nb > 0 ? d - nb : 0, h = d < na ? d : na;
    while (l < h) {
        const int m = (l + h) >> 1;
        if (A[m] < B[d - m - 1]) l = m + 1;  // real keys are unique; sentinels may tie, in any order
        else h = m;
    }
    return l;
}

// Merges the sorted runs src[lo, mid) and src[mid, hi) into dst[lo, hi); all threads of the CTA call it.
__device__ __forceinline__ void MergeRuns(const unsigned long long *__restrict__ src, unsigned long long *__restrict__ dst,
                                          int lo, int mid, int hi)
{
    const int na = mid - lo, nb = hi - mid, n = na + nb;
    const int per = (n + kSegThreads - 1) / kSegThreads;
    const int d0 = (int)threadIdx.x * per < n ? (int)threadIdx.x * per : n;
    const int d1 = d0 + per < n ? d0 + per : n;
    if (d0 >= d1) return;
    const unsigned long long *A = src + lo, *B = src + mid;
    int ai = MergePathSplit(A, na, B, nb, d0), bi = d0 - ai;
    for (int o = d0; o < d1; ++o) {
        const bool takeA = bi >= nb || (ai < na && A[ai] < B[bi]);
        dst[lo + o] = takeA ? A[ai++] : B[bi++];
    }
}

// Sorts n <= kSegChunk keys by the whole CTA: keys come from load(i), the sorted keys end up in the returned
// shared-memory buffer (one of s0 / s1), padded with sentinels up to kSegChunk.
template <class LoadFn>
__device__ __forceinline__ unsigned long long *ChunkSort(unsigned long long *s0, unsigned long long *s1, int n, LoadFn load)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        unsigned long long v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int i = warp * kWarpMax + r * 32 + lane;
            v[r] = i < n ? load(i) : kSentinel;
        }
        if (warp * kWarpMax < n) WarpSort<8>(v, lane);  // a run of sentinels alone is sorted already
#pragma unroll
        for (int r = 0; r < 8; ++r) s0[warp * kWarpMax + r * 32 + lane] = v[r];
    }
    __syncthreads();
    unsigned long long *src = s0, *dst = s1;
    for (int width = kWarpMax; width < kSegChunk && width < n; width <<= 1) {
        // thread t writes outputs [t * 8, t * 8 + 8): they lie inside one pair of runs
        const int o0 = (int)threadIdx.x * kPerThread;
        const int lo = o0 / (2 * width) * (2 * width);
        const unsigned long long *A = src + lo, *B = src + lo + width;
        const int d0 = o0 - lo;
        int ai = MergePathSplit(A, width, B, width, d0), bi = d0 - ai;
#pragma unroll
        for (int o = 0; o < kPerThread; ++o) {
            const bool takeA = bi >= width || (ai < width && A[ai] < B[bi]);
            dst[o0 + o] = takeA ? A[ai++] : B[bi++];
        }
        __syncthreads();
        unsigned long long *t = src;
        src = dst;
        dst = t;
    }
    // Runs beyond the last merged width hold sentinels only (width >= n), so src[0, n) is the sorted segment.
    return src;
}

template <class Io>
static __global__ void __launch_bounds__(kSegThreads) SegSortCtaKernel(const int *__restrict__ offsets, int base,
                                                                       int segments, Io io,
                                                                       unsigned long long *__restrict__ data,
                                                                       unsigned long long *__restrict__ scratch,
                                                                       int *longList)
{
    __shared__ unsigned long long s0[kSegChunk];
    __shared__ unsigned long long s1[kSegChunk];
    __shared__ int sTake;
    const int medium = longList[0], big = longList[1];
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) sTake = atomicAdd(longList + 2, 1);
        __syncthreads();
        const int li = sTake;
        if (li >= medium + big) break;
        const int seg = li < big ? longList[kListHead + segments - 1 - li] : longList[kListHead + li - big];
        const int a = offsets[seg] - base;
        const int len = offsets[seg + 1] - base - a;
        if (len <= kSegChunk) {
            const unsigned long long *sorted = ChunkSort(s0, s1, len, [&](int i) { return io.Load(a, i); });
            unsigned long long key[kPerThread];
            typename Io::Payload pay[kPerThread];
#pragma unroll
            for (int o = 0; o < kPerThread; ++o) {
                const int i = o * kSegThreads + (int)threadIdx.x;
                key[o] = i < len ? sorted[i] : kSentinel;
                pay[o] = i < len ? io.Fetch(a, key[o]) : typename Io::Payload{};
            }
            __syncthreads();  // all fetches of the segment (and all reads of the shared buffers) are done
#pragma unroll
            for (int o = 0; o < kPerThread; ++o) {
                const int i = o * kSegThreads + (int)threadIdx.x;
                if (i < len) io.Commit(a, i, key[o], pay[o]);
            }
            __syncthreads();
            continue;
        }
        // Longer than a chunk: sorted chunks go to the key array, then pairwise merges between it and the scratch.
        for (int c0 = 0; c0 < len; c0 += kSegChunk) {
            const int n = len - c0 < kSegChunk ? len - c0 : kSegChunk;
            const unsigned long long *sorted = ChunkSort(s0, s1, n, [&](int i) { return io.Load(a, c0 + i); });
            for (int i = threadIdx.x; i < n; i += kSegThreads) data[a + c0 + i] = sorted[i];
            __syncthreads();
        }
        unsigned long long *src = data, *dst = scratch;
        for (int width = kSegChunk; width < len; width <<= 1) {
            __threadfence_block();
            __syncthreads();  // the previous pass (or the chunk sorts) are complete and visible to the whole CTA
            for (int lo = 0; lo < len; lo += 2 * width) {
                const int mid = lo + width < len ? lo + width : len;
                const int hi = lo + 2 * width < len ? lo + 2 * width : len;
                if (mid < hi) MergeRuns(src, dst, a + lo, a + mid, a + hi);
                else
                    for (int i = lo + threadIdx.x; i < hi; i += kSegThreads) dst[a + i] = src[a + i];  // an odd run out
            }
            unsigned long long *t = src;
            src = dst;
            dst = t;
        }
        __threadfence_block();
        __syncthreads();
        // Split the sorted keys into the caller's outputs, a chunk at a time: what Commit needs is fetched for the
        // whole segment first and parked in the array the sorted keys are NOT in (4 bytes per element).
        unsigned *park = reinterpret_cast<unsigned *>((src == data ? scratch : data) + a);
        for (int i = threadIdx.x; i < len; i += kSegThreads) park[i] = Io::Pack(io.Fetch(a, src[a + i]));
        __threadfence_block();
        __syncthreads();
        for (int i = threadIdx.x; i < len; i += kSegThreads) io.Commit(a, i, src[a + i], Io::Unpack(park[i]));
        __syncthreads();
    }
}

// Workspace for the list of long segments (counters + one entry per segment).
inline size_t ListBytes(long long segments) { return (sizeof(int) * (size_t)(segments + kListHead) + 255) / 256 * 256; }

// Sorts every segment.  `longList` must hold ListBytes(segments) bytes; `data` and `scratch` as many keys as all
// segments together (they are touched only for segments of more than kSegChunk keys, unless Io loads from them).
// Returns the cudaError_t of the launches.
template <class Io>
inline cudaError_t Sort(const int *offsets, int base, int segments, const Io &io, unsigned long long *data,
                        unsigned long long *scratch, int *longList, cudaStream_t stream)
{
    if (segments <= 0) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(longList, 0, sizeof(int) * kListHead, stream);
    if (e != cudaSuccess) return e;
    const long long want = ((long long)segments + 7) / 8;
    const long long cap = (long long)b200sp_sm_count() * 32;
    SegSortWarpKernel<Io><<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(offsets, base, segments, io, longList);
    SegSortCtaKernel<Io><<<(unsigned)(b200sp_sm_count() * 6), kSegThreads, 0, stream>>>(offsets, base, segments, io, data,
                                                                                       scratch, longList);
    b200sp_note_launches(2);
    return cudaGetLastError();
}

}  // namespace b200sp_segsort
