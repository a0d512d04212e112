// Segmented sort of 64-bit keys, shared by aclsparseXcsrsort and aclsparseCsr2cscEx2.
//
// The reference ships device sorts of its own for both operators (sparse/csrsort/arch35/csrsort_host.cpp:146-222,
// sparse/csr2csc_ex2/arch35/csr2csc_ex2_host.cpp:539-640); these are the B200 ones.  Both callers make every key
// unique by packing what must be ordered into the high word and a tie-breaker into the low word
// (csrsort: column | position in the row; csr2csc: entry index | row), so any correct sort gives the stable
// order the goldens define, and one routine serves both:
//   segments of up to 32 keys    a warp per segment, a bitonic network over registers (shuffles);
//   up to kSegChunk keys         a CTA per segment, a bitonic network in shared memory;
//   longer                       the same CTA sorts the segment chunk by chunk, then merges the sorted runs
//                                pairwise (merge path: every thread finds its slice of the output by a binary
//                                search on a diagonal, then merges it sequentially), ping-ponging between the data
//                                and a scratch array until one run is left.
// Nothing synchronises with the host: the first kernel appends the segments that are too long for a warp to a
// list in the workspace and the second walks that list with a fixed grid.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"

namespace b200sp_segsort {

constexpr int kSegChunk = 2048;           // keys a CTA sorts in shared memory at once
constexpr int kSegThreads = 256;
constexpr unsigned long long kSentinel = ~0ull;  // sorts after every real key

// offsets[s] - base .. offsets[s + 1] - base delimit segment s in `data`.
static __global__ void __launch_bounds__(256) SegSortShortKernel(const int *__restrict__ offsets, int base, int segments,
                                                          unsigned long long *__restrict__ data,
                                                          int *__restrict__ longList)
{
    const int lane = threadIdx.x & 31;
    const long long warpsTotal = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long s = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s < segments; s += warpsTotal) {
        const int a = offsets[s] - base, b = offsets[s + 1] - base;
        const int len = b - a;
        if (len <= 1) continue;
        if (len > 32) {
            if (lane == 0) longList[1 + atomicAdd(longList, 1)] = (int)s;
            continue;
        }
        unsigned long long v = lane < len ? data[a + lane] : kSentinel;
#pragma unroll
        for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
            for (int j = k >> 1; j > 0; j >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, j);
                const bool up = (lane & k) == 0;      // this run of k lanes ascends
                const bool lower = (lane & j) == 0;   // this lane is the lower partner
                const bool takeMin = lower == up;
                v = takeMin ? (v < other ? v : other) : (v > other ? v : other);
            }
        }
        if (lane < len) data[a + lane] = v;
    }
}

// Bitonic sort of s[0 .. P) (P a power of two >= 2), ascending; all threads of the CTA call it.
__device__ __forceinline__ void BitonicShared(unsigned long long *s, int P)
{
    for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (P >> 1); t += kSegThreads) {
                const int i = ((t / j) * (j << 1)) + (t % j);
                const int p = i + j;
                const bool up = (i & k) == 0;
                const unsigned long long x = s[i], y = s[p];
                if ((x > y) == up) {
                    s[i] = y;
                    s[p] = x;
                }
            }
            __syncthreads();
        }
    }
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
    // merge path: the first d0 outputs take ai keys of A and d0 - ai of B
    int l = d0 - nb > 0 ? d0 - nb : 0, h = d0 < na ? d0 : na;
    while (l < h) {
        const int m = (l + h) >> 1;
        if (A[m] < B[d0 - m - 1]) l = m + 1;  // keys are unique: no ties to break
        else h = m;
    }
    int ai = l, bi = d0 - l;
    for (int o = d0; o < d1; ++o) {
        const bool takeA = bi >= nb || (ai < na && A[ai] < B[bi]);
        dst[lo + o] = takeA ? A[ai++] : B[bi++];
    }
}

static __global__ void __launch_bounds__(kSegThreads) SegSortLongKernel(const int *__restrict__ offsets, int base,
                                                                 unsigned long long *__restrict__ data,
                                                                 unsigned long long *__restrict__ scratch,
                                                                 const int *__restrict__ longList)
{
    __shared__ unsigned long long s[kSegChunk];
    const int count = longList[0];
    for (int li = blockIdx.x; li < count; li += gridDim.x) {
        const int seg = longList[1 + li];
        const int a = offsets[seg] - base, b = offsets[seg + 1] - base;
        const int len = b - a;
        for (int c0 = 0; c0 < len; c0 += kSegChunk) {
            const int n = len - c0 < kSegChunk ? len - c0 : kSegChunk;
            int P = 64;
            while (P < n) P <<= 1;
            for (int i = threadIdx.x; i < P; i += kSegThreads) s[i] = i < n ? data[a + c0 + i] : kSentinel;
            __syncthreads();
            BitonicShared(s, P);
            for (int i = threadIdx.x; i < n; i += kSegThreads) data[a + c0 + i] = s[i];
            __syncthreads();
        }
        if (len <= kSegChunk) continue;
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
        if (src != data)
            for (int i = threadIdx.x; i < len; i += kSegThreads) data[a + i] = scratch[a + i];
        __syncthreads();
    }
}

// Workspace for the list of long segments (count + one entry per segment).
inline size_t ListBytes(long long segments) { return (sizeof(int) * (size_t)(segments + 1) + 255) / 256 * 256; }

// Sorts every segment of `data` in place.  `longList` must hold ListBytes(segments) bytes; `scratch` as many keys as
// `data`.  Returns the cudaError_t of the launches.
inline cudaError_t Sort(const int *offsets, int base, int segments, unsigned long long *data, unsigned long long *scratch,
                        int *longList, cudaStream_t stream)
{
    if (segments <= 0) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(longList, 0, sizeof(int), stream);
    if (e != cudaSuccess) return e;
    const long long want = ((long long)segments + 7) / 8;
    const long long cap = (long long)b200sp_sm_count() * 32;
    SegSortShortKernel<<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(offsets, base, segments, data, longList);
    SegSortLongKernel<<<(unsigned)(b200sp_sm_count() * 6), kSegThreads, 0, stream>>>(offsets, base, data, scratch, longList);
    b200sp_note_launches(2);
    return cudaGetLastError();
}

}  // namespace b200sp_segsort
