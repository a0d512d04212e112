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
//   up to kSegChunk = 2048 keys  a CTA per segment: a stable radix sort on the high word, 8 bits per pass, as many
//                                passes as the segment's largest high word has bytes, between two shared-memory
//                                buffers (the low word needs no pass: the keys arrive ordered by it, or the high
//                                words are unique);
//   longer                       the same passes between the key array and a scratch array in global memory.
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

constexpr int kRadixBits = 8;
constexpr int kBins = 1 << kRadixBits;
constexpr int kCtaWarps = kSegThreads / 32;
static_assert(kBins == kSegThreads, "the scan below gives every thread one bin");

// One stable pass of a CTA-wide least-significant-digit radix sort: n keys in their current order load(0 .. n)
// go to store(position, key), ordered by bits [shift, shift + 8) and, among equal digits, by current order.
// Every warp owns a contiguous slice of the current order; after a histogram per warp and one scan over
// (digit, warp), a warp walks its slice 32 keys at a time and ranks equal digits by lane with match.any:
// no barrier and no counter reset inside the walk.  sHist holds kBins * kCtaWarps counters, sPart kCtaWarps.
template <class LoadFn, class StoreFn>
__device__ __forceinline__ void RadixPass(int n, int shift, int *sHist, int *sPart, LoadFn load, StoreFn store)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = ((n + kCtaWarps - 1) / kCtaWarps + 31) & ~31;
    const int w0 = warp * per < n ? warp * per : n;
    const int w1 = w0 + per < n ? w0 + per : n;
    for (int i = threadIdx.x; i < kBins * kCtaWarps; i += kSegThreads) sHist[i] = 0;
    __syncthreads();
    for (int i = w0 + lane; i < w1; i += 4 * 32) {  // four loads in flight per lane
        unsigned long long k[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) k[u] = i + 32 * u < w1 ? load(i + 32 * u) : 0ull;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + 32 * u < w1) atomicAdd(&sHist[warp * kBins + ((unsigned)(k[u] >> shift) & (kBins - 1))], 1);
    }
    __syncthreads();
    {  // exclusive scan over (digit, warp): thread t owns digit t
        int c[kCtaWarps], tot = 0;
#pragma unroll
        for (int w = 0; w < kCtaWarps; ++w) {
            c[w] = sHist[w * kBins + threadIdx.x];
            tot += c[w];
        }
        int incl = tot;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += t;
        }
        if (lane == 31) sPart[warp] = incl;
        __syncthreads();
        int before = incl - tot;
        for (int w = 0; w < warp; ++w) before += sPart[w];
#pragma unroll
        for (int w = 0; w < kCtaWarps; ++w) {
            sHist[w * kBins + threadIdx.x] = before;
            before += c[w];
        }
    }
    __syncthreads();
    unsigned long long ahead = w0 + lane < w1 ? load(w0 + lane) : 0ull;  // the next step's key is requested a step early
    for (int i0 = w0; i0 < w1; i0 += 32) {
        const int i = i0 + lane;
        const bool live = i < w1;
        const unsigned long long key = ahead;
        ahead = i + 32 < w1 ? load(i + 32) : 0ull;
        const unsigned d = live ? ((unsigned)(key >> shift) & (kBins - 1)) : (unsigned)kBins;  // idle lanes: a group apart
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        int pos = 0;
        if (live) pos = sHist[warp * kBins + d] + rank;
        __syncwarp();
        if (live && rank == 0) sHist[warp * kBins + d] += __popc(peers);  // the lowest lane of every group
        __syncwarp();
        if (live) store(pos, key);
    }
    __syncthreads();
}

// Passes needed for the high words of a segment's keys: the CTA ORs them together and counts the bytes in use.
template <class LoadFn>
__device__ __forceinline__ int RadixPasses(int n, int *sWord, LoadFn load)
{
    if (threadIdx.x == 0) *sWord = 0;
    __syncthreads();
    unsigned seen = 0;
    for (int i = threadIdx.x; i < n; i += kSegThreads) seen |= (unsigned)(load(i) >> 32);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) seen |= __shfl_xor_sync(0xffffffffu, seen, off);
    if ((threadIdx.x & 31) == 0 && seen != 0) atomicOr(sWord, (int)seen);
    __syncthreads();
    const unsigned all = (unsigned)*sWord;
    __syncthreads();
    const int bits = all == 0 ? 1 : 32 - __clz(all);
    return (bits + kRadixBits - 1) / kRadixBits;
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
    __shared__ int sHist[kBins * kCtaWarps];
    __shared__ int sPart[kCtaWarps];
    __shared__ int sTake, sWord;
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
        auto fromCaller = [&](int i) { return io.Load(a, i); };
        const int passes = RadixPasses(len, &sWord, fromCaller);
        if (len <= kSegChunk) {  // between two shared-memory buffers
            unsigned long long *src = s1, *dst = s0;
            for (int p = 0; p < passes; ++p) {
                const int shift = 32 + kRadixBits * p;
                unsigned long long *to = dst;
                if (p == 0) {
                    RadixPass(len, shift, sHist, sPart, fromCaller, [&](int j, unsigned long long k) { to[j] = k; });
                } else {
                    const unsigned long long *from = src;
                    RadixPass(len, shift, sHist, sPart, [&](int i) { return from[i]; },
                              [&](int j, unsigned long long k) { to[j] = k; });
                }
                unsigned long long *t = src;
                src = dst;
                dst = t;
            }
            const unsigned long long *sorted = src;
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
            continue;
        }
        // Longer than a chunk: between the scratch array and the key array in global memory (the first pass writes
        // the scratch array: a caller may keep its unsorted keys in the key array).
        unsigned long long *src = data, *dst = scratch;
        for (int p = 0; p < passes; ++p) {
            const int shift = 32 + kRadixBits * p;
            unsigned long long *to = dst + a;
            if (p == 0) {
                RadixPass(len, shift, sHist, sPart, fromCaller, [&](int j, unsigned long long k) { to[j] = k; });
            } else {
                const unsigned long long *from = src + a;
                RadixPass(len, shift, sHist, sPart, [&](int i) { return from[i]; },
                          [&](int j, unsigned long long k) { to[j] = k; });
            }
            unsigned long long *t = src;
            src = dst;
            dst = t;
        }
        // Split the sorted keys into the caller's outputs: what Commit needs is fetched for the whole segment
        // first and parked in the array the sorted keys are NOT in (4 bytes per element).
        unsigned *park = reinterpret_cast<unsigned *>(dst + a);
        for (int i = threadIdx.x; i < len; i += kSegThreads) park[i] = Io::Pack(io.Fetch(a, src[a + i]));
        __syncthreads();
        for (int i = threadIdx.x; i < len; i += kSegThreads) io.Commit(a, i, src[a + i], Io::Unpack(park[i]));
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
