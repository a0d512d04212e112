// A side stream per host thread and device, for products that run two grids side by side.
//
// A product that launches two kernels over disjoint outputs forks the smaller one onto this stream
// (event recorded on the caller's stream, waited on here) and joins it back (event recorded here,
// waited on by the caller's stream), so that both share the SMs and the caller still sees one
// stream-ordered operation.  Created at first use, destroyed with the thread; holds no device memory.
// Per thread, because an event recorded by one caller must not be waited on by another caller's
// side stream.
#pragma once

#include <cuda_runtime_api.h>

namespace b200sp {

constexpr int kMaxDevices = 64;

struct SideLanes {
    cudaStream_t stream[1] = {nullptr};
    cudaEvent_t fork = nullptr;
    cudaEvent_t join[1] = {nullptr};
    bool ready = false;
};

struct SideLaneSet {
    SideLanes lanes[kMaxDevices];
    ~SideLaneSet()
    {
        int prev = 0;
        const bool havePrev = cudaGetDevice(&prev) == cudaSuccess;
        for (int d = 0; d < kMaxDevices; ++d) {
            SideLanes &l = lanes[d];
            if (!l.ready) continue;
            if (cudaSetDevice(d) != cudaSuccess) continue;
            if (l.stream[0] != nullptr) (void)cudaStreamDestroy(l.stream[0]);  // runs what is queued, then frees
            if (l.join[0] != nullptr) (void)cudaEventDestroy(l.join[0]);
            if (l.fork != nullptr) (void)cudaEventDestroy(l.fork);
        }
        if (havePrev) (void)cudaSetDevice(prev);
        (void)cudaGetLastError();
    }
};

// The side stream gets the highest priority the device offers: its grid is the small one that should be
// resident first, and (B200SP_SIDE_PRIORITY = 0 restores the default) a priority of its own keeps it
// off the hardware queue of the caller's stream.
#ifndef B200SP_SIDE_PRIORITY
#define B200SP_SIDE_PRIORITY 1
#endif
inline cudaError_t CreateSideStream(cudaStream_t *s)
{
#if B200SP_SIDE_PRIORITY
    int least = 0, greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) == cudaSuccess && greatest < least)
        return cudaStreamCreateWithPriority(s, cudaStreamNonBlocking, greatest);
    (void)cudaGetLastError();
#endif
    return cudaStreamCreateWithFlags(s, cudaStreamNonBlocking);
}

// The calling thread's side lanes on the current device, or nullptr when they cannot be created (the caller
// then runs its kernels one after the other on its own stream).
inline SideLanes *GetSideLanes()
{
    static thread_local SideLaneSet set;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    SideLanes &l = set.lanes[dev];
    if (!l.ready) {
        const bool ok = cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) == cudaSuccess &&
                        CreateSideStream(&l.stream[0]) == cudaSuccess &&
                        cudaEventCreateWithFlags(&l.join[0], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            (void)cudaGetLastError();
            return nullptr;
        }
        l.ready = true;
    }
    return &l;
}

}  // namespace b200sp
