// Replication of x (SpMV) or B (SpMM) across the GPUs of one box by peer stores.
//
// The reference is single-device, so nothing here has a counterpart there.  The multi-GPU mode cuts A into row
// blocks, one per rank (one process per GPU); every rank needs all of x / B before its product.  When the operand
// is produced sharded (the y of the previous product in an iterative solver, the C of the previous layer in a
// graph network) the exchange is an all-gather, done here without a library collective: every rank owns a
// cudaMalloc'ed region that holds `replicas` copies of the whole operand plus arrival flags, maps the regions of
// its peers through CUDA IPC, and one kernel per step
//   1. copies the rank's own slice into the same offset of the chosen replica on EVERY rank (plain 16-byte
//      stores through the peer mappings: NVLink carries them, nothing is read remotely),
//   2. lets the last CTA to finish publish the step's sequence number in this rank's flag on every rank
//      (after a system-wide fence, so a peer that sees the flag sees the data),
//   3. and, if asked, has that CTA wait until the flags of the wanted ranks have reached the same number.
// The product that follows in the stream then reads a complete local replica.  With two replicas used in turn a
// rank can never overwrite data a slower peer is still reading: to start step k + 1 a rank must have seen the
// step-k flags of all peers, which a peer raises only after its own product of step k - 1.
// Every wait is bounded (kWaitCycles of the SM clock); a wait that runs out sets an error word the host can read
// and the kernel returns, so a missing peer can never hang the GPU.
// No load with cluster multicast and no library kernel ever touches a peer mapping: only this file's stores do.
#include <cstdint>
#include <cstdio>
#include <new>

#include <cuda_runtime.h>

#include "b200sp_kernels.h"
#include "b200sp_mg.h"

namespace {

constexpr int kMaxRanks = B200SP_MG_MAX_RANKS;
constexpr long long kDefaultWaitCycles = 1ll << 32;  // about two seconds of SM clock: far beyond any healthy step

struct Control {            // at the start of every rank's region
    uint32_t flag[B200SP_MG_MAX_REPLICAS][kMaxRanks];  // flag[r][p]: last sequence number rank p published for replica r
    uint32_t arrived;       // CTAs of the running push kernel that have finished their stores (local use only)
    uint32_t error;         // set when a wait ran out
    uint32_t pad[62];
};
static_assert(sizeof(Control) % 256 == 0, "replicas start 256-byte aligned");

struct PeerTable {
    unsigned char *base[kMaxRanks];  // region of every rank as mapped into this process (own region included)
};

inline size_t AlignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

__device__ __forceinline__ uint32_t LoadFlag(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void StoreFlag(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// grid-stride copy of `bytes` (a multiple of 16, both sides 16-byte aligned) from src to dstOffset of every rank's
// region, then the publish / wait protocol described at the top.
__global__ void __launch_bounds__(256) MgPushKernel(PeerTable peers, int rank, int world, const uint4 *__restrict__ src,
                                                    size_t dstOffset, size_t vecs, int replica, uint32_t seq,
                                                    uint32_t waitMask, long long waitCycles)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        const uint4 v = __ldcs(src + i);
        for (int p = 0; p < world; ++p) reinterpret_cast<uint4 *>(peers.base[p] + dstOffset)[i] = v;
    }
    Control *mine = reinterpret_cast<Control *>(peers.base[rank]);
    __shared__ int sLast;
    __syncthreads();  // every thread of the CTA has issued its stores ...
    if (threadIdx.x == 0) {
        __threadfence_system();  // ... and this fence, ordered after them by the barrier, makes them visible system-wide
        const uint32_t old = atomicAdd(&mine->arrived, 1u);
        sLast = (old == gridDim.x - 1);
        if (sLast) mine->arrived = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sLast) return;
    __threadfence_system();
    if ((int)threadIdx.x < world) {
        Control *theirs = reinterpret_cast<Control *>(peers.base[threadIdx.x]);
        StoreFlag(&theirs->flag[replica][rank], seq);
    }
    if ((int)threadIdx.x < world && ((waitMask >> threadIdx.x) & 1u)) {
        const uint32_t *f = &mine->flag[replica][threadIdx.x];
        const long long t0 = clock64();
        // sequence numbers only grow; the signed difference tolerates their wrap-around
        while ((int32_t)(LoadFlag(f) - seq) < 0) {
            if (clock64() - t0 > waitCycles) {
                atomicExch(&mine->error, 1u);
                break;
            }
        }
    }
    __threadfence_system();
}

// Wait alone (a rank that contributes nothing to a step, e.g. the receivers of a one-to-all replication).
__global__ void MgWaitKernel(PeerTable peers, int rank, int world, int replica, uint32_t seq, uint32_t waitMask,
                             long long waitCycles)
{
    Control *mine = reinterpret_cast<Control *>(peers.base[rank]);
    if ((int)threadIdx.x < world && ((waitMask >> threadIdx.x) & 1u)) {
        const uint32_t *f = &mine->flag[replica][threadIdx.x];
        const long long t0 = clock64();
        while ((int32_t)(LoadFlag(f) - seq) < 0) {
            if (clock64() - t0 > waitCycles) {
                atomicExch(&mine->error, 1u);
                break;
            }
        }
    }
    __threadfence_system();
}

}  // namespace

struct b200spMgExchange {
    int rank = 0, world = 1, replicas = 1, device = 0;
    size_t bytes = 0, replicaStride = 0, regionBytes = 0;
    unsigned char *region = nullptr;       // this rank's allocation
    PeerTable peers{};
    bool opened[kMaxRanks] = {};           // peer mappings this process opened (to close them again)
    bool imported = false;
    long long waitCycles = kDefaultWaitCycles;
};

extern "C" {

int b200spMgExchangeCreate(b200spMgExchange **out, int rank, int world, size_t bytes, int replicas)
{
    if (out == nullptr || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || replicas < 1 ||
        replicas > B200SP_MG_MAX_REPLICAS)
        return (int)cudaErrorInvalidValue;
    auto *ex = new (std::nothrow) b200spMgExchange;
    if (ex == nullptr) return (int)cudaErrorMemoryAllocation;
    ex->rank = rank;
    ex->world = world;
    ex->replicas = replicas;
    ex->bytes = bytes;
    ex->replicaStride = AlignUp(bytes > 0 ? bytes : 16, 256);
    ex->regionBytes = sizeof(Control) + ex->replicaStride * (size_t)replicas;
    cudaError_t e = cudaGetDevice(&ex->device);
    // cudaMalloc, not a pooled allocation: only such memory can be exported to other processes
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ex->region), ex->regionBytes);
    if (e == cudaSuccess) e = cudaMemset(ex->region, 0, sizeof(Control));
    if (e != cudaSuccess) {
        if (ex->region != nullptr) (void)cudaFree(ex->region);
        delete ex;
        return (int)e;
    }
    ex->peers.base[rank] = ex->region;
    if (world == 1) ex->imported = true;
    *out = ex;
    return 0;
}

int b200spMgExchangeExport(b200spMgExchange *ex, void *handle)
{
    if (ex == nullptr || handle == nullptr) return (int)cudaErrorInvalidValue;
    static_assert(sizeof(cudaIpcMemHandle_t) <= B200SP_MG_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, ex->region);
    if (e != cudaSuccess) return (int)e;
    unsigned char *dst = static_cast<unsigned char *>(handle);
    for (size_t i = 0; i < B200SP_MG_HANDLE_BYTES; ++i) dst[i] = i < sizeof(h) ? reinterpret_cast<unsigned char *>(&h)[i] : 0;
    return 0;
}

int b200spMgExchangeImport(b200spMgExchange *ex, const void *handles)
{
    if (ex == nullptr || handles == nullptr) return (int)cudaErrorInvalidValue;
    const unsigned char *src = static_cast<const unsigned char *>(handles);
    for (int p = 0; p < ex->world; ++p) {
        if (p == ex->rank || ex->opened[p]) continue;
        cudaIpcMemHandle_t h;
        for (size_t i = 0; i < sizeof(h); ++i) reinterpret_cast<unsigned char *>(&h)[i] = src[(size_t)p * B200SP_MG_HANDLE_BYTES + i];
        void *mapped = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return (int)e;
        ex->peers.base[p] = static_cast<unsigned char *>(mapped);
        ex->opened[p] = true;
    }
    ex->imported = true;
    return 0;
}

void *b200spMgExchangeReplica(b200spMgExchange *ex, int replica)
{
    if (ex == nullptr || replica < 0 || replica >= ex->replicas) return nullptr;
    return ex->region + sizeof(Control) + ex->replicaStride * (size_t)replica;
}

int b200spMgPush(b200spMgExchange *ex, int replica, const void *src, size_t offset, size_t bytes, uint32_t seq,
                 uint32_t wait_mask, void *stream)
{
    if (ex == nullptr || !ex->imported || replica < 0 || replica >= ex->replicas || offset + bytes > ex->bytes ||
        offset % 16 != 0 || bytes % 16 != 0 || (bytes > 0 && (src == nullptr || reinterpret_cast<uintptr_t>(src) % 16 != 0)))
        return (int)cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t vecs = bytes / 16;
    // enough CTAs to keep the links busy, few enough that the step's launch stays cheap for a small slice
    const size_t want = (vecs + 256 * 4 - 1) / (256 * 4);
    const size_t cap = (size_t)b200sp_sm_count() * 4;
    const unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
    const size_t dstOffset = sizeof(Control) + ex->replicaStride * (size_t)replica + offset;
    MgPushKernel<<<grid, 256, 0, st>>>(ex->peers, ex->rank, ex->world, static_cast<const uint4 *>(src), dstOffset, vecs,
                                       replica, seq, wait_mask, ex->waitCycles);
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

int b200spMgWait(b200spMgExchange *ex, int replica, uint32_t seq, uint32_t wait_mask, void *stream)
{
    if (ex == nullptr || !ex->imported || replica < 0 || replica >= ex->replicas) return (int)cudaErrorInvalidValue;
    MgWaitKernel<<<1, 32 < ex->world ? ex->world : 32, 0, static_cast<cudaStream_t>(stream)>>>(
        ex->peers, ex->rank, ex->world, replica, seq, wait_mask, ex->waitCycles);
    b200sp_note_launches(1);
    return (int)cudaGetLastError();
}

int b200spMgExchangeSetWaitLimit(b200spMgExchange *ex, long long sm_cycles)
{
    if (ex == nullptr || sm_cycles < 1) return (int)cudaErrorInvalidValue;
    ex->waitCycles = sm_cycles;
    return 0;
}

int b200spMgExchangeClearError(b200spMgExchange *ex)
{
    if (ex == nullptr) return (int)cudaErrorInvalidValue;
    Control *c = reinterpret_cast<Control *>(ex->region);
    return (int)cudaMemset(&c->error, 0, sizeof(uint32_t));
}

int b200spMgExchangeError(b200spMgExchange *ex)
{
    if (ex == nullptr) return -1;
    uint32_t flag = 0;
    const Control *c = reinterpret_cast<const Control *>(ex->region);
    if (cudaMemcpy(&flag, &c->error, sizeof(flag), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return (int)flag;
}

int b200spMgExchangeDestroy(b200spMgExchange *ex)
{
    if (ex == nullptr) return 0;
    int prev = 0;
    const bool havePrev = cudaGetDevice(&prev) == cudaSuccess;
    (void)cudaSetDevice(ex->device);
    (void)cudaDeviceSynchronize();
    for (int p = 0; p < ex->world; ++p)
        if (ex->opened[p]) (void)cudaIpcCloseMemHandle(ex->peers.base[p]);
    if (ex->region != nullptr) (void)cudaFree(ex->region);
    if (havePrev) (void)cudaSetDevice(prev);
    delete ex;
    return 0;
}

}  // extern "C"
