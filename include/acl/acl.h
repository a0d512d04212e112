/*
 * acl/acl.h -- the slice of the CANN runtime that callers of the SpMV / SpMM path
 * use around the sparse API, mapped onto the CUDA runtime as header-only inlines.
 *
 * The reference's own harnesses allocate, copy and synchronise with these calls
 * (test/spmv/arch22/spmv_test.cpp:326-351, 428-446, 483-491;
 *  test/spmm/arch35/spmm_test.cpp:72-89, 431-458;
 *  test/spmm/arch22/spmm_test.cpp:208-295 for the event-timed loop).
 * With this header on the include path such a caller builds against the CUDA
 * runtime with no source change; link with -lcudart.
 */
#ifndef B200SP_ACL_H_
#define B200SP_ACL_H_

#include <cuda_runtime_api.h>
#include "acl/acl_base_rt.h"

typedef enum {
    ACL_MEM_MALLOC_HUGE_FIRST = 0,
    ACL_MEM_MALLOC_HUGE_ONLY = 1,
    ACL_MEM_MALLOC_NORMAL_ONLY = 2
} aclrtMemMallocPolicy;

typedef enum {
    ACL_MEMCPY_HOST_TO_HOST = 0,
    ACL_MEMCPY_HOST_TO_DEVICE = 1,
    ACL_MEMCPY_DEVICE_TO_HOST = 2,
    ACL_MEMCPY_DEVICE_TO_DEVICE = 3
} aclrtMemcpyKind;

static inline aclError b200spAclErr(cudaError_t e) { return e == cudaSuccess ? ACL_SUCCESS : 100000 + (int)e; }

static inline aclError aclInit(const char *configPath) { (void)configPath; return ACL_SUCCESS; }
static inline aclError aclFinalize(void) { return ACL_SUCCESS; }
static inline aclError aclrtSetDevice(int32_t deviceId) { return b200spAclErr(cudaSetDevice(deviceId)); }
static inline aclError aclrtGetDevice(int32_t *deviceId) { int d = 0; cudaError_t e = cudaGetDevice(&d); *deviceId = d; return b200spAclErr(e); }
/* The CANN call tears the device context down; on a shared CUDA process that would
 * also destroy other users' allocations, so only pending work is drained here. */
static inline aclError aclrtResetDevice(int32_t deviceId) { (void)deviceId; return b200spAclErr(cudaDeviceSynchronize()); }
static inline aclError aclrtSynchronizeDevice(void) { return b200spAclErr(cudaDeviceSynchronize()); }

static inline aclError aclrtCreateStream(aclrtStream *stream) { return b200spAclErr(cudaStreamCreate((cudaStream_t *)stream)); }
static inline aclError aclrtDestroyStream(aclrtStream stream) { return b200spAclErr(cudaStreamDestroy((cudaStream_t)stream)); }
static inline aclError aclrtSynchronizeStream(aclrtStream stream) { return b200spAclErr(cudaStreamSynchronize((cudaStream_t)stream)); }

static inline aclError aclrtMalloc(void **devPtr, size_t size, aclrtMemMallocPolicy policy)
{
    (void)policy;
    /* CANN rejects size 0; cudaMalloc(0) returns a null pointer.  Keep one byte so
     * callers that malloc empty arrays still get a valid, freeable pointer. */
    return b200spAclErr(cudaMalloc(devPtr, size ? size : 1));
}
static inline aclError aclrtFree(void *devPtr) { return b200spAclErr(cudaFree(devPtr)); }
static inline aclError aclrtMallocHost(void **hostPtr, size_t size) { return b200spAclErr(cudaMallocHost(hostPtr, size ? size : 1)); }
static inline aclError aclrtFreeHost(void *hostPtr) { return b200spAclErr(cudaFreeHost(hostPtr)); }

static inline aclError aclrtMemcpy(void *dst, size_t destMax, const void *src, size_t count, aclrtMemcpyKind kind)
{
    if (count > destMax) return 100001;
    if (count == 0) return ACL_SUCCESS;
    enum cudaMemcpyKind k = cudaMemcpyDefault;
    switch (kind) {
        case ACL_MEMCPY_HOST_TO_HOST: k = cudaMemcpyHostToHost; break;
        case ACL_MEMCPY_HOST_TO_DEVICE: k = cudaMemcpyHostToDevice; break;
        case ACL_MEMCPY_DEVICE_TO_HOST: k = cudaMemcpyDeviceToHost; break;
        case ACL_MEMCPY_DEVICE_TO_DEVICE: k = cudaMemcpyDeviceToDevice; break;
    }
    return b200spAclErr(cudaMemcpy(dst, src, count, k));
}
static inline aclError aclrtMemset(void *devPtr, size_t maxCount, int32_t value, size_t count)
{
    if (count > maxCount) return 100001;
    return b200spAclErr(cudaMemset(devPtr, value, count));
}

static inline aclError aclrtCreateEvent(aclrtEvent *event) { return b200spAclErr(cudaEventCreate((cudaEvent_t *)event)); }
static inline aclError aclrtDestroyEvent(aclrtEvent event) { return b200spAclErr(cudaEventDestroy((cudaEvent_t)event)); }
static inline aclError aclrtRecordEvent(aclrtEvent event, aclrtStream stream) { return b200spAclErr(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); }
static inline aclError aclrtSynchronizeEvent(aclrtEvent event) { return b200spAclErr(cudaEventSynchronize((cudaEvent_t)event)); }
static inline aclError aclrtEventElapsedTime(float *ms, aclrtEvent start, aclrtEvent end) { return b200spAclErr(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end)); }

#endif /* B200SP_ACL_H_ */
