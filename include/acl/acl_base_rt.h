/*
 * acl/acl_base_rt.h -- stand-in for the CANN runtime base header on a CUDA host.
 *
 * The sparse API header (cann_ops_sparse.h) pulls `aclDataType` and `aclrtStream`
 * from this include (reference: include/cann_ops_sparse.h:18).  CANN itself is not
 * present on a B200 box, so this file provides the same identifier names on top of
 * the CUDA runtime: source written against the reference header compiles unchanged.
 *
 *  - aclDataType enumerators carry the numeric values documented for CANN's
 *    acl_base.h, so a value stored by a caller means the same thing in both stacks.
 *  - aclrtStream is the CUDA stream handle; a null stream selects the legacy
 *    default stream.
 */
#ifndef B200SP_ACL_BASE_RT_H_
#define B200SP_ACL_BASE_RT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    ACL_DT_UNDEFINED = -1,
    ACL_FLOAT = 0,
    ACL_FLOAT16 = 1,
    ACL_INT8 = 2,
    ACL_INT32 = 3,
    ACL_UINT8 = 4,
    ACL_INT16 = 6,
    ACL_UINT16 = 7,
    ACL_UINT32 = 8,
    ACL_INT64 = 9,
    ACL_UINT64 = 10,
    ACL_DOUBLE = 11,
    ACL_BOOL = 12,
    ACL_STRING = 13,
    ACL_COMPLEX64 = 16,
    ACL_COMPLEX128 = 17,
    ACL_BF16 = 27,
    ACL_INT4 = 29,
    ACL_UINT1 = 30,
    ACL_COMPLEX32 = 33,
    ACL_HIFLOAT8 = 34,
    ACL_FLOAT8_E5M2 = 35,
    ACL_FLOAT8_E4M3FN = 36,
    ACL_FLOAT8_E8M0 = 37,
    ACL_FLOAT6_E3M2 = 38,
    ACL_FLOAT6_E2M3 = 39,
    ACL_FLOAT4_E2M1 = 40,
    ACL_FLOAT4_E1M2 = 41
} aclDataType;

typedef int aclError;
#define ACL_SUCCESS 0
#define ACL_ERROR_NONE 0

/* A CUDA stream (cudaStream_t is `struct CUstream_st *`). */
struct CUstream_st;
typedef struct CUstream_st *aclrtStream;
struct CUevent_st;
typedef struct CUevent_st *aclrtEvent;

#ifdef __cplusplus
}
#endif

#endif /* B200SP_ACL_BASE_RT_H_ */
