/* Stand-in for ARM's <arm_fp16.h> on x86-64 hosts: the reference SpMV harness
 * (test/spmv/arch22/spmv_test.cpp:23,28) only needs the scalar type name `__fp16`.
 * GCC's _Float16 is IEEE binary16 with round-to-nearest-even conversions, the same
 * arithmetic type. */
#ifndef B200SP_REF_SHIM_ARM_FP16_H_
#define B200SP_REF_SHIM_ARM_FP16_H_
typedef _Float16 __fp16;
#endif
