// C ABI over the golden and generators of the reference's SpMM harness for Ascend 910B
// (REF_SOURCE = <reference>/test/spmm/arch22/spmm_test.cpp, compiled from where it lies).
// TEST INFRASTRUCTURE ONLY.
#define main ref_spmm22_harness_main
#include REF_SOURCE
#undef main

extern "C" void ref_spmm_csr_cpu(uint64_t M, uint64_t K, uint64_t N, const int *offsets, const int *indices,
                                 const float *values, const float *B, const float *C, float *Y, float alpha,
                                 float beta)
{
    spmm_csr_cpu(M, K, N, offsets, indices, values, B, C, Y, alpha, beta);
}

// dist 0 = uniform rows, 1 = power-law rows (the harness's two generators, mt19937(42) columns).
extern "C" void ref_generate_csr(int dist, uint64_t rows, uint64_t cols, uint64_t nnz, int *offsets, int *indices,
                                 float *values)
{
    if (dist == 0) generate_random_csr(rows, cols, nnz, offsets, indices, values);
    else generate_powerlaw_csr(rows, cols, nnz, offsets, indices, values);
}

extern "C" int ref_verify_result(const float *actual, const float *expected, uint64_t count, float rel_tol,
                                 float abs_tol)
{
    return verify_result(actual, expected, count, rel_tol, abs_tol);
}
