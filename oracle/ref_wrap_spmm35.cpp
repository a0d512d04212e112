// C ABI over the golden functions of the reference's SpMM harness for Ascend 950
// (REF_SOURCE = <reference>/test/spmm/arch35/spmm_test.cpp, compiled from where it lies).
// TEST INFRASTRUCTURE ONLY.
#define main ref_spmm35_harness_main
#include REF_SOURCE
#undef main

extern "C" void ref_spmm_f32(int32_t m, int32_t n, int64_t nnz, const int32_t *row_ptr, const int32_t *col_ind,
                             const float *val, const float *B, int64_t b_elems, int32_t ldb, int b_row_major,
                             int op_b_transpose, float *C, int64_t c_elems, int32_t ldc, int c_row_major,
                             float alpha, float beta)
{
    std::vector<int32_t> rp(row_ptr, row_ptr + m + 1), ci(col_ind, col_ind + nnz);
    std::vector<float> v(val, val + nnz), b(B, B + b_elems), c(C, C + c_elems);
    SpmmCpuFp32(m, n, rp, ci, v, b, ldb, b_row_major != 0, op_b_transpose != 0, &c, ldc, c_row_major != 0, alpha,
                beta);
    std::copy(c.begin(), c.end(), C);
}

extern "C" void ref_spmm_i8(int32_t m, int32_t n, int64_t nnz, const int32_t *row_ptr, const int32_t *col_ind,
                            const int8_t *val, const int8_t *B, int64_t b_elems, int32_t ldb, int b_row_major,
                            int op_b_transpose, int32_t *C, int64_t c_elems, int32_t ldc, int c_row_major,
                            int32_t alpha, int32_t beta)
{
    std::vector<int32_t> rp(row_ptr, row_ptr + m + 1), ci(col_ind, col_ind + nnz);
    std::vector<int8_t> v(val, val + nnz), b(B, B + b_elems);
    std::vector<int32_t> c(C, C + c_elems);
    SpmmCpuInt8(m, n, rp, ci, v, b, ldb, b_row_major != 0, op_b_transpose != 0, &c, ldc, c_row_major != 0, alpha,
                beta);
    std::copy(c.begin(), c.end(), C);
}

extern "C" void ref_f32_to_f16(const float *in, uint16_t *out, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) out[i] = Fp32ToFp16Bits(in[i]);
}
extern "C" void ref_f16_to_f32(const uint16_t *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) out[i] = Fp16BitsToFp32(in[i]);
}

// The harness's deterministic CSR generator (std::srand(seed) + std::rand()).
// Returns the nnz actually produced; arrays must hold m + 1 / nnz entries.
extern "C" int32_t ref_generate_random_csr(uint32_t seed, int32_t m, int32_t k, int32_t nnz, int32_t *row_ptr,
                                           int32_t *col_ind, float *val)
{
    std::srand(seed);
    std::vector<int32_t> rp, ci;
    std::vector<float> v;
    GenerateRandomCsr(m, k, nnz, &rp, &ci, &v);
    std::copy(rp.begin(), rp.end(), row_ptr);
    std::copy(ci.begin(), ci.end(), col_ind);
    std::copy(v.begin(), v.end(), val);
    return rp.back();
}

// Times the harness's SpmmCpuFp32 itself on compact row-major operands: `reps` passes over rows
// [0, m), the row loop cut into `threads` static chunks (one SpmmCpuFp32 call per chunk on its
// slice of the row offsets and of C).  Returns the mean seconds per pass and,
// when per_pass_seconds is not NULL, the time of each pass.
#include <thread>
#include <time.h>
extern "C" double ref_spmm_bench_f32(int32_t m, int32_t k, int32_t n, int64_t nnz, const int32_t *row_ptr,
                                     const int32_t *col_ind, const float *val, const float *B, const float *C,
                                     float alpha, float beta, int threads, int reps, double *per_pass_seconds)
{
    if (threads < 1) threads = 1;
    const std::vector<int32_t> ci(col_ind, col_ind + nnz);
    const std::vector<float> v(val, val + nnz), b(B, B + (int64_t)k * n);
    std::vector<std::vector<int32_t>> rp(threads);
    std::vector<std::vector<float>> cs(threads);
    const int64_t chunk = ((int64_t)m + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t lo = std::min<int64_t>(m, t * chunk), hi = std::min<int64_t>(m, lo + chunk);
        rp[t].assign(row_ptr + lo, row_ptr + hi + 1);
        cs[t].assign(C + lo * n, C + hi * n);
    }
    struct timespec t0, t1, ta, tb;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int r = 0; r < reps; ++r) {
        clock_gettime(CLOCK_MONOTONIC, &ta);
        std::vector<std::thread> pool;
        for (int t = 0; t < threads; ++t)
            pool.emplace_back([&, t] {
                if (rp[t].size() < 2) return;
                SpmmCpuFp32((int32_t)rp[t].size() - 1, n, rp[t], ci, v, b, n, true, false, &cs[t], n, true, alpha, beta);
            });
        for (auto &th : pool) th.join();
        clock_gettime(CLOCK_MONOTONIC, &tb);
        if (per_pass_seconds) per_pass_seconds[r] = (tb.tv_sec - ta.tv_sec) + (tb.tv_nsec - ta.tv_nsec) * 1e-9;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return ((t1.tv_sec - t0.tv_sec) + (t1.tv_nsec - t0.tv_nsec) * 1e-9) / (reps > 0 ? reps : 1);
}
