// Exposes the golden functions of the reference's own SpMV harness through a C ABI.
// The harness source is compiled from where it lies (REF_SOURCE is set by
// oracle/build_oracle.py to <reference>/test/spmv/arch22/spmv_test.cpp); nothing of it is
// copied here.  Its main() is renamed so the file can live in a shared library.
// TEST INFRASTRUCTURE ONLY (checker for oracle/oracle.cpp and CPU baseline).
#define main ref_spmv_harness_main
#include REF_SOURCE
#undef main

#include <cstring>

namespace {
template <typename CompT, typename ValT, typename OutT>
void Run(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, const void *yIn, void *yOut,
         int64_t rows, int64_t cols, int64_t nnz, bool trans, CompT alpha, CompT beta)
{
    const int64_t xs = trans ? rows : cols, ys = trans ? cols : rows;
    std::vector<int32_t> rp(rowPtr, rowPtr + rows + 1), ci(colInd, colInd + nnz);
    std::vector<ValT> v(static_cast<const ValT *>(val), static_cast<const ValT *>(val) + nnz);
    std::vector<ValT> xv(static_cast<const ValT *>(x), static_cast<const ValT *>(x) + xs);
    std::vector<OutT> yv(static_cast<const OutT *>(yIn), static_cast<const OutT *>(yIn) + ys);
    std::vector<OutT> z = trans ? SpmvTransCpu<CompT, ValT, OutT>(rp, ci, v, xv, yv, rows, cols, alpha, beta)
                                : SpmvCpu<CompT, ValT, OutT>(rp, ci, v, xv, yv, alpha, beta);
    std::memcpy(yOut, z.data(), sizeof(OutT) * z.size());
}
}  // namespace

// Type ids: 0 f32, 1 f16, 2 bf16 (the harness's truncating host type), 3 i32.
extern "C" int ref_spmv(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x,
                        const void *y_in, void *y_out, int64_t rows, int64_t cols, int64_t nnz, int trans,
                        int comp_type, int val_type, int out_type, const void *alpha, const void *beta)
{
    const bool t = trans != 0;
    if (comp_type == 3) {
        if (val_type != 3 || out_type != 3) return -1;
        Run<int32_t, int32_t, int32_t>(row_ptr, col_ind, val, x, y_in, y_out, rows, cols, nnz, t,
                                       *static_cast<const int32_t *>(alpha), *static_cast<const int32_t *>(beta));
        return 0;
    }
    const float a = *static_cast<const float *>(alpha), b = *static_cast<const float *>(beta);
#define CASE(V, O, VT, OT)                                                                        \
    if (val_type == V && out_type == O) {                                                         \
        Run<float, VT, OT>(row_ptr, col_ind, val, x, y_in, y_out, rows, cols, nnz, t, a, b);      \
        return 0;                                                                                 \
    }
    CASE(0, 0, float, float)
    CASE(1, 0, half, float)
    CASE(1, 1, half, half)
    CASE(2, 0, bfloat16_t, float)
    CASE(2, 2, bfloat16_t, bfloat16_t)
    CASE(3, 0, int32_t, float)
#undef CASE
    return -1;
}

// The harness's mixed-tolerance verifier on fp32 data; returns its status (0 = pass).
extern "C" int ref_spmv_verify_f32(const float *gold, const float *got, int64_t n, float *mare, float *mere)
{
    std::vector<float> g(gold, gold + n), r(got, got + n);
    return Verification<float>(g, r, *mare, *mere, GetMixedToleranceParams<float>());
}

// Times the harness's SpmvCpu<float> itself: `reps` passes over the whole matrix, the row loop cut
// into `threads` static chunks (one std::thread each, every chunk a separate SpmvCpu call on
// its slice of the row offsets; per-row arithmetic untouched).  Returns the mean seconds per pass and,
// when per_pass_seconds is not NULL, the time of each pass.
#include <thread>
#include <time.h>
extern "C" double ref_spmv_bench_f32(const int32_t *row_ptr, const int32_t *col_ind, const float *val,
                                     const float *x, const float *y, int64_t rows, int64_t cols, int64_t nnz,
                                     float alpha, float beta, int threads, int reps, double *per_pass_seconds)
{
    if (threads < 1) threads = 1;
    const std::vector<int32_t> ci(col_ind, col_ind + nnz);
    const std::vector<float> v(val, val + nnz), xv(x, x + cols);
    std::vector<std::vector<int32_t>> rp(threads);
    std::vector<std::vector<float>> ys(threads);
    const int64_t chunk = (rows + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t lo = std::min<int64_t>(rows, t * chunk), hi = std::min<int64_t>(rows, lo + chunk);
        rp[t].assign(row_ptr + lo, row_ptr + hi + 1);  // offsets stay global: they index ci / v directly
        ys[t].assign(y + lo, y + hi);
    }
    volatile float sink = 0.0f;
    struct timespec t0, t1, ta, tb;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int r = 0; r < reps; ++r) {
        clock_gettime(CLOCK_MONOTONIC, &ta);
        std::vector<std::thread> pool;
        for (int t = 0; t < threads; ++t)
            pool.emplace_back([&, t] {
                if (rp[t].size() < 2) return;
                std::vector<float> z = SpmvCpu<float, float, float>(rp[t], ci, v, xv, ys[t], alpha, beta);
                sink = sink + z[0];
            });
        for (auto &th : pool) th.join();
        clock_gettime(CLOCK_MONOTONIC, &tb);
        if (per_pass_seconds) per_pass_seconds[r] = (tb.tv_sec - ta.tv_sec) + (tb.tv_nsec - ta.tv_nsec) * 1e-9;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return ((t1.tv_sec - t0.tv_sec) + (t1.tv_nsec - t0.tv_nsec) * 1e-9) / (reps > 0 ? reps : 1);
}
