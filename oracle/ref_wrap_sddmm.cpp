// Exposes the reference's SDDMM golden, its fp16 converters, its sparsity generator and its test frame's
// mixed-tolerance verifier through a C ABI:
//   SddmmGolden / MakeSddmmSparsity / Fp32ToFp16Bits / Fp16BitsToFp32   test/sddmm/sddmm/sddmm_golden.h:63,106,158,200
//   Verifier::verifyVector with applyMixedTolerance                       test/frame/verify.h:238-246,315-331
// The headers are compiled from where they lie (REF_SDDMM_GOLDEN is set by oracle/build_oracle.py, the test
// frame's directory is on the include path); nothing of them is copied here.  TEST INFRASTRUCTURE ONLY.
#include "cann_ops_sparse.h"
#include REF_SDDMM_GOLDEN

#include <cstring>

extern "C" void ref_sddmm_f64(int64_t m, int64_t n, int64_t k, const double *X, int64_t x_len, const double *Y,
                              int64_t y_len, const int32_t *row_offsets, const int32_t *col_ind, const double *c_init,
                              int64_t nnz, double alpha, double beta, int op_x_t, int op_y_t, double *out)
{
    sparse_test::SddmmCsr csr;
    csr.m = m;
    csr.n = n;
    csr.nnz = nnz;
    csr.rowOffsets.assign(row_offsets, row_offsets + m + 1);
    csr.colIndices.assign(col_ind, col_ind + nnz);
    csr.values.assign(c_init, c_init + nnz);
    std::vector<double> x(X, X + x_len), y(Y, Y + y_len);
    const std::vector<double> r = sparse_test::SddmmGolden(
        m, n, k, x, y, csr, alpha, beta, op_x_t ? ACL_SPARSE_OP_TRANSPOSE : ACL_SPARSE_OP_NON_TRANSPOSE,
        op_y_t ? ACL_SPARSE_OP_TRANSPOSE : ACL_SPARSE_OP_NON_TRANSPOSE);
    if (nnz > 0) std::memcpy(out, r.data(), sizeof(double) * (size_t)nnz);
}

// Pattern of MakeSddmmSparsity: first call with col_ind == NULL returns nnz, second fills the arrays.
extern "C" int64_t ref_sddmm_sparsity(int64_t m, int64_t n, double ratio, double lo, double hi, uint32_t seed,
                                      int32_t *row_offsets, int32_t *col_ind, double *values)
{
    const sparse_test::SddmmCsr c = sparse_test::MakeSddmmSparsity(m, n, ratio, lo, hi, seed);
    if (col_ind != nullptr) {
        std::memcpy(row_offsets, c.rowOffsets.data(), sizeof(int32_t) * c.rowOffsets.size());
        if (c.nnz > 0) {
            std::memcpy(col_ind, c.colIndices.data(), sizeof(int32_t) * (size_t)c.nnz);
            std::memcpy(values, c.values.data(), sizeof(double) * (size_t)c.nnz);
        }
    }
    return c.nnz;
}

extern "C" void ref_sddmm_f32_to_f16(const float *in, uint16_t *out, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) out[i] = sparse_test::Fp32ToFp16Bits(in[i]);
}
extern "C" void ref_sddmm_f16_to_f32(const uint16_t *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) out[i] = sparse_test::Fp16BitsToFp32(in[i]);
}

// dtype: 0 = ACL_FLOAT, 1 = ACL_FLOAT16, 27 = ACL_BF16.  Returns 1 when the frame's verifier passes.
extern "C" int ref_verify_mixed_tolerance(const float *output, const float *golden, int64_t count, int dtype)
{
    sparse_test::VerifyConfig cfg;
    sparse_test::applyMixedTolerance(cfg, static_cast<aclDataType>(dtype), golden, (size_t)count);
    return sparse_test::Verifier::verifyVector(output, golden, (size_t)count, 1, cfg, "ref") ? 1 : 0;
}

// The dense inputs as the reference's SDDMM test draws them (GenerateSddmmInputs,
// test/sddmm/sddmm/arch35/sddmm_test.cpp:141-157): std::mt19937(seed) through
// std::uniform_real_distribution<double>(lo, hi); X uses seed + 1, Y seed + 2.
extern "C" void ref_sddmm_uniform(uint32_t seed, double lo, double hi, int64_t n, double *out)
{
    std::mt19937 rng(seed);
    std::uniform_real_distribution<double> dist(lo, hi);
    for (int64_t i = 0; i < n; ++i) out[i] = dist(rng);
}
