// CPU oracle for the CSR SpMV / SpMM path.  TEST INFRASTRUCTURE ONLY: nothing in the
// shipped library links, loads or calls this file; it is built into oracle/_build/liboracle.so
// and used by tests/, the smoke check and bench.py's CPU-baseline leg as the checker.
//
// Every routine restates, in plain loops, the golden the reference's own harnesses verify
// their device results against:
//   oracle_spmv          SpmvCpu        test/spmv/arch22/spmv_test.cpp:156-173
//   oracle_spmv_trans    SpmvTransCpu   test/spmv/arch22/spmv_test.cpp:177-197
//   oracle_spmm_f32      SpmmCpuFp32    test/spmm/arch35/spmm_test.cpp:125-161
//                        (= spmm_csr_cpu, test/spmm/arch22/spmm_test.cpp:133-147, when both
//                        operands are compact row-major)
//   oracle_spmm_16       the fp16 recipe  test/spmm/arch35/spmm_test.cpp:604-622
//                        (round inputs to 16 bit, fp32 loop, clamp to +-65504, round output)
//   oracle_spmm_i8       SpmmCpuInt8    test/spmm/arch35/spmm_test.cpp:163-200, with the
//                        device kernel's int64 saturating epilogue
//                        (sparse/spmm/arch35/spmm_kernel.cpp:251-266) selectable
//   oracle_f32_to_f16 / f16_to_f32   Fp32ToFp16Bits / Fp16BitsToFp32  spmm_test.cpp:303-373
//   oracle_f32_to_bf16_trunc         host bfloat16_t of spmv_test.cpp:30-50 (truncates)
//   oracle_f32_to_bf16_rne           round-to-nearest-even, what the device cast does
//   verifiers: mixed tolerance (spmv_test.cpp:208-324), MERE / MARE (spmm_test.cpp:202-252),
//   arch22 diff-and-relative rule (spmm/arch22/spmm_test.cpp:149-170).
//
// Parity is pinned: tests/test_oracle_pins.py checks these routines against the 4x3 known
// answer of sparse/spmm/README.md:276-305,404-412 and, when the reference sources are
// present, bit-for-bit against the reference's own golden functions compiled from where
// they lie (oracle/_ref, built by oracle/build_oracle.py).
//
// Summation order is the golden's: one accumulator per output, non-zeros in CSR order.
// The SpMM loops run non-zeros outermost and columns innermost; each output still sees its
// products in the same order, so results are bit-identical to the golden's j-outer loops.
// `threads` > 1 splits the row loop statically; per-row arithmetic is untouched.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

enum Type : int { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, I8 = 4 };

// ---- 16-bit float conversions -------------------------------------------------------

inline uint32_t Bits(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
inline float FromBits(uint32_t u)
{
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

inline float HalfToFloat(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    const uint32_t man = h & 0x3ffu;
    if (exp == 0x1f) return FromBits(sign | 0x7f800000u | (man << 13));
    if (exp != 0) return FromBits(sign | ((exp + 112u) << 23) | (man << 13));
    if (man == 0) return FromBits(sign);
    // subnormal: value = man * 2^-24, exact in fp32
    const float v = (float)man * 5.9604644775390625e-08f;
    return (h & 0x8000u) ? -v : v;
}

inline uint16_t FloatToHalfRne(float f)
{
    const uint32_t u = Bits(f);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t absu = u & 0x7fffffffu;
    if (absu >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (absu > 0x7f800000u ? 0x0200u : 0u));
    if (absu >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);  // >= 65536 -> inf
    if (absu < 0x33000000u) return sign;                          // < 2^-25 -> 0
    uint32_t mant, shift;
    int32_t e = (int32_t)(absu >> 23) - 127;
    if (e >= -14) {  // normal half
        mant = absu & 0x7fffffu;
        shift = 13;
        uint32_t out = ((uint32_t)(e + 15) << 10) | (mant >> shift);
        const uint32_t rem = mant & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (out & 1u))) ++out;  // may carry into the exponent: correct
        return (uint16_t)(sign | out);
    }
    // subnormal half: align the 24-bit significand to 2^-24 units
    mant = (absu & 0x7fffffu) | 0x800000u;
    shift = (uint32_t)(-e - 1);  // 14..24
    uint32_t out = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (out & 1u))) ++out;
    return (uint16_t)(sign | out);
}

inline float Bf16ToFloat(uint16_t b) { return FromBits((uint32_t)b << 16); }
inline uint16_t FloatToBf16Trunc(float f) { return (uint16_t)(Bits(f) >> 16); }
inline uint16_t FloatToBf16Rne(float f)
{
    const uint32_t u = Bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
    const uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

// ---- typed element access -----------------------------------------------------------

template <typename CompT>
inline CompT LoadAs(const void *p, int type, int64_t i)
{
    switch (type) {
        case F32: return (CompT) static_cast<const float *>(p)[i];
        case F16: return (CompT)HalfToFloat(static_cast<const uint16_t *>(p)[i]);
        case BF16: return (CompT)Bf16ToFloat(static_cast<const uint16_t *>(p)[i]);
        case I32: return (CompT) static_cast<const int32_t *>(p)[i];
        case I8: return (CompT) static_cast<const int8_t *>(p)[i];
    }
    return CompT(0);
}

template <typename CompT>
inline void StoreFrom(void *p, int type, int64_t i, CompT v, int bf16Trunc)
{
    switch (type) {
        case F32: static_cast<float *>(p)[i] = (float)v; break;
        case F16: static_cast<uint16_t *>(p)[i] = FloatToHalfRne((float)v); break;
        case BF16:
            static_cast<uint16_t *>(p)[i] = bf16Trunc ? FloatToBf16Trunc((float)v) : FloatToBf16Rne((float)v);
            break;
        case I32: static_cast<int32_t *>(p)[i] = (int32_t)v; break;
        default: break;
    }
}

template <typename F>
void ParallelRows(int64_t rows, int threads, F &&body)
{
    if (threads <= 1 || rows < 2) {
        body(0, rows);
        return;
    }
    std::vector<std::thread> pool;
    const int64_t chunk = (rows + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t lo = std::min<int64_t>(rows, t * chunk), hi = std::min<int64_t>(rows, lo + chunk);
        if (lo < hi) pool.emplace_back([=, &body] { body(lo, hi); });
    }
    for (auto &th : pool) th.join();
}

// ---- SpMV ---------------------------------------------------------------------------

template <typename CompT>
void SpmvRows(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, int valType,
              const void *yIn, void *yOut, int outType, int64_t lo, int64_t hi, CompT alpha, CompT beta,
              int bf16Trunc)
{
    for (int64_t i = lo; i < hi; ++i) {
        CompT sum = 0;
        for (int32_t j = rowPtr[i]; j < rowPtr[i + 1]; ++j)
            sum += LoadAs<CompT>(val, valType, j) * LoadAs<CompT>(x, valType, colInd[j]);
        const CompT z = alpha * sum + beta * LoadAs<CompT>(yIn, outType, i);
        StoreFrom<CompT>(yOut, outType, i, z, bf16Trunc);
    }
}

template <typename CompT>
void SpmvTrans(const int32_t *rowPtr, const int32_t *colInd, const void *val, const void *x, int valType,
               const void *yIn, void *yOut, int outType, int64_t rows, int64_t cols, CompT alpha, CompT beta,
               int bf16Trunc)
{
    // The running value is rounded to the output type after every update, as the golden does.
    for (int64_t j = 0; j < cols; ++j)
        StoreFrom<CompT>(yOut, outType, j, beta * LoadAs<CompT>(yIn, outType, j), bf16Trunc);
    for (int64_t i = 0; i < rows; ++i) {
        const CompT xv = alpha * LoadAs<CompT>(x, valType, i);
        if (xv == CompT(0)) continue;
        for (int32_t k = rowPtr[i]; k < rowPtr[i + 1]; ++k) {
            const int32_t c = colInd[k];
            StoreFrom<CompT>(yOut, outType, c, LoadAs<CompT>(yOut, outType, c) + xv * LoadAs<CompT>(val, valType, k),
                             bf16Trunc);
        }
    }
}

// ---- SpMM ---------------------------------------------------------------------------

struct DenseLayout {
    int64_t ldb, ldc;
    int bRowMajor, cRowMajor, opB;
};

inline int64_t BIndex(const DenseLayout &d, int64_t c, int64_t j)
{
    if (!d.opB) return d.bRowMajor ? c * d.ldb + j : j * d.ldb + c;
    return d.bRowMajor ? j * d.ldb + c : c * d.ldb + j;
}
inline int64_t CIndex(const DenseLayout &d, int64_t r, int64_t j) { return d.cRowMajor ? r * d.ldc + j : j * d.ldc + r; }

void SpmmRowsF32(int64_t lo, int64_t hi, int64_t n, const int32_t *rowPtr, const int32_t *colInd, const float *val,
                 const float *B, float *C, const DenseLayout &d, float alpha, float beta, bool clampHalf)
{
    std::vector<float> acc((size_t)n);
    const bool bContig = BIndex(d, 0, 1) == 1;  // op(B) rows contiguous
    for (int64_t r = lo; r < hi; ++r) {
        std::fill(acc.begin(), acc.end(), 0.0f);
        for (int32_t p = rowPtr[r]; p < rowPtr[r + 1]; ++p) {
            const float v = val[p];
            const int64_t c = colInd[p];
            if (bContig) {
                const float *brow = B + BIndex(d, c, 0);
                for (int64_t j = 0; j < n; ++j) acc[j] += v * brow[j];
            } else {
                for (int64_t j = 0; j < n; ++j) acc[j] += v * B[BIndex(d, c, j)];
            }
        }
        for (int64_t j = 0; j < n; ++j) {
            const int64_t ci = CIndex(d, r, j);
            float z = alpha * acc[j] + beta * C[ci];
            if (clampHalf) z = std::min(std::max(z, -65504.0f), 65504.0f);
            C[ci] = z;
        }
    }
}

}  // namespace

extern "C" {

// ---- conversions (array forms) --------------------------------------------------------
void oracle_f32_to_f16(const float *in, uint16_t *out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = FloatToHalfRne(in[i]); }
void oracle_f16_to_f32(const uint16_t *in, float *out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = HalfToFloat(in[i]); }
void oracle_f32_to_bf16_rne(const float *in, uint16_t *out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = FloatToBf16Rne(in[i]); }
void oracle_f32_to_bf16_trunc(const float *in, uint16_t *out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = FloatToBf16Trunc(in[i]); }
void oracle_bf16_to_f32(const uint16_t *in, float *out, int64_t n) { for (int64_t i = 0; i < n; ++i) out[i] = Bf16ToFloat(in[i]); }

// y_out = alpha * A x + beta * y_in.  comp_type F32 or I32; x has val_type; y has out_type.
// alpha / beta point to a float or an int32 by comp_type.  Returns 0, or -1 on a type
// combination the golden has no instantiation for.
int oracle_spmv(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x, const void *y_in,
                void *y_out, int64_t rows, int comp_type, int val_type, int out_type, const void *alpha,
                const void *beta, int bf16_trunc, int threads)
{
    if (comp_type == F32) {
        const float a = *static_cast<const float *>(alpha), b = *static_cast<const float *>(beta);
        ParallelRows(rows, threads, [&](int64_t lo, int64_t hi) {
            SpmvRows<float>(row_ptr, col_ind, val, x, val_type, y_in, y_out, out_type, lo, hi, a, b, bf16_trunc);
        });
        return 0;
    }
    if (comp_type == I32 && val_type == I32 && out_type == I32) {
        const int32_t a = *static_cast<const int32_t *>(alpha), b = *static_cast<const int32_t *>(beta);
        ParallelRows(rows, threads, [&](int64_t lo, int64_t hi) {
            // unsigned arithmetic: the golden's int32 sums wrap on overflow
            for (int64_t i = lo; i < hi; ++i) {
                uint32_t sum = 0;
                for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j)
                    sum += (uint32_t) static_cast<const int32_t *>(val)[j] *
                           (uint32_t) static_cast<const int32_t *>(x)[col_ind[j]];
                static_cast<int32_t *>(y_out)[i] =
                    (int32_t)((uint32_t)a * sum + (uint32_t)b * (uint32_t) static_cast<const int32_t *>(y_in)[i]);
            }
        });
        return 0;
    }
    return -1;
}

// y_out = alpha * A^T x + beta * y_in (y has `cols` entries).  Sequential, row by row.
int oracle_spmv_trans(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x,
                      const void *y_in, void *y_out, int64_t rows, int64_t cols, int comp_type, int val_type,
                      int out_type, const void *alpha, const void *beta, int bf16_trunc)
{
    if (comp_type == F32) {
        SpmvTrans<float>(row_ptr, col_ind, val, x, val_type, y_in, y_out, out_type, rows, cols,
                         *static_cast<const float *>(alpha), *static_cast<const float *>(beta), bf16_trunc);
        return 0;
    }
    if (comp_type == I32 && val_type == I32 && out_type == I32) {
        const uint32_t a = (uint32_t) * static_cast<const int32_t *>(alpha);
        const uint32_t b = (uint32_t) * static_cast<const int32_t *>(beta);
        auto *z = static_cast<uint32_t *>(y_out);
        for (int64_t j = 0; j < cols; ++j) z[j] = b * (uint32_t) static_cast<const int32_t *>(y_in)[j];
        for (int64_t i = 0; i < rows; ++i) {
            const uint32_t xv = a * (uint32_t) static_cast<const int32_t *>(x)[i];
            if (xv == 0) continue;
            for (int32_t k = row_ptr[i]; k < row_ptr[i + 1]; ++k)
                z[col_ind[k]] += xv * (uint32_t) static_cast<const int32_t *>(val)[k];
        }
        return 0;
    }
    return -1;
}

// C = alpha * A * op(B) + beta * C, all fp32, any layout.  C is updated in place.
void oracle_spmm_f32(int64_t m, int64_t n, const int32_t *row_ptr, const int32_t *col_ind, const float *val,
                     const float *B, int64_t ldb, int b_row_major, int op_b_transpose, float *C, int64_t ldc,
                     int c_row_major, float alpha, float beta, int threads)
{
    const DenseLayout d{ldb, ldc, b_row_major, c_row_major, op_b_transpose};
    ParallelRows(m, threads, [&](int64_t lo, int64_t hi) {
        SpmmRowsF32(lo, hi, n, row_ptr, col_ind, val, B, C, d, alpha, beta, false);
    });
}

// 16-bit storage variant: A and B hold fp16 (in_type = 1) or bf16 (in_type = 2) bit patterns
// of `b_elems` / nnz elements; C holds out_type (0 f32, 1 f16, 2 bf16) with `c_elems`
// elements.  Inputs are widened, the fp32 loop runs, fp16 output is clamped to +-65504,
// the result is rounded to out_type (RNE).
int oracle_spmm_16(int64_t m, int64_t n, int64_t nnz, const int32_t *row_ptr, const int32_t *col_ind,
                   const uint16_t *val, const uint16_t *B, int64_t b_elems, int64_t ldb, int b_row_major,
                   int op_b_transpose, void *C, int64_t c_elems, int64_t ldc, int c_row_major, float alpha,
                   float beta, int in_type, int out_type, int threads)
{
    if ((in_type != F16 && in_type != BF16) || (out_type != F32 && out_type != F16 && out_type != BF16)) return -1;
    std::vector<float> v((size_t)nnz), b((size_t)b_elems), c((size_t)c_elems);
    for (int64_t i = 0; i < nnz; ++i) v[i] = LoadAs<float>(val, in_type, i);
    for (int64_t i = 0; i < b_elems; ++i) b[i] = LoadAs<float>(B, in_type, i);
    for (int64_t i = 0; i < c_elems; ++i) c[i] = LoadAs<float>(C, out_type, i);
    const DenseLayout d{ldb, ldc, b_row_major, c_row_major, op_b_transpose};
    ParallelRows(m, threads, [&](int64_t lo, int64_t hi) {
        SpmmRowsF32(lo, hi, n, row_ptr, col_ind, v.data(), b.data(), c.data(), d, alpha, beta, out_type == F16);
    });
    // Only the m x n window is written back; padding between rows keeps its old bits.
    for (int64_t r = 0; r < m; ++r)
        for (int64_t j = 0; j < n; ++j) {
            const int64_t ci = CIndex(d, r, j);
            StoreFrom<float>(C, out_type, ci, c[ci], 0);
        }
    return 0;
}

// int8 x int8 -> int32.  saturate = 0: the golden's plain int32 arithmetic (wraps);
// saturate = 1: int64 epilogue clamped to the int32 range, as the device kernel does.
void oracle_spmm_i8(int64_t m, int64_t n, const int32_t *row_ptr, const int32_t *col_ind, const int8_t *val,
                    const int8_t *B, int64_t ldb, int b_row_major, int op_b_transpose, int32_t *C, int64_t ldc,
                    int c_row_major, int32_t alpha, int32_t beta, int saturate)
{
    const DenseLayout d{ldb, ldc, b_row_major, c_row_major, op_b_transpose};
    for (int64_t r = 0; r < m; ++r)
        for (int64_t j = 0; j < n; ++j) {
            uint32_t acc = 0;
            for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p)
                acc += (uint32_t)((int32_t)val[p] * (int32_t)B[BIndex(d, col_ind[p], j)]);
            const int64_t ci = CIndex(d, r, j);
            if (saturate) {
                int64_t w = (int64_t)alpha * (int64_t)(int32_t)acc + (int64_t)beta * (int64_t)C[ci];
                w = std::min<int64_t>(std::max<int64_t>(w, INT32_MIN), INT32_MAX);
                C[ci] = (int32_t)w;
            } else {
                C[ci] = (int32_t)((uint32_t)alpha * acc + (uint32_t)beta * (uint32_t)C[ci]);
            }
        }
}

// ---- error scales for the per-row tolerance  |err_i| <= tol * sum_j |a_ij * x_j| ----------
void oracle_spmv_abs_rowsum(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x,
                            int val_type, int64_t rows, double *out)
{
    for (int64_t i = 0; i < rows; ++i) {
        double s = 0.0;
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j)
            s += std::fabs(LoadAs<double>(val, val_type, j) * LoadAs<double>(x, val_type, col_ind[j]));
        out[i] = s;
    }
}

// out[r * n + j] = sum_p |a_p| * |B[col_p, j]| for compact row-major B (ldb = n).
void oracle_spmm_abs_sum(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *B,
                         int val_type, int64_t m, int64_t n, double *out)
{
    for (int64_t r = 0; r < m; ++r) {
        double *o = out + r * n;
        std::fill(o, o + n, 0.0);
        for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
            const double v = std::fabs(LoadAs<double>(val, val_type, p));
            const int64_t c = col_ind[p];
            for (int64_t j = 0; j < n; ++j) o[j] += v * std::fabs(LoadAs<double>(B, val_type, c * n + j));
        }
    }
}

// ---- CSR producers (integer work: results must match the reference's goldens bit for bit) ----------

// aclsparseXcsrsort: inside every row the column indices are put in ascending order, equal columns keep their
// input order, and the permutation array travels with them (csrsortGolden, test/csrsort/arch35/
// csrsort_golden.h:38-70).  row_ptr is in `index_base`.
void oracle_csrsort(const int32_t *row_ptr, const int32_t *col_ind, const int32_t *perm, int m, int index_base,
                    int32_t *col_out, int32_t *perm_out)
{
    std::vector<int32_t> order;
    for (int r = 0; r < m; ++r) {
        const int lo = row_ptr[r] - index_base, hi = row_ptr[r + 1] - index_base;
        order.resize((size_t)std::max(hi - lo, 0));
        for (int i = 0; i < hi - lo; ++i) order[(size_t)i] = lo + i;
        std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return col_ind[a] < col_ind[b]; });
        for (int i = 0; i < hi - lo; ++i) {
            col_out[lo + i] = col_ind[order[(size_t)i]];
            perm_out[lo + i] = perm[order[(size_t)i]];
        }
    }
}

// aclsparseXcoo2csr: row pointers from sorted COO row indices by counting and a running sum; indices outside
// [0, m) after removing the base are ignored (Coo2CsrGolden, test/coo2csr/coo2csr_golden.h:44-77).
void oracle_coo2csr(const int32_t *coo_row, int nnz, int m, int index_base, int32_t *row_ptr)
{
    for (int i = 0; i <= m; ++i) row_ptr[i] = index_base;
    if (nnz <= 0 || m <= 0) return;
    std::vector<int64_t> count((size_t)m, 0);
    for (int k = 0; k < nnz; ++k) {
        const int r = (int)((uint32_t)coo_row[k] - (uint32_t)index_base);
        if (r >= 0 && r < m) ++count[(size_t)r];
    }
    int64_t running = 0;
    for (int i = 0; i < m; ++i) {
        running += count[(size_t)i];
        row_ptr[i + 1] = (int32_t)(running + index_base);
    }
}

// aclsparseCsr2cscEx2: column counts, exclusive scan, then every entry is dropped into its column in row order,
// values moved as raw bytes (Csr2CscGolden, test/csr2csc_ex2/csr2csc_ex2_golden.h:50-110).
void oracle_csr2csc(int m, int n, int nnz, const int32_t *row_ptr, const int32_t *col_ind, const void *values,
                    int value_bytes, int index_base, int32_t *col_ptr, int32_t *row_ind, void *val_out)
{
    for (int j = 0; j <= n; ++j) col_ptr[j] = index_base;
    if (nnz <= 0) return;
    std::vector<int32_t> next((size_t)n, 0);
    for (int k = 0; k < nnz; ++k) ++next[(size_t)(col_ind[k] - index_base)];
    int32_t running = 0;
    for (int j = 0; j < n; ++j) {
        const int32_t c = next[(size_t)j];
        next[(size_t)j] = running;
        running += c;
        col_ptr[j + 1] = running + index_base;
    }
    const unsigned char *src = static_cast<const unsigned char *>(values);
    unsigned char *dst = static_cast<unsigned char *>(val_out);
    for (int r = 0; r < m; ++r) {
        for (int k = row_ptr[r] - index_base; k < row_ptr[r + 1] - index_base; ++k) {
            const int32_t where = next[(size_t)(col_ind[k] - index_base)]++;
            row_ind[where] = r + index_base;
            if (src != nullptr && dst != nullptr)
                std::memcpy(dst + (size_t)where * (size_t)value_bytes, src + (size_t)k * (size_t)value_bytes,
                            (size_t)value_bytes);
        }
    }
}

// ---- SDDMM: out[p] = alpha * <op(X) row i, op(Y) column j> + beta * c_init[p] in fp64 on the pattern of C
// (SddmmGolden, test/sddmm/sddmm/sddmm_golden.h:106-150).  X is m x k (or k x m when transposed), Y is k x n (or
// n x k when transposed), both row-major and compact. ---------------------------------------------------
void oracle_sddmm_f64(int64_t m, int64_t n, int64_t k, const double *X, const double *Y, const int32_t *row_offsets,
                      const int32_t *col_ind, const double *c_init, double alpha, double beta, int op_x_t, int op_y_t,
                      double *out)
{
    for (int64_t i = 0; i < m; ++i) {
        for (int32_t p = row_offsets[i]; p < row_offsets[i + 1]; ++p) {
            const int64_t j = col_ind[p];
            double dot = 0.0;
            for (int64_t t = 0; t < k; ++t) {
                const double xv = op_x_t ? X[t * m + i] : X[i * k + t];
                const double yv = op_y_t ? Y[j * k + t] : Y[t * n + j];
                dot += xv * yv;
            }
            out[p] = alpha * dot + beta * c_init[p];
        }
    }
}

// Mixed tolerance of the reference's test frame (test/frame/verify.h:193-300): an element fails when
// |out - gold| > atol + rtol * |gold|; the case passes when at least `ratio` of the elements do not fail and no
// element is further from its golden than max(limit, 32 ulp of the golden in the output type) or is NaN / inf.
// Returns 1 on pass; stats = {matched ratio, max abs error}.
int oracle_verify_mixed_tolerance(const float *out, const float *gold, int64_t count, double rtol, double atol,
                                  double limit, int mantissa_bits, int emin, double ratio, double *stats)
{
    int64_t failed = 0;
    bool beyond = false;
    double worst = 0.0;
    for (int64_t i = 0; i < count; ++i) {
        const float o = out[i], g = gold[i];
        if (std::isnan(o) || std::isnan(g) || std::isinf(o) || std::isinf(g)) {
            beyond = true;
            ++failed;
            continue;
        }
        const double diff = std::fabs((double)o - (double)g), mag = std::fabs((double)g);
        worst = std::max(worst, diff);
        double ulp;
        if (mag == 0.0) {
            ulp = std::pow(2.0, (double)(emin - mantissa_bits));
        } else {
            int e = 0;
            std::frexp(mag, &e);
            ulp = std::ldexp(1.0, std::max(e - 1, emin) - mantissa_bits);
        }
        if (diff > atol + rtol * mag) ++failed;
        if (diff > std::max(limit, 32.0 * ulp)) beyond = true;
    }
    const double matched = count > 0 ? (double)(count - failed) / (double)count : 1.0;
    if (stats != nullptr) {
        stats[0] = matched;
        stats[1] = worst;
    }
    return (matched >= ratio && !beyond) ? 1 : 0;
}

// ---- whole-result checks at benchmark size -------------------------------------------------
// The per-row tolerance of the benchmark, |got - gold| <= tol * (|alpha| * sum_j |a_ij * b_j| + |beta * old|),
// applied to EVERY output of a full-size product without materialising golden or scale arrays (config 5 has
// 537 M outputs): rows are split over `threads`, every thread forms the golden row (the arithmetic of SpmvRows /
// SpmmRowsF32 above: fp32 products added in CSR order, then alpha * sum + beta * old) and its fp64 scale and
// compares.  16-bit inputs are passed widened to fp32, which is exact.  Returns the number of outputs outside
// the tolerance; *worst receives the largest err / scale seen (0 when every scale is 0 and every error too).
int64_t oracle_check_spmv_f32(const int32_t *row_ptr, const int32_t *col_ind, const float *val, const float *x,
                              const float *y_old, const float *got, int64_t rows, float alpha, float beta, double tol,
                              int threads, double *worst)
{
    std::vector<int64_t> bad((size_t)std::max(threads, 1), 0);
    std::vector<double> worstOf((size_t)std::max(threads, 1), 0.0);
    const int64_t chunk = threads > 1 ? (rows + threads - 1) / threads : rows;
    ParallelRows(rows, threads, [&](int64_t lo, int64_t hi) {
        const size_t slot = chunk > 0 ? (size_t)(lo / chunk) : 0;
        for (int64_t i = lo; i < hi; ++i) {
            float sum = 0;
            double scale = 0.0;
            for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) {
                sum += val[j] * x[col_ind[j]];
                scale += std::fabs((double)val[j] * (double)x[col_ind[j]]);
            }
            const float old = beta != 0.0f ? y_old[i] : 0.0f;
            const float z = beta != 0.0f ? alpha * sum + beta * old : alpha * sum;
            scale = std::fabs((double)alpha) * scale + std::fabs((double)beta * (double)old);
            const double err = std::fabs((double)got[i] - (double)z);
            if (!(err <= tol * scale + 1e-37)) ++bad[slot];
            if (scale > 0.0) worstOf[slot] = std::max(worstOf[slot], err / scale);
            else if (err > 0.0) worstOf[slot] = INFINITY;
        }
    });
    int64_t total = 0;
    double w = 0.0;
    for (size_t t = 0; t < bad.size(); ++t) {
        total += bad[t];
        w = std::max(w, worstOf[t]);
    }
    if (worst != nullptr) *worst = w;
    return total;
}

// Compact row-major B (ldb = n), C_old and got (ldc = n).
int64_t oracle_check_spmm_f32(const int32_t *row_ptr, const int32_t *col_ind, const float *val, const float *B,
                              const float *c_old, const float *got, int64_t m, int64_t n, float alpha, float beta,
                              double tol, int threads, double *worst)
{
    std::vector<int64_t> bad((size_t)std::max(threads, 1), 0);
    std::vector<double> worstOf((size_t)std::max(threads, 1), 0.0);
    const int64_t chunk = threads > 1 ? (m + threads - 1) / threads : m;
    ParallelRows(m, threads, [&](int64_t lo, int64_t hi) {
        const size_t slot = chunk > 0 ? (size_t)(lo / chunk) : 0;
        std::vector<float> acc((size_t)n);
        std::vector<double> scale((size_t)n);
        for (int64_t r = lo; r < hi; ++r) {
            std::fill(acc.begin(), acc.end(), 0.0f);
            std::fill(scale.begin(), scale.end(), 0.0);
            for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                const float v = val[p];
                const float *brow = B + (int64_t)col_ind[p] * n;
                for (int64_t j = 0; j < n; ++j) {
                    acc[j] += v * brow[j];
                    scale[j] += std::fabs((double)v * (double)brow[j]);
                }
            }
            for (int64_t j = 0; j < n; ++j) {
                const float old = beta != 0.0f ? c_old[r * n + j] : 0.0f;
                const float z = beta != 0.0f ? alpha * acc[j] + beta * old : alpha * acc[j];
                const double sc = std::fabs((double)alpha) * scale[j] + std::fabs((double)beta * (double)old);
                const double err = std::fabs((double)got[r * n + j] - (double)z);
                if (!(err <= tol * sc + 1e-37)) ++bad[slot];
                if (sc > 0.0) worstOf[slot] = std::max(worstOf[slot], err / sc);
                else if (err > 0.0) worstOf[slot] = INFINITY;
            }
        }
    });
    int64_t total = 0;
    double w = 0.0;
    for (size_t t = 0; t < bad.size(); ++t) {
        total += bad[t];
        w = std::max(w, worstOf[t]);
    }
    if (worst != nullptr) *worst = w;
    return total;
}

// ---- verifiers --------------------------------------------------------------------------

// Mixed tolerance of the SpMV harness: pass when at least `ratio` of the elements satisfy
// |got - gold| <= atol + rtol * |gold| and the largest absolute error is <= limit.
// Returns 0 on pass, 1 on fail; writes {matched ratio, max abs error} to stats.
int oracle_verify_mixed(const float *gold, const float *got, int64_t n, float rtol, float atol, float limit,
                        float ratio, float *stats)
{
    int64_t pass = 0;
    float maxErr = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        const float err = std::fabs(got[i] - gold[i]);
        maxErr = std::max(maxErr, err);
        if (err <= atol + rtol * std::fabs(gold[i])) ++pass;
    }
    const float matched = n ? (float)pass / (float)n : 1.0f;
    if (stats) {
        stats[0] = matched;
        stats[1] = maxErr;
    }
    // NaN in maxErr must fail: written as !(<=)
    return (matched < ratio || !(maxErr <= limit)) ? 1 : 0;
}

// MERE / MARE of the SpMM harness over the m x n window of C.
// stats = {mean relative error, max relative error, max abs error}; relative error uses |gold| + 1e-7.
int oracle_verify_mere_mare(const float *got, const float *gold, int64_t m, int64_t n, int64_t ldc, int c_row_major,
                            double mere_thr, double mare_thr, double *stats)
{
    double sum = 0.0, mare = 0.0, mae = 0.0;
    bool bad = false;
    for (int64_t r = 0; r < m; ++r)
        for (int64_t j = 0; j < n; ++j) {
            const int64_t i = c_row_major ? r * ldc + j : j * ldc + r;
            const double diff = std::fabs((double)got[i] - (double)gold[i]);
            const double rel = diff / (std::fabs((double)gold[i]) + 1e-7);
            if (!(rel == rel)) bad = true;
            sum += rel;
            mare = std::max(mare, rel);
            mae = std::max(mae, diff);
        }
    const double mere = (m * n) ? sum / (double)(m * n) : 0.0;
    if (stats) {
        stats[0] = mere;
        stats[1] = mare;
        stats[2] = mae;
    }
    return (!bad && mere < mere_thr && mare < mare_thr) ? 0 : 1;
}

// arch22 rule: an element is an error when both |diff| > abs_tol and |diff| / max(|gold|, 1e-6) > rel_tol.
int64_t oracle_verify_abs_and_rel(const float *got, const float *gold, int64_t count, float rel_tol, float abs_tol)
{
    int64_t errors = 0;
    for (int64_t i = 0; i < count; ++i) {
        const float diff = std::fabs(got[i] - gold[i]);
        const float denom = std::fmax(std::fabs(gold[i]), 1e-6f);
        if (!(diff <= abs_tol) && !(diff / denom <= rel_tol)) ++errors;
    }
    return errors;
}

// SpMVOp: Z = alpha * A * X + beta * Y, one row at a time in CSR order with Priest's doubly compensated dot
// product, restated from the reference's device code (sparse/spmv_op/arch35/spmv_op_kernel.cpp:88-127 for the
// recurrence, :157-180 for the row bounds, the beta == 0 short cut and the final combination).  row_offsets is
// int32 or int64; index_base is subtracted from offsets and columns alike.  Parity of this restatement is
// unpinned: the reference code is AscendC device code that does not compile here, and its own golden
// (test/spmv_op/spmv_op_golden.h) needs Eigen, which is absent; the tests check it against an exact (fp64)
// product within the error bound the reference states for the algorithm and with the reference test table's
// criteria.
void oracle_spmv_op(const void *row_offsets, int offsets_are_64, const int32_t *col_ind, const float *val,
                    const float *x, const float *y, float *z, int64_t rows, int index_base, float alpha, float beta)
{
    auto offset = [&](int64_t i) -> int64_t {
        return offsets_are_64 ? static_cast<const int64_t *>(row_offsets)[i]
                              : (int64_t)static_cast<const int32_t *>(row_offsets)[i];
    };
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t s = offset(r) - index_base, e = offset(r + 1) - index_base;
        float hi = 0.0f, md = 0.0f, lo = 0.0f;
        for (int64_t p = s; p < e; ++p) {
            const float v = val[p], xv = x[col_ind[p] - index_base];
            const float prod = v * xv;
            const float pi = std::fmaf(v, xv, -prod);
            const float s1 = hi + prod;
            const float v1 = s1 - hi;
            const float e1 = (hi - (s1 - v1)) + (prod - v1);
            hi = s1;
            const float ee = e1 + pi;
            const float s2 = md + ee;
            const float v2 = s2 - md;
            const float e2 = (md - (s2 - v2)) + (ee - v2);
            md = s2;
            lo = lo + e2;
        }
        const float yv = beta == 0.0f ? 0.0f : y[r];
        const float corr = md + lo;
        const float step1 = std::fmaf(alpha, corr, beta * yv);
        z[r] = std::fmaf(alpha, hi, step1);
    }
}

int oracle_hardware_threads(void)
{
    const unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

}  // extern "C"
