// Exposes the reference's golden functions for the three CSR producers through a C ABI:
//   csrsortGolden   test/csrsort/arch35/csrsort_golden.h:38
//   Coo2CsrGolden   test/coo2csr/coo2csr_golden.h:44
//   Csr2CscGolden   test/csr2csc_ex2/csr2csc_ex2_golden.h:50
// The headers are compiled from where they lie (the REF_* macros are set by oracle/build_oracle.py);
// nothing of them is copied here.  TEST INFRASTRUCTURE ONLY (checker for oracle/oracle.cpp).
#include REF_CSRSORT_GOLDEN
#include REF_COO2CSR_GOLDEN
#include REF_CSR2CSC_GOLDEN

#include <cstring>

extern "C" void ref_csrsort(const int32_t *row_ptr, const int32_t *col_ind, const int32_t *perm, int m, int nnz,
                            int index_base, int32_t *col_out, int32_t *perm_out)
{
    std::vector<int32_t> rp(row_ptr, row_ptr + m + 1), ci(col_ind, col_ind + nnz), p(perm, perm + nnz);
    const sparse_test::CsrsortGoldenResult r = sparse_test::csrsortGolden(rp, ci, p, m, index_base);
    if (nnz > 0) {
        std::memcpy(col_out, r.colInd.data(), sizeof(int32_t) * (size_t)nnz);
        std::memcpy(perm_out, r.P.data(), sizeof(int32_t) * (size_t)nnz);
    }
}

extern "C" int ref_coo2csr(const int32_t *coo_row, int nnz, int m, int index_base, int32_t *row_ptr_out)
{
    std::vector<int32_t> rows(coo_row, coo_row + (nnz > 0 ? nnz : 0));
    const std::vector<int32_t> rp = sparse_test::Coo2CsrGolden(rows, nnz, m, index_base);
    if (rp.empty()) return -1;
    std::memcpy(row_ptr_out, rp.data(), sizeof(int32_t) * rp.size());
    return 0;
}

namespace {
template <typename T>
void Csr2Csc(const sparse_test::CsrMatrix &csr, const void *values, int index_base, int32_t *col_ptr, int32_t *row_ind,
             void *val_out)
{
    std::vector<T> v(static_cast<const T *>(values), static_cast<const T *>(values) + csr.nnz);
    const sparse_test::Csr2CscGoldenResult r = sparse_test::Csr2CscGolden<T>(csr, v, index_base);
    std::memcpy(col_ptr, r.cscColPtr.data(), sizeof(int32_t) * r.cscColPtr.size());
    if (csr.nnz > 0) {
        std::memcpy(row_ind, r.cscRowInd.data(), sizeof(int32_t) * (size_t)csr.nnz);
        std::memcpy(val_out, r.cscVal.data(), r.cscVal.size());
    }
}
}  // namespace

// value_bytes: 1, 2 or 4 (values are moved as raw bytes, so one instantiation per width covers every type)
extern "C" int ref_csr2csc(int m, int n, int nnz, const int32_t *row_ptr, const int32_t *col_ind, const void *values,
                           int value_bytes, int index_base, int32_t *col_ptr, int32_t *row_ind, void *val_out)
{
    sparse_test::CsrMatrix csr;
    csr.rows = m;
    csr.cols = n;
    csr.nnz = nnz;
    csr.rowOffsets.assign(row_ptr, row_ptr + m + 1);
    csr.colIndices.assign(col_ind, col_ind + nnz);
    switch (value_bytes) {
        case 1: Csr2Csc<uint8_t>(csr, values, index_base, col_ptr, row_ind, val_out); return 0;
        case 2: Csr2Csc<uint16_t>(csr, values, index_base, col_ptr, row_ind, val_out); return 0;
        case 4: Csr2Csc<uint32_t>(csr, values, index_base, col_ptr, row_ind, val_out); return 0;
        default: return -1;
    }
}
