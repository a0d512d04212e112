// nnz-balanced 1-D row partition of a CSR matrix for the multi-GPU mode.
// The reference has no multi-device code; its closest relative is the per-core work
// split by non-zero count in sparse/spmm/arch35/spmm_csr_mat.cpp:28-66 (greedy bins over
// cores).  Across GPUs the blocks must stay contiguous (y / C are row-sharded in place),
// so the cut points are found by binary search on the row offsets instead.
#include <algorithm>

#include "b200sp_mg.h"

extern "C" {

int b200spMgPartitionRows(const int32_t *row_ptr, int64_t rows, int32_t parts, int64_t *cuts)
{
    if (row_ptr == nullptr || cuts == nullptr || parts < 1 || rows < 0) return -1;
    const int64_t nnz = static_cast<int64_t>(row_ptr[rows]) - row_ptr[0];
    if (nnz < 0) return -1;
    cuts[0] = 0;
    for (int32_t g = 1; g < parts; ++g) {
        // 128-bit product avoided: nnz < 2^31 and parts is small.
        const int64_t target = row_ptr[0] + nnz * g / parts;
        const int32_t *pos = std::lower_bound(row_ptr, row_ptr + rows + 1, target,
                                              [](int32_t v, int64_t t) { return static_cast<int64_t>(v) < t; });
        int64_t r = pos - row_ptr;
        r = std::min<int64_t>(std::max<int64_t>(r, cuts[g - 1]), rows);
        cuts[g] = r;
    }
    cuts[parts] = rows;
    return 0;
}

double b200spMgImbalance(const int32_t *row_ptr, int64_t rows, int32_t parts, const int64_t *cuts)
{
    if (row_ptr == nullptr || cuts == nullptr || parts < 1 || rows < 0) return -1.0;
    const int64_t nnz = static_cast<int64_t>(row_ptr[rows]) - row_ptr[0];
    if (nnz <= 0) return 1.0;
    int64_t worst = 0;
    for (int32_t g = 0; g < parts; ++g) {
        if (cuts[g] < 0 || cuts[g + 1] > rows || cuts[g] > cuts[g + 1]) return -1.0;
        worst = std::max<int64_t>(worst, static_cast<int64_t>(row_ptr[cuts[g + 1]]) - row_ptr[cuts[g]]);
    }
    return static_cast<double>(worst) * parts / static_cast<double>(nnz);
}

}  // extern "C"
