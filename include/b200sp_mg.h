/*
 * b200sp_mg.h -- helpers for running the CSR SpMV / SpMM path on several GPUs of one box.
 *
 * The reference library is single-device (no collective or multi-device code exists in it),
 * so these entry points have no counterpart there.  They sit above the aclsparse API:
 * A is cut into contiguous row blocks of near-equal non-zero count, every GPU gets one block
 * (its own handle and descriptors), x or B is replicated, y or C stays row-sharded.
 */
#ifndef B200SP_MG_H_
#define B200SP_MG_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Row cuts for `parts` GPUs: cuts[g] is the first row r with row_ptr[r] >= g * nnz / parts,
 * cuts[0] = 0, cuts[parts] = rows.  `row_ptr` is a HOST array of rows + 1 zero-based
 * offsets.  Returns 0, or -1 on bad arguments (NULL pointers, parts < 1, rows < 0,
 * decreasing offsets at the probed positions). */
int b200spMgPartitionRows(const int32_t *row_ptr, int64_t rows, int32_t parts, int64_t *cuts);

/* Load imbalance of a partition: max over parts of the part's non-zero count divided by
 * nnz / parts (1.0 = perfect).  Returns a negative value on bad arguments. */
double b200spMgImbalance(const int32_t *row_ptr, int64_t rows, int32_t parts, const int64_t *cuts);

#ifdef __cplusplus
}
#endif

#endif /* B200SP_MG_H_ */
