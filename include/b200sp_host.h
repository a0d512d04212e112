/*
 * b200sp_host.h -- CSR SpMV / SpMM with the dense operands in HOST memory.
 *
 * y_host = alpha * A * x_host + beta * y_host   (and the same for C_host with B_host),
 * A resident on the device and analysed once.  The reference has no counterpart: its harnesses copy, compute and
 * copy back one after the other (test/spmv/arch22/spmv_test.cpp:415-479); a caller that keeps x / y (B / C) on the
 * host uses this instead of doing the same by hand.
 *
 * One call has to move x (or B) to the device, y (or C) to the device when beta != 0, and the result back.  The
 * rows of A are cut into `panels` of near-equal non-zero count, each with its own handle, descriptors, analysed
 * buffer and stream: after x / B has arrived, panel p's "old rows in -> product -> result rows out" runs while
 * panel p + 1's input and panel p - 1's output are on the bus.  The panels are plain aclsparseSpMV / aclsparseSpMM
 * calls on row slices; a panel is analysed on its own, so a row may be summed by a different kernel (and in a
 * different order) than in a call on the whole matrix: results agree within the fp32 summation tolerance.
 * A run issues a few dozen stream operations; with `use_graph` they are recorded once per set of host pointers
 * and scalars into a CUDA graph and replayed as one launch.
 *
 * Host buffers should be page-locked (cudaHostAlloc / cudaHostRegister) for the copies to overlap.
 * All functions return 0, a cudaError_t (> 0) or -(aclsparseStatus_t) (< 0).
 */
#ifndef B200SP_HOST_H_
#define B200SP_HOST_H_

#include <stddef.h>
#include <stdint.h>

#include "cann_ops_sparse.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200spHostProduct b200spHostProduct;

/* `h_row_ptr`: HOST array of rows + 1 zero-based offsets; `d_col_ind` / `d_values`: DEVICE arrays of A (borrowed,
 * must outlive the object).  n = 0: SpMV (dense operands are vectors of `cols` and `rows` elements); n > 0: SpMM
 * with row-major B (cols x n, ld = n) and C (rows x n, ld = n).  `dense_type` must equal `value_type`.
 * `d_dense` / `d_out`: device buffers for the whole x / B and y / C to stage through, or NULL to let the object
 * allocate them.  `panels` >= 1 (4 is a good default); `streams` >= 1 panel streams (3). */
int b200spHostProductCreate(b200spHostProduct **out, int64_t rows, int64_t cols, int64_t nnz,
                            const int32_t *h_row_ptr, const int32_t *d_col_ind, const void *d_values,
                            aclDataType value_type, int64_t n, aclDataType dense_type, aclDataType out_type,
                            void *d_dense, void *d_out, int panels, int streams);

/* Enqueues one product on the object's streams and returns.  alpha / beta: host scalars (float, or int32_t for
 * int32 results; NULL = 1 and 0).  `h_dense`: x / B on the host; `h_out`: the old y / C (read only when
 * beta != 0); `h_result`: where the new y / C goes (may be h_out).  use_graph != 0: record / replay a CUDA graph. */
int b200spHostProductRun(b200spHostProduct *p, const void *alpha, const void *h_dense, const void *beta,
                         const void *h_out, void *h_result, int use_graph);

/* Records an event after everything enqueued so far and makes `stream` (a cudaStream_t) wait for it. */
int b200spHostProductJoin(b200spHostProduct *p, void *stream);

/* Blocks until everything enqueued so far is done (h_result is complete). */
int b200spHostProductSynchronize(b200spHostProduct *p);

int b200spHostProductDestroy(b200spHostProduct *p);

#ifdef __cplusplus
}
#endif

#endif /* B200SP_HOST_H_ */
