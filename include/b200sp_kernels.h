/*
 * b200sp_kernels.h -- inner C-ABI between the aclsparse host layer and the sm_100a kernels.
 *
 * The reference keeps its host code and its device code in separate translation units
 * joined by plain extern "C" launchers that take raw device pointers, a small POD
 * "tiling" struct and a stream:
 *   spmv_kernel_do(...)      sparse/spmv/arch22/spmv_host.cpp:29-34
 *   spmm_kernel_launch(...)  sparse/spmm/arch35/spmm_host.cpp:29-33
 * The functions below are the B200 counterparts of those two launchers plus the
 * analysis passes that fill the caller's workspace.  No C++ or torch types cross this
 * boundary; a foreign-language binding can call it directly with device pointers.
 *
 * Every function returns 0 on success or the cudaError_t of the failing runtime call.
 * Unless stated otherwise nothing here allocates, frees or synchronises: work is
 * enqueued on `stream` (a cudaStream_t passed as void*, NULL = default stream).
 */
#ifndef B200SP_KERNELS_H_
#define B200SP_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types understood by the kernels (value, vector and output types). */
typedef enum b200spType_t {
    B200SP_F32 = 0,
    B200SP_F16 = 1,
    B200SP_BF16 = 2,
    B200SP_I32 = 3,
    B200SP_I8 = 4
} b200spType_t;

/* alpha / beta as the kernels take them.  When a *_dev pointer is non-NULL the kernel
 * reads the scalar from device memory (DEVICE pointer mode); otherwise the host copy of
 * the matching compute type is used. */
typedef struct b200spScalars {
    float alpha_f;
    float beta_f;
    int32_t alpha_i;
    int32_t beta_i;
    const void *alpha_dev;
    const void *beta_dev;
} b200spScalars;

/* ------------------------------------------------------------------ SpMV ------------- */

/* Bytes of workspace the SpMV analysis needs for a rows x cols matrix with nnz entries
 * (enough for either kind of plan below). */
size_t b200sp_spmv_plan_bytes(int64_t rows, int64_t cols, int64_t nnz);
/* Bytes a tile plan alone needs (what a per-call analysis with plan_info == NULL writes). */
size_t b200sp_spmv_tile_plan_bytes(int64_t rows, int64_t nnz);

/* Ints of plan_info that b200sp_spmv_analyze writes and b200sp_spmv_launch reads. */
#define B200SP_SPMV_PLAN_INFO_INTS 8

/* Analysis pass, two kinds:
 *  plan_info == NULL : tile plan.  Splits the merged (row-end, nnz) sequence of the CSR matrix into
 *      equal tiles and writes the tile table plus zeroed arrival counters into `plan`.  Nothing
 *      synchronises.  b200sp_spmv_launch then runs the merge-path tile kernel.
 *  plan_info != NULL : binned plan.  B200SP_SPMV_PLAN_INFO_INTS ints are written to it: [0] kind = 1 or 2,
 *      [1] medium rows, [2] long rows, [3] lanes per short row, [4] column blocks of x and [5] columns per
 *      block (kind 2 only), [6] the length from which a row counts as long, [7] the 8192-entry segments the long rows
 *      were cut into (kind 1 runs a CTA per segment).  Rows are binned by length
 *      -- short (<= 32 entries), medium, long -- the medium and long rows are listed in `plan`, and the call
 *      synchronises `stream` once to read the counts back.  b200sp_spmv_launch then runs one kernel per
 *      non-empty bin, concurrently: lane groups over all rows for the short ones, a warp per medium row, and for
 *      the long rows either a CTA per row (kind 1) or, when there are at least 64 of them and at least 48 per
 *      column block, their column indices ascend and cols <= 2,097,152 (kind 2), CTAs that each keep a block
 *      of x (up to 32,768 columns) in shared memory and sum the pieces of all long rows that fall into it.
 *      The plan of kind 2 depends on col_ind as well as row_ptr, and on the SM count of the current device.
 * col_ind may be NULL (kind 2 is then never chosen; a tile plan does not read it).
 * Returns cudaErrorInvalidValue when plan_bytes is too small. */
int b200sp_spmv_analyze(const int32_t *row_ptr, const int32_t *col_ind, int64_t rows, int64_t cols, int64_t nnz,
                        void *plan, size_t plan_bytes, int32_t *plan_info, void *stream);

/* y = alpha * A * x + beta * y, A in CSR with int32 zero-based indices.
 * comp_type is B200SP_F32 or B200SP_I32; x has val_type; y has out_type.
 * `plan` / `plan_info` come from b200sp_spmv_analyze for the same row_ptr / rows / nnz (plan_info =
 * NULL for a tile plan).  With plan == NULL a row-group kernel that needs no workspace is used. */
int b200sp_spmv_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x, void *y,
                       int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars, int comp_type,
                       int val_type, int out_type, void *plan, const int32_t *plan_info, void *stream);

/* Longest row of A, read back to *max_len (synchronises `stream` once).  scratch4 is any 4 bytes of
 * device memory.  The analysis of the transposed product: it decides `by_nnz` below. */
int b200sp_spmv_max_row_length(const int32_t *row_ptr, int64_t rows, void *scratch4, int32_t *max_len, void *stream);

/* y = alpha * A^T * x + beta * y (y has `cols` entries).  First scales y by beta, then
 * scatters alpha * x[i] * a_ij into y[j] with atomic adds.  For 16-bit y an fp32
 * accumulator of `cols` floats in `scratch` is used (scratch_bytes >= 4 * cols).
 * by_nnz = 0: a lane group per row (best when rows are alike); by_nnz = 1: a warp per 256 consecutive
 * non-zeros, whatever their rows (a row of 16384 entries is then spread over 64 warps). */
int b200sp_spmv_trans_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *x,
                             void *y, int64_t rows, int64_t cols, int64_t nnz, const b200spScalars *scalars,
                             int comp_type, int val_type, int out_type, void *scratch, size_t scratch_bytes,
                             int by_nnz, void *stream);

/* Largest rows + nnz that b200sp_spmv_f32_noalloc accepts. */
#define B200SP_NOALLOC_MAX_ITEMS (1LL << 26)

/* y = alpha * A * x + beta * y for fp32 CSR, for callers that must not allocate device memory.
 * (No counterpart in the reference: its SpMV takes whatever workspace it needs from the handle.)
 *
 * Some callers cannot reach cudaMalloc at the moment they need a product: code that runs inside
 * a framework whose caching allocator owns all device memory and hands none back, a solver
 * loop whose memory was sized and frozen at start-up, a plug-in that is only given pointers.
 * The regular path needs a workspace from them (aclsparseSpMVGetBufferSize) or takes the 4 MiB
 * the handle allocated in aclsparseCreate.  This entry point needs neither a handle nor a buffer:
 * the tile table, arrival counters and partial sums live in an array that is part of the
 * library image in device memory (about 0.3 MB on every GPU that loads the library, held until
 * the process exits).  It calls no cudaMalloc / cudaFree and no routine that allocates.
 *
 * Limits and rules:
 *  - rows + nnz <= B200SP_NOALLOC_MAX_ITEMS; a larger matrix is refused with cudaErrorInvalidValue
 *    and a message on stderr, nothing is launched.
 *  - The first call on each device looks up the array's device address (one runtime query, with
 *    that device current).  Make that first call outside any stream capture.
 *  - Every call on a device uses the same array and rewrites it (the tile table is rebuilt and
 *    the counters are zeroed at the start of each call, so stale contents never matter).  Two
 *    calls that can overlap on the GPU -- different streams, or different host threads -- race on
 *    it: keep the calls of one device in one stream, or order them with events.
 *  - All pointers are device pointers; 16-byte aligned col_ind / val take the vector-load kernel. */
int b200sp_spmv_f32_noalloc(const int32_t *row_ptr, const int32_t *col_ind, const float *val, const float *x,
                            float *y, int64_t rows, int64_t cols, int64_t nnz, float alpha, float beta,
                            void *stream);

/* ------------------------------------------------------------------ SpMVOp ----------- */

/* Number of row-length classes the SpMVOp analysis sorts rows into (class c holds the rows whose
 * length needs c bits: 0, 1, 2-3, 4-7, ...). */
#define B200SP_SPMVOP_CLASSES 33

/* Bytes of workspace for b200sp_spmvop_analyze on a matrix of `rows` rows. */
size_t b200sp_spmvop_plan_bytes(int64_t rows);

/* Orders the rows by descending length class into `plan` (a permutation of 0..rows-1) and writes to
 * class_start[c], c = 0..B200SP_SPMVOP_CLASSES, where the rows of class (CLASSES - 1 - c) start in it
 * (class_start[CLASSES] = rows).  row_offsets is int32 or int64 (offsets_are_64).  Synchronises
 * `stream` once.  Counterpart of the reference's spmv_op_preprocess_kernel_do. */
int b200sp_spmvop_analyze(const void *row_offsets, int offsets_are_64, int64_t rows, void *plan, size_t plan_bytes,
                          int32_t *class_start, void *stream);

/* z = alpha * A * x + beta * y, fp32, doubly compensated row sums.  index_base is 0 or 1.  alpha_dev /
 * beta_dev, when not NULL, are device pointers that replace alpha / beta.  With plan == NULL every row
 * gets the same number of lanes (chosen from nnz / rows); with a plan from b200sp_spmvop_analyze each
 * length class gets its own.  z may be y.  Counterpart of the reference's spmv_op_kernel_do. */
int b200sp_spmvop_launch(const void *row_offsets, int offsets_are_64, const int32_t *col_ind, const float *val,
                         const float *x, const float *y, float *z, int64_t rows, int64_t nnz, int index_base,
                         float alpha, float beta, const float *alpha_dev, const float *beta_dev, const void *plan,
                         const int32_t *class_start, void *stream);

/* z = beta * y (beta == 0: zeros, y not read).  Counterpart of spmv_op_beta_y_kernel_do. */
int b200sp_spmvop_scale(const float *y, float *z, int64_t rows, float beta, const float *beta_dev, void *stream);

/* ------------------------------------------------------------------ SpMM ------------- */

/* Dense operand layout, same meaning as the reference's SpmmTilingData
 * (sparse/spmm/arch35/spmm.h:49-61): ld in elements, order 0 = row-major, 1 = column-major,
 * op_b 0 = N, 1 = T. */
typedef struct b200spSpmmShape {
    int64_t m;          /* rows of A and C            */
    int64_t k;          /* cols of A                  */
    int64_t n;          /* cols of C                  */
    int64_t nnz;
    int64_t ldb;
    int64_t ldc;
    int32_t order_b;
    int32_t order_c;
    int32_t op_b;
    int32_t kahan;      /* 1 = compensated fp32 accumulation */
    int32_t block_units; /* from b200sp_spmm_analyze_blocks: units of the column-block path, 0 = not in use */
    int32_t long_rows;  /* from b200sp_spmm_analyze_blocks: rows the analysis listed as long */
} b200spSpmmShape;

/* Bytes of workspace for the SpMM analysis + long-row partial sums. */
size_t b200sp_spmm_plan_bytes(int64_t rows, int64_t nnz, int64_t n);

/* Analysis pass: finds rows too long for one warp, cuts them into segments and writes
 * the segment table into `plan`.  This call synchronises `stream` once to read back
 * the segment count (4 bytes), returned in *segments. */
int b200sp_spmm_analyze(const int32_t *row_ptr, int64_t rows, int64_t nnz, int64_t n, void *plan,
                        size_t plan_bytes, int32_t *segments, void *stream);

/* Second, optional analysis pass, after b200sp_spmm_analyze on the same plan: decides whether the long rows are
 * better summed block by block of B (B much larger than L2, rows of B of `b_row_bytes` >= 512 bytes, every long
 * row's columns ascending, partial rows within the plan's budget) and, if so, writes every long row's cut
 * positions and a table of work units into the plan.  Reads col_ind, so the plan then depends on it too.
 * *block_units = the number of units (0 = keep the segments), *long_rows = the number of long rows.
 * Synchronises `stream` twice. */
int b200sp_spmm_analyze_blocks(const int32_t *row_ptr, const int32_t *col_ind, int64_t rows, int64_t cols,
                               int64_t nnz, int64_t n, int64_t b_row_bytes, void *plan, size_t plan_bytes,
                               int32_t *block_units, int32_t *long_rows, void *stream);

/* C = alpha * A * op(B) + beta * C.  val_type is the type of A and B, out_type of C.
 * `plan` / `segments` come from b200sp_spmm_analyze on the same row_ptr / rows / nnz / n. */
int b200sp_spmm_launch(const int32_t *row_ptr, const int32_t *col_ind, const void *val, const void *B, void *C,
                       const b200spSpmmShape *shape, const b200spScalars *scalars, int val_type, int out_type,
                       void *plan, int32_t segments, void *stream);

/* 1 when a wait on the copy engine ran out of time in the SpMM row-stream kernel since the library was
 * loaded or the flag was last cleared (the affected rows of C were then not written), 0 when none did, -1 when
 * the flag cannot be read.  Synchronises the device.  Callers that need certainty poll it after synchronising. */
int b200sp_spmm_stream_error(void);
/* Clears that flag (synchronises the device).  aclsparseSpMMPreprocess also reads and clears it and returns
 * ACL_SPARSE_STATUS_EXECUTION_FAILED when it was set: a caller that never polls still learns of a product that
 * was cut short at its next analysis. */
int b200sp_spmm_stream_error_clear(void);
/* For tests of that path: later row-stream launches wait at most wait_cycles SM clocks on a copy barrier
 * (0 = the default, about a second) and expect extra_tx bytes more than they copy on every barrier, so that with
 * extra_tx > 0 every wait runs out: the kernel must set the flag, stop writing C and return.  (0, 0) restores the
 * normal behaviour.  Not thread-safe; nothing faults or hangs in either setting. */
void b200sp_spmm_stream_wait_test(long long wait_cycles, unsigned extra_tx);

/* Number of streaming multiprocessors of the current device (cached after the first call). */
int b200sp_sm_count(void);

/* Kernels this library has launched in the calling process so far (every analysis, SpMV and SpMM
 * kernel counts one).  A benchmark reads it before and after a timed region. */
unsigned long long b200sp_kernel_launches(void);
/* Used by the library's own launch sites to keep that count. */
void b200sp_note_launches(int n);

#ifdef __cplusplus
}
#endif

#endif /* B200SP_KERNELS_H_ */
