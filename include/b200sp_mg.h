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

/* ---- replication of x / B by peer stores (one process per GPU, all on one box) -------------------------
 *
 * Each rank creates an exchange (one cudaMalloc'ed region: `replicas` copies of the whole `bytes`-byte operand
 * plus arrival flags), exports a 64-byte handle, gathers the handles of all ranks by whatever means the job
 * has (torch.distributed, MPI, a file) and imports them.  A step is then ONE kernel per rank:
 * b200spMgPush copies the rank's slice into the same offset of the chosen replica on every rank, publishes
 * `seq` in this rank's flag on every rank and, for the ranks named in wait_mask, waits until their flags have
 * reached `seq` too.  What follows in the stream reads a complete local replica (b200spMgExchangeReplica).
 * Use two replicas in turn and a sequence number that grows by one per step.
 * Waits are bounded: when one runs out (about two seconds of SM clock unless changed) the kernel sets an error
 * word and returns; b200spMgExchangeError reads it.  All functions return 0 or a cudaError_t. */
#define B200SP_MG_MAX_RANKS 16
#define B200SP_MG_MAX_REPLICAS 4
#define B200SP_MG_HANDLE_BYTES 64

typedef struct b200spMgExchange b200spMgExchange;

int b200spMgExchangeCreate(b200spMgExchange **out, int rank, int world, size_t bytes, int replicas);
/* Writes this rank's B200SP_MG_HANDLE_BYTES-byte handle. */
int b200spMgExchangeExport(b200spMgExchange *ex, void *handle);
/* `handles`: world x B200SP_MG_HANDLE_BYTES bytes in rank order (the own entry is ignored).  Maps the peers'
 * regions into this process; the devices must be able to access each other (NVLink / PCIe peer access). */
int b200spMgExchangeImport(b200spMgExchange *ex, const void *handles);
/* Device pointer of local replica `replica` (256-byte aligned), or NULL. */
void *b200spMgExchangeReplica(b200spMgExchange *ex, int replica);
/* `src` (device, 16-byte aligned), `offset` and `bytes` multiples of 16 with offset + bytes <= the operand size;
 * bytes may be 0 (the rank only publishes and waits).  wait_mask: bit p set = wait for rank p. */
int b200spMgPush(b200spMgExchange *ex, int replica, const void *src, size_t offset, size_t bytes, uint32_t seq,
                 uint32_t wait_mask, void *stream);
/* The wait alone, as a kernel of its own. */
int b200spMgWait(b200spMgExchange *ex, int replica, uint32_t seq, uint32_t wait_mask, void *stream);
/* Limit of every later wait, in SM clock cycles. */
int b200spMgExchangeSetWaitLimit(b200spMgExchange *ex, long long sm_cycles);
/* 1 when a wait ran out since creation / the last clear, 0 when none did, -1 when the word cannot be read.
 * Synchronises the device. */
int b200spMgExchangeError(b200spMgExchange *ex);
int b200spMgExchangeClearError(b200spMgExchange *ex);
/* Synchronises the device, unmaps the peers' regions and frees the own one.  Every rank must have stopped
 * pushing before any rank destroys its exchange. */
int b200spMgExchangeDestroy(b200spMgExchange *ex);

#ifdef __cplusplus
}
#endif

#endif /* B200SP_MG_H_ */
