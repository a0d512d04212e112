"""Multi-GPU mode: A is cut into contiguous row blocks of near-equal non-zero count, one
per rank (one process per GPU); x (SpMV) or B (SpMM) is replicated by a broadcast from the
owning rank; y / C stay row-sharded, so nothing is communicated after the product.

The reference library is single-device, so this layer has no counterpart there; it sits
above the aclsparse API and uses one handle and one set of descriptors per rank.
`torch.distributed` carries the broadcast (NCCL over NVLink on GPUs; gloo in CPU tests of
the partition / broadcast bookkeeping).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int32, c_int64, c_void_p

import numpy as np


def partition_rows(row_ptr: np.ndarray, parts: int) -> np.ndarray:
    """Row cuts (parts + 1 entries) that balance non-zeros: cuts[g] is the first row whose
    offset reaches g * nnz / parts.  Computed by the C helper b200spMgPartitionRows."""
    from . import lib

    rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
    cuts = np.zeros(parts + 1, dtype=np.int64)
    rc = lib().b200spMgPartitionRows(rp.ctypes.data_as(c_void_p), c_int64(rp.size - 1), c_int32(parts),
                                     cuts.ctypes.data_as(ctypes.POINTER(c_int64)))
    if rc != 0:
        raise ValueError("b200spMgPartitionRows rejected its arguments")
    return cuts


def imbalance(row_ptr: np.ndarray, cuts: np.ndarray) -> float:
    """max part nnz / (nnz / parts); 1.0 is perfect balance."""
    from . import lib

    rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
    c = np.ascontiguousarray(cuts, dtype=np.int64)
    return float(lib().b200spMgImbalance(rp.ctypes.data_as(c_void_p), c_int64(rp.size - 1), c_int32(c.size - 1),
                                         c.ctypes.data_as(ctypes.POINTER(c_int64))))


def local_rows(cuts: np.ndarray, rank: int) -> tuple[int, int]:
    return int(cuts[rank]), int(cuts[rank + 1])


def slice_csr(row_ptr: np.ndarray, col_ind: np.ndarray, values: np.ndarray, r0: int, r1: int):
    """Rows [r0, r1) as their own CSR arrays: offsets rebased to 0, column indices stay global."""
    a, b = int(row_ptr[r0]), int(row_ptr[r1])
    return (row_ptr[r0:r1 + 1] - a).astype(np.int32), col_ind[a:b], values[a:b]


def broadcast_(tensor, src: int = 0, group=None, async_op: bool = False):
    """Replicates x / B in place from rank `src` (no-op without an initialised process group)."""
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.broadcast(tensor, src=src, group=group, async_op=async_op)


class ShardedSpmv:
    """One rank's share of y = alpha * A x + beta * y.

    `row_ptr / col_ind / values` are this rank's rows (slice_csr output) as torch CUDA
    tensors; `x` is a full-length device vector that `step()` refreshes by broadcast from
    `src` before the local product; `y` holds only this rank's rows.
    """

    def __init__(self, row_ptr, col_ind, values, cols: int, x, y, group=None, src: int = 0):
        from . import api

        self.api = api
        self.group, self.src = group, src
        self.handle = api.Handle()
        self.A = api.CsrMatrix(row_ptr, col_ind, values, row_ptr.numel() - 1, cols)
        self.x, self.y = api.DnVec(x), api.DnVec(y)
        self.buffer = api.spmv_preprocess(self.handle, self.A, self.x, self.y)

    def step(self, alpha: float, beta: float, broadcast: bool = True) -> None:
        if broadcast:
            broadcast_(self.x.values, self.src, self.group)
        self.api.spmv(self.handle, self.A, self.x, self.y, alpha, beta, buffer=self.buffer)

    def close(self) -> None:
        self.handle.close()


class ShardedSpmm:
    """One rank's share of C = alpha * A B + beta * C (B replicated by broadcast, C row-sharded)."""

    def __init__(self, row_ptr, col_ind, values, cols: int, B, C, group=None, src: int = 0):
        from . import api

        self.api = api
        self.group, self.src = group, src
        self.handle = api.Handle()
        self.A = api.CsrMatrix(row_ptr, col_ind, values, row_ptr.numel() - 1, cols)
        self.B, self.C = api.DnMat.row_major(B), api.DnMat.row_major(C)
        self.buffer = api.spmm_preprocess(self.handle, self.A, self.B, self.C)

    def step(self, alpha: float, beta: float, broadcast: bool = True) -> None:
        if broadcast:
            broadcast_(self.B.values, self.src, self.group)
        self.api.spmm(self.handle, self.A, self.B, self.C, alpha, beta, buffer=self.buffer)

    def close(self) -> None:
        self.handle.close()
