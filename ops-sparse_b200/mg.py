"""Multi-GPU mode: A is cut into contiguous row blocks of near-equal non-zero count, one
per rank (one process per GPU); x (SpMV) or B (SpMM) is replicated before every product;
y / C stay row-sharded, so nothing is communicated after the product.

The reference library is single-device, so this layer has no counterpart there; it sits
above the aclsparse API and uses one handle and one set of descriptors per rank.
Replication comes in three forms (`replicate=` of the sharded operators):
  "peer"            the operand is held sharded (rank r owns slice r: the y of the previous product of a
                    solver, the C of the previous layer of a graph network) and every rank stores its slice
                    into every rank's replica with the library's own kernel over CUDA-IPC peer mappings
                    (b200spMgPush: one launch per step, no library collective);
  "nccl-allgather"  the same exchange as torch.distributed.all_gather_into_tensor;
  "nccl-broadcast"  rank `src` holds the whole operand and broadcasts it (torch.distributed.broadcast).
`torch.distributed` carries the set-up (handle exchange) and the NCCL forms; gloo in CPU tests of the
partition / slice bookkeeping.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_int, c_int32, c_int64, c_longlong, c_size_t, c_uint32, c_void_p

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


def slice_cuts(n: int, parts: int, align: int = 1) -> np.ndarray:
    """Cuts (parts + 1 entries) of a length-n operand into near-equal slices whose starts are multiples of
    `align` elements (so that every slice starts on a 16-byte boundary when align = 16 / itemsize)."""
    if parts < 1 or n < 0 or align < 1:
        raise ValueError("slice_cuts: parts >= 1, n >= 0, align >= 1")
    cuts = np.zeros(parts + 1, dtype=np.int64)
    for g in range(1, parts):
        c = (n * g // parts) // align * align
        cuts[g] = max(c, cuts[g - 1])
    cuts[parts] = n
    return cuts


class _DeviceView:
    """Raw device memory as something torch.as_tensor understands (the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerExchange:
    """All-gather of a dense operand held in slices, one per rank, into a complete local replica on every rank:
    the library's push kernel over peer mappings (include/b200sp_mg.h).  `shape` / `dtype` describe the WHOLE
    operand; slices are taken along dimension 0.  Two replicas are used in turn."""

    REPLICAS = 2

    def __init__(self, shape, dtype, device, group=None):
        import torch
        import torch.distributed as dist
        from . import lib

        self.L = lib()
        self._declare(self.L)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.shape, self.dtype, self.device = tuple(shape), dtype, device
        item = torch.empty(0, dtype=dtype).element_size()
        row_bytes = item * int(np.prod(self.shape[1:], dtype=np.int64)) if len(self.shape) > 1 else item
        self.nbytes = row_bytes * self.shape[0]
        if self.nbytes % 16 != 0:
            raise ValueError("PeerExchange: the operand's size in bytes must be a multiple of 16")
        align = 1
        while (align * row_bytes) % 16 != 0:
            align *= 2
        self.cuts = slice_cuts(self.shape[0], self.world, align)
        self.row_bytes = row_bytes
        self._ex = c_void_p()
        with torch.cuda.device(device):
            rc = self.L.b200spMgExchangeCreate(byref(self._ex), self.rank, self.world, self.nbytes, self.REPLICAS)
            if rc != 0:
                raise RuntimeError(f"b200spMgExchangeCreate failed (cuda error {rc})")
            if self.world > 1:
                mine = (ctypes.c_ubyte * 64)()
                rc = self.L.b200spMgExchangeExport(self._ex, mine)
                if rc != 0:
                    raise RuntimeError(f"b200spMgExchangeExport failed (cuda error {rc})")
                gathered = [None] * self.world
                dist.all_gather_object(gathered, bytes(mine), group=group)
                blob = (ctypes.c_ubyte * (64 * self.world)).from_buffer_copy(b"".join(gathered))
                rc = self.L.b200spMgExchangeImport(self._ex, blob)
                if rc != 0:
                    raise RuntimeError(f"b200spMgExchangeImport failed (cuda error {rc}): the GPUs of this job "
                                       "cannot map each other's memory")
        self.replicas = []
        for r in range(self.REPLICAS):
            ptr = self.L.b200spMgExchangeReplica(self._ex, r)
            flat = torch.as_tensor(_DeviceView(ptr, self.nbytes), device=device)
            self.replicas.append(flat.view(dtype).view(self.shape))
        self.seq = 0

    @staticmethod
    def _declare(L):
        L.b200spMgExchangeCreate.argtypes = [POINTER(c_void_p), c_int, c_int, c_size_t, c_int]
        L.b200spMgExchangeExport.argtypes = [c_void_p, c_void_p]
        L.b200spMgExchangeImport.argtypes = [c_void_p, c_void_p]
        L.b200spMgExchangeReplica.argtypes = [c_void_p, c_int]
        L.b200spMgExchangeReplica.restype = c_void_p
        L.b200spMgPush.argtypes = [c_void_p, c_int, c_void_p, c_size_t, c_size_t, c_uint32, c_uint32, c_void_p]
        L.b200spMgWait.argtypes = [c_void_p, c_int, c_uint32, c_uint32, c_void_p]
        L.b200spMgExchangeSetWaitLimit.argtypes = [c_void_p, c_longlong]
        L.b200spMgExchangeError.argtypes = [c_void_p]
        L.b200spMgExchangeClearError.argtypes = [c_void_p]
        L.b200spMgExchangeDestroy.argtypes = [c_void_p]

    def my_rows(self) -> tuple[int, int]:
        return int(self.cuts[self.rank]), int(self.cuts[self.rank + 1])

    def gather(self, my_slice, stream=None) -> int:
        """Enqueues one exchange step on `stream` (default: torch's current stream): this rank's slice
        (rows my_rows() of the operand, on the device, contiguous) goes to every rank and the kernel returns
        once every rank's slice has arrived here.  Returns the index of the replica that is complete after it."""
        import torch

        r0, r1 = self.my_rows()
        if my_slice.shape[0] != r1 - r0 or not my_slice.is_contiguous():
            raise ValueError("PeerExchange.gather: the slice must be this rank's contiguous rows of the operand")
        self.seq += 1
        replica = self.seq % self.REPLICAS
        st = c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)
        mask = (1 << self.world) - 1
        rc = self.L.b200spMgPush(self._ex, replica, c_void_p(my_slice.data_ptr()), r0 * self.row_bytes,
                                 (r1 - r0) * self.row_bytes, self.seq, mask, st)
        if rc != 0:
            raise RuntimeError(f"b200spMgPush failed (cuda error {rc})")
        return replica

    def broadcast(self, whole, src: int = 0, stream=None) -> int:
        """One-to-all form: rank `src` stores the whole operand into every rank's replica; the others only wait."""
        import torch

        self.seq += 1
        replica = self.seq % self.REPLICAS
        st = c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)
        if self.rank == src:
            rc = self.L.b200spMgPush(self._ex, replica, c_void_p(whole.data_ptr()), 0, self.nbytes, self.seq, 0, st)
        else:
            rc = self.L.b200spMgWait(self._ex, replica, self.seq, 1 << src, st)
        if rc != 0:
            raise RuntimeError(f"peer broadcast failed (cuda error {rc})")
        return replica

    def error(self) -> int:
        return int(self.L.b200spMgExchangeError(self._ex))

    def close(self) -> None:
        import torch.distributed as dist

        if self._ex:
            self.replicas = []
            if dist.is_initialized() and self.world > 1:
                dist.barrier(group=self.group)  # no rank unmaps while another may still be storing
            self.L.b200spMgExchangeDestroy(self._ex)
            self._ex = c_void_p()


class _Sharded:
    """What the two sharded operators share: the replication of the dense operand before the product."""

    def _setup_replication(self, dense, replicate, group, src):
        import torch.distributed as dist

        self.group, self.src, self.replicate = group, src, replicate
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.exchange = None
        if self.world > 1 and replicate == "peer":
            self.exchange = PeerExchange(dense.shape, dense.dtype, dense.device, group)
            r0, r1 = self.exchange.my_rows()
            self.my_slice = dense[r0:r1].clone()  # this rank's shard of the operand (what a caller would own)
        elif self.world > 1 and replicate == "nccl-allgather":
            cuts = slice_cuts(dense.shape[0], self.world)
            if len(set(np.diff(cuts).tolist())) != 1:
                raise ValueError("nccl-allgather needs equal slices: rows of the operand divisible by the ranks")
            self.my_slice = dense[int(cuts[self.rank]):int(cuts[self.rank + 1])].clone()

    def _replicate(self, dense_full):
        """Brings the dense operand up to date on this rank; returns the tensor index to multiply with
        (0 = the caller's full-size buffer, 1 + r = replica r of the peer exchange)."""
        import torch.distributed as dist

        if self.world == 1:
            return 0
        if self.replicate == "peer":
            return 1 + self.exchange.gather(self.my_slice)
        if self.replicate == "nccl-allgather":
            dist.all_gather_into_tensor(dense_full, self.my_slice, group=self.group)
            return 0
        broadcast_(dense_full, self.src, self.group)
        return 0

    def replication_error(self) -> int:
        return self.exchange.error() if self.exchange is not None else 0

    def products(self, alpha, beta, count: int) -> None:
        """`count` local products without an exchange, against the operand as the last exchange left it, issued
        by the library's compiled loop (include/b200sp_bench.h): what a step costs when nothing is replicated."""
        import torch

        spmm = hasattr(self, "Bs")
        dense = (self.Bs if spmm else self.xs)[getattr(self, "_last", 0)]
        out = self.C if spmm else self.y
        api, L = self.api, self.api.lib()
        ct = api._compute_type(self.A.values, out.values)
        a_c, b_c = (ctypes.c_int32(int(alpha)), ctypes.c_int32(int(beta))) if ct == api.ACL_INT32 else \
            (ctypes.c_float(alpha), ctypes.c_float(beta))
        with torch.cuda.device(out.values.device):
            if spmm:
                rc = L.b200spRepeatSpMM(self.handle.raw, 0, 0, byref(a_c), self.A.raw, dense.raw, byref(b_c), out.raw, ct,
                                        0, api._ptr(self.buffer), int(count))
            else:
                rc = L.b200spRepeatSpMV(self.handle.raw, 0, byref(a_c), self.A.raw, dense.raw, byref(b_c), out.raw, ct, 0,
                                        api._ptr(self.buffer), int(count))
        if rc != 0:
            raise RuntimeError(f"compiled product loop returned status {rc}")

    def _compiled_steps(self, alpha, beta, count, spmm: bool) -> bool:
        """`count` steps (exchange + product) issued by the library's compiled loop (include/b200sp_bench.h)
        instead of one Python call per launch; only for the peer exchange.  Returns False when not applicable."""
        import torch

        if self.exchange is None or count <= 0:
            return False
        ex, L, api = self.exchange, self.exchange.L, self.api
        r0, r1 = ex.my_rows()
        dense = self.Bs if spmm else self.xs
        descrs = (c_void_p * ex.REPLICAS)(*[d.raw for d in dense[1:]])
        out = self.C if spmm else self.y
        ct = api._compute_type(self.A.values, out.values)
        a_c, b_c = ctypes.c_float(alpha), ctypes.c_float(beta)
        if ct == api.ACL_INT32:
            a_c, b_c = ctypes.c_int32(int(alpha)), ctypes.c_int32(int(beta))
        head = (ex._ex, c_void_p(self.my_slice.data_ptr()), r0 * ex.row_bytes, (r1 - r0) * ex.row_bytes, ex.seq + 1,
                ex.REPLICAS, (1 << ex.world) - 1, self.handle.raw)
        tail = (byref(a_c), self.A.raw, descrs, byref(b_c), out.raw, ct, 0, api._ptr(self.buffer), int(count))
        with torch.cuda.device(ex.device):
            rc = L.b200spMgRepeatSpMM(*head, 0, 0, *tail) if spmm else L.b200spMgRepeatSpMV(*head, 0, *tail)
        if rc != 0:
            raise RuntimeError(f"compiled step loop returned status {rc}")
        ex.seq += int(count)
        self._last = 1 + ex.seq % ex.REPLICAS
        return True


class ShardedSpmv(_Sharded):
    """One rank's share of y = alpha * A x + beta * y.

    `row_ptr / col_ind / values` are this rank's rows (slice_csr output) as torch CUDA
    tensors; `x` is a full-length device vector that `step()` brings up to date before the local
    product (see the module docstring for the forms); `y` holds only this rank's rows.
    """

    def __init__(self, row_ptr, col_ind, values, cols: int, x, y, group=None, src: int = 0,
                 replicate: str = "nccl-broadcast"):
        from . import api

        self.api = api
        self.handle = api.Handle()
        self.A = api.CsrMatrix(row_ptr, col_ind, values, row_ptr.numel() - 1, cols)
        self.x, self.y = api.DnVec(x), api.DnVec(y)
        self.buffer = api.spmv_preprocess(self.handle, self.A, self.x, self.y)
        self._setup_replication(x, replicate, group, src)
        self.xs = [self.x] + ([api.DnVec(t) for t in self.exchange.replicas] if self.exchange is not None else [])

    def step(self, alpha: float, beta: float, broadcast: bool = True) -> None:
        which = self._replicate(self.x.values) if broadcast else getattr(self, "_last", 0)
        self._last = which
        self.api.spmv(self.handle, self.A, self.xs[which], self.y, alpha, beta, buffer=self.buffer)

    def steps(self, alpha: float, beta: float, count: int) -> None:
        """`count` steps with the exchange; through the compiled loop where the peer exchange is in use."""
        if not self._compiled_steps(alpha, beta, count, spmm=False):
            for _ in range(count):
                self.step(alpha, beta)

    def close(self) -> None:
        if self.exchange is not None:
            self.exchange.close()
        self.handle.close()


class ShardedSpmm(_Sharded):
    """One rank's share of C = alpha * A B + beta * C (B replicated before the product, C row-sharded)."""

    def __init__(self, row_ptr, col_ind, values, cols: int, B, C, group=None, src: int = 0,
                 replicate: str = "nccl-broadcast"):
        from . import api

        self.api = api
        self.handle = api.Handle()
        self.A = api.CsrMatrix(row_ptr, col_ind, values, row_ptr.numel() - 1, cols)
        self.B, self.C = api.DnMat.row_major(B), api.DnMat.row_major(C)
        self.buffer = api.spmm_preprocess(self.handle, self.A, self.B, self.C)
        self._setup_replication(B, replicate, group, src)
        self.Bs = [self.B] + ([api.DnMat.row_major(t) for t in self.exchange.replicas]
                              if self.exchange is not None else [])

    def step(self, alpha: float, beta: float, broadcast: bool = True) -> None:
        which = self._replicate(self.B.values) if broadcast else getattr(self, "_last", 0)
        self._last = which
        self.api.spmm(self.handle, self.A, self.Bs[which], self.C, alpha, beta, buffer=self.buffer)

    def steps(self, alpha: float, beta: float, count: int) -> None:
        """`count` steps with the exchange; through the compiled loop where the peer exchange is in use."""
        if not self._compiled_steps(alpha, beta, count, spmm=True):
            for _ in range(count):
                self.step(alpha, beta)

    def close(self) -> None:
        if self.exchange is not None:
            self.exchange.close()
        self.handle.close()
