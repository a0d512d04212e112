"""Products whose dense operands live in host memory: y_host = alpha * A * x_host + beta * y_host (and the
same for C_host with B_host), A resident on the GPU and analysed once.

This is the Python face of the library's own entry points for that (include/b200sp_host.h,
csrc/common/host_product.cpp): the rows of A are cut into panels of near-equal non-zero count, each with its own
handle, descriptors, analysed buffer and stream, so that after x / B has arrived panel p's
"old rows in -> product -> result rows out" runs while panel p + 1's input and panel p - 1's output are on the
bus.  Nothing is computed or copied here: every copy and every kernel of a step is issued by the library, which
can also record a step into a CUDA graph so that it is one launch.  A panel is analysed on its own, so a row may
be summed by a different kernel (and in a different order) than in a call on the whole matrix: results agree
within the fp32 summation tolerance, not bit for bit.

The reference has no counterpart (its harnesses copy, compute and copy back in sequence:
test/spmv/arch22/spmv_test.cpp:415-479).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_int, c_int32, c_int64, c_void_p

import numpy as np
import torch

from . import mg


def aligned_cuts(row_ptr: np.ndarray, parts: int, multiple: int = 4) -> np.ndarray:
    """The row cuts the library uses: nnz-balanced, moved forward to the next row whose offset is a multiple of
    `multiple`, so that every panel's slice of col_ind / values keeps the 16-byte alignment the vector-load
    kernels want."""
    cuts = mg.partition_rows(row_ptr, parts).copy()
    rows = row_ptr.size - 1
    for i in range(1, parts):
        r = int(cuts[i])
        while r < rows and int(row_ptr[r]) % multiple != 0:
            r += 1
        cuts[i] = max(r, int(cuts[i - 1]))
    cuts[parts] = rows
    return cuts


class _Replay:
    """What capture() returns: replay() runs the recorded step."""

    def __init__(self, owner, args):
        self.owner, self.args = owner, args

    def replay(self) -> None:
        self.owner._run(*self.args, use_graph=True)


class HostOperandProduct:
    """One rank's product with host-resident dense operands, pipelined over row panels.

    `row_ptr` (numpy, offsets from 0), `d_col_ind`, `d_values` are this rank's CSR arrays (the last two on the
    device); `dense` and `out` are device buffers for the whole x / B and this rank's rows of y / C that the steps
    stage through (their shapes and dtypes also say what the product is).
    """

    def __init__(self, row_ptr: np.ndarray, d_col_ind: torch.Tensor, d_values: torch.Tensor, cols: int,
                 dense: torch.Tensor, out: torch.Tensor, panels: int = 4, streams: int = 3):
        from . import api, lib

        self.L = lib()
        self._declare(self.L)
        self.is_spmm = dense.dim() == 2
        self.dense, self.out = dense, out
        self._keep = (d_col_ind, d_values)
        row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
        rows = row_ptr.size - 1
        panels = max(1, min(panels, max(rows, 1)))
        self.cuts = aligned_cuts(row_ptr, panels)
        n = int(dense.shape[1]) if self.is_spmm else 0
        self.int_scalars = api._compute_type(d_values, out) == api.ACL_INT32
        self._p = c_void_p()
        with torch.cuda.device(dense.device):
            rc = self.L.b200spHostProductCreate(
                byref(self._p), rows, cols, int(d_col_ind.numel()), row_ptr.ctypes.data_as(POINTER(c_int32)),
                c_void_p(d_col_ind.data_ptr()), c_void_p(d_values.data_ptr()), api.acl_type_of(d_values.dtype), n,
                api.acl_type_of(dense.dtype), api.acl_type_of(out.dtype), c_void_p(dense.data_ptr()),
                c_void_p(out.data_ptr()), panels, max(1, min(streams, panels)))
        if rc != 0:
            raise RuntimeError(f"b200spHostProductCreate failed ({rc})")

    @staticmethod
    def _declare(L):
        P = c_void_p
        L.b200spHostProductCreate.argtypes = [POINTER(P), c_int64, c_int64, c_int64, POINTER(c_int32), P, P, c_int,
                                              c_int64, c_int, c_int, P, P, c_int, c_int]
        L.b200spHostProductRun.argtypes = [P, P, P, P, P, P, c_int]
        L.b200spHostProductJoin.argtypes = [P, P]
        L.b200spHostProductSynchronize.argtypes = [P]
        L.b200spHostProductDestroy.argtypes = [P]

    def _run(self, dense_h, out_h, result_h, alpha, beta, use_graph: bool) -> None:
        a = ctypes.c_int32(int(alpha)) if self.int_scalars else ctypes.c_float(alpha)
        b = ctypes.c_int32(int(beta)) if self.int_scalars else ctypes.c_float(beta)
        with torch.cuda.device(self.dense.device):
            rc = self.L.b200spHostProductRun(self._p, byref(a), c_void_p(dense_h.data_ptr()), byref(b),
                                             c_void_p(out_h.data_ptr()), c_void_p(result_h.data_ptr()),
                                             1 if use_graph else 0)
            if rc == 0:  # what the caller enqueues next on its stream comes after this step
                rc = self.L.b200spHostProductJoin(self._p, c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"b200spHostProductRun failed ({rc})")

    def step(self, dense_h: torch.Tensor, out_h: torch.Tensor, result_h: torch.Tensor, alpha: float, beta: float,
             upload_dense: bool = True) -> None:
        """Enqueues one product; `result_h` holds it once the device (or the caller's current stream) is
        synchronised.  The host tensors should be pinned."""
        if not upload_dense:
            raise ValueError("a step always uploads x / B: it is part of the call")
        self._run(dense_h, out_h, result_h, alpha, beta, use_graph=False)

    def capture(self, dense_h: torch.Tensor, out_h: torch.Tensor, result_h: torch.Tensor, alpha: float, beta: float,
                upload_dense: bool = True) -> _Replay:
        """Has the library record one step on these (pinned) host buffers into a CUDA graph; `replay()` of the
        returned object then runs it as one launch.  One ordinary step runs first so that everything created
        lazily (side streams, kernel attributes) exists before the recording."""
        self.step(dense_h, out_h, result_h, alpha, beta, upload_dense)
        torch.cuda.synchronize(self.dense.device)
        replay = _Replay(self, (dense_h, out_h, result_h, alpha, beta))
        replay.replay()  # records
        torch.cuda.synchronize(self.dense.device)
        return replay

    def synchronize(self) -> None:
        self.L.b200spHostProductSynchronize(self._p)

    def close(self) -> None:
        if self._p:
            self.L.b200spHostProductDestroy(self._p)
            self._p = c_void_p()
