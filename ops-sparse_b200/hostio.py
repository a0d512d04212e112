"""Products whose dense operands live in host memory: y_host = alpha * A * x_host + beta * y_host (and the
same for C_host with B_host), A resident on the GPU and analysed once.

A call has to move x (or B) to the device, y (or C) to the device and the result back.  Done one after the
other those copies cost more than the product itself (config 2: 12.6 MB over PCIe against a 95 us kernel), so
the rows of A are cut into panels of near-equal non-zero count, each with its own descriptors, analysed
buffer and stream: after x / B has arrived, panel p's "y in -> product -> y out" runs while panel p + 1's
input and panel p - 1's output are on the bus (host-to-device and device-to-host copies use different
engines).  The panels are plain aclsparseSpMV / aclsparseSpMM calls on row slices.  A panel is analysed on
its own, so a row may be summed by a different kernel (and in a different order) than in a call on the whole
matrix: results agree within the fp32 summation tolerance, not bit for bit.  A step issues a few dozen
stream operations; `capture()` records them once into a CUDA graph so that a step is one launch.

The reference has no counterpart (its harnesses copy, compute and copy back in sequence:
test/spmv/arch22/spmv_test.cpp:415-479); this sits above the aclsparse API like the multi-GPU layer.
"""
from __future__ import annotations

import numpy as np
import torch

from . import mg


def aligned_cuts(row_ptr: np.ndarray, parts: int, multiple: int = 4) -> np.ndarray:
    """nnz-balanced row cuts moved forward to the next row whose offset is a multiple of `multiple`, so that
    every panel's slice of col_ind / values keeps the 16-byte alignment the vector-load kernels want."""
    cuts = mg.partition_rows(row_ptr, parts).copy()
    rows = row_ptr.size - 1
    for i in range(1, parts):
        r = int(cuts[i])
        while r < rows and int(row_ptr[r]) % multiple != 0:
            r += 1
        cuts[i] = max(r, int(cuts[i - 1]))
    cuts[parts] = rows
    return cuts


class HostOperandProduct:
    """One rank's product with host-resident dense operands, pipelined over row panels.

    `row_ptr` (numpy, offsets from 0), `d_col_ind`, `d_values` are this rank's CSR arrays (the last two on the
    device); `dense` is the device copy of x / B that step() refreshes from the host (and broadcasts from
    rank `src` when a process group is up), `out` the device copy of this rank's rows of y / C.
    """

    def __init__(self, row_ptr: np.ndarray, d_col_ind: torch.Tensor, d_values: torch.Tensor, cols: int,
                 dense: torch.Tensor, out: torch.Tensor, panels: int = 4, streams: int = 3, group=None, src: int = 0):
        self.is_spmm = dense.dim() == 2
        self.dense, self.out, self.group, self.src = dense, out, group, src
        rows = row_ptr.size - 1
        panels = max(1, min(panels, max(rows, 1)))
        self.cuts = aligned_cuts(np.ascontiguousarray(row_ptr, dtype=np.int32), panels)
        self.streams = [torch.cuda.Stream(device=dense.device) for _ in range(max(1, min(streams, panels)))]
        self.dense_ready = torch.cuda.Event()
        self.ops = []
        dev = dense.device
        for p in range(panels):
            r0, r1 = int(self.cuts[p]), int(self.cuts[p + 1])
            a, b = int(row_ptr[r0]), int(row_ptr[r1])
            rp = torch.from_numpy((row_ptr[r0:r1 + 1] - a).astype(np.int32)).to(dev)
            s = self.streams[p % len(self.streams)]
            with torch.cuda.stream(s):  # the panel's handle binds to this stream
                if self.is_spmm:
                    op = mg.ShardedSpmm(rp, d_col_ind[a:b], d_values[a:b], cols, dense, out[r0:r1])
                else:
                    op = mg.ShardedSpmv(rp, d_col_ind[a:b], d_values[a:b], cols, dense, out[r0:r1])
            self.ops.append((r0, r1, s, op))
        torch.cuda.synchronize(dev)

    def step(self, dense_h: torch.Tensor, out_h: torch.Tensor, result_h: torch.Tensor, alpha: float, beta: float,
             upload_dense: bool = True, broadcast: bool = False) -> None:
        """Enqueues one product; `result_h` holds it once every panel stream (or the device) is synchronised.
        In a multi-rank job every rank uploads x / B from its own host copy (upload_dense on all ranks), or one
        rank uploads and `broadcast` replicates it from rank `src`."""
        main = torch.cuda.current_stream()
        if upload_dense:
            self.dense.copy_(dense_h, non_blocking=True)
        if broadcast:
            mg.broadcast_(self.dense, self.src, self.group)
        self.dense_ready.record(main)
        for i, (r0, r1, s, op) in enumerate(self.ops):
            if r1 == r0:
                continue
            s.wait_event(self.dense_ready)
            with torch.cuda.stream(s):
                # beta * old is applied by the product kernel's own epilogue, so the old rows of this panel go
                # up first; the copy of panel p + 1 overlaps the product of panel p on another stream.
                if beta != 0.0:
                    self.out[r0:r1].copy_(out_h[r0:r1], non_blocking=True)
                op.step(alpha, beta, broadcast=False)
                result_h[r0:r1].copy_(self.out[r0:r1], non_blocking=True)
        for s in self.streams:
            main.wait_stream(s)

    def capture(self, dense_h: torch.Tensor, out_h: torch.Tensor, result_h: torch.Tensor, alpha: float, beta: float,
                upload_dense: bool = True) -> "torch.cuda.CUDAGraph":
        """Records one step on these (pinned) host buffers into a CUDA graph; `graph.replay()` then runs it.
        Single-process only (the broadcast of a multi-rank step is not recorded).  One ordinary step runs first
        so that everything created lazily (side streams, kernel attributes) exists before the capture."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            raise RuntimeError("capture() records no collective: use step() in multi-rank jobs")
        self.step(dense_h, out_h, result_h, alpha, beta, upload_dense)
        torch.cuda.synchronize(self.dense.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step(dense_h, out_h, result_h, alpha, beta, upload_dense)
        return graph

    def close(self) -> None:
        for _, _, _, op in self.ops:
            op.close()
        self.ops = []
