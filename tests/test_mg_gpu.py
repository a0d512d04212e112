"""GPU: replication of x across ranks by peer stores (include/b200sp_mg.h, ops-sparse_b200/mg.py).

One-GPU tests drive the exchange with a single rank: the push lands in the local replica, and a wait for a
sequence number nobody publishes runs out after its (shortened) limit, sets the error word and returns -- the
context stays usable, which is the failure-detection contract of every wait in this library.  The two-rank test
needs two GPUs (skipped otherwise): each rank owns a slice of x that changes every step, and the sharded SpMV
after every exchange must match the oracle on the whole vector."""
from __future__ import annotations

import os
import socket
import sys
from ctypes import c_void_p
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_single_rank_push_and_bounded_wait(pkg, device):
    from ops_sparse_b200 import mg
    ex = mg.PeerExchange((4096,), torch.float32, device)
    try:
        src = torch.arange(4096, dtype=torch.float32, device=device)
        r = ex.gather(src)
        torch.cuda.synchronize()
        assert ex.error() == 0 and torch.equal(ex.replicas[r], src)
        r2 = ex.gather(src * 2)
        torch.cuda.synchronize()
        assert r2 != r and torch.equal(ex.replicas[r2], src * 2) and torch.equal(ex.replicas[r], src)
        # a wait for a step that nobody publishes: it must give up, report, and leave the GPU usable
        assert ex.L.b200spMgExchangeSetWaitLimit(ex._ex, 1 << 22) == 0  # about two milliseconds of SM clock
        st = c_void_p(torch.cuda.current_stream().cuda_stream)
        assert ex.L.b200spMgWait(ex._ex, 0, ex.seq + 100, 1, st) == 0
        torch.cuda.synchronize()
        assert ex.error() == 1
        assert ex.L.b200spMgExchangeClearError(ex._ex) == 0 and ex.error() == 0
        r3 = ex.gather(src + 1)  # and the exchange still works afterwards
        torch.cuda.synchronize()
        assert ex.error() == 0 and torch.equal(ex.replicas[r3], src + 1)
    finally:
        ex.close()


def test_push_rejects_bad_arguments(pkg, device):
    from ops_sparse_b200 import mg
    ex = mg.PeerExchange((1024,), torch.float32, device)
    try:
        src = torch.zeros(1025, dtype=torch.float32, device=device)
        st = c_void_p(torch.cuda.current_stream().cuda_stream)
        push = ex.L.b200spMgPush
        assert push(ex._ex, 0, c_void_p(src.data_ptr()), 0, 4096 + 16, 1, 0, st) != 0      # past the operand
        assert push(ex._ex, 0, c_void_p(src.data_ptr() + 4), 0, 64, 1, 0, st) != 0          # unaligned source
        assert push(ex._ex, 0, c_void_p(src.data_ptr()), 8, 64, 1, 0, st) != 0              # unaligned offset
        assert push(ex._ex, 5, c_void_p(src.data_ptr()), 0, 64, 1, 0, st) != 0              # no such replica
        torch.cuda.synchronize()
    finally:
        ex.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    oracle = entry.load_oracle()
    from ops_sparse_b200 import mg, synth

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    try:
        c = synth.config2(seed=31, rows=40000)
        A = c["A"]
        cuts = mg.partition_rows(A.row_ptr, world)
        r0, r1 = mg.local_rows(cuts, rank)
        rp, ci, v = mg.slice_csr(A.row_ptr, A.col_ind, A.values, r0, r1)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        x_full = to(c["x"])
        y = to(c["y"][r0:r1])
        op = mg.ShardedSpmv(to(rp), to(ci), to(v), A.cols, x_full.clone(), y, replicate="peer")
        op.x.values.zero_()  # the product may only read what the exchange delivered
        s0, s1 = op.exchange.my_rows()
        x_host = c["x"].copy()
        for step in range(5):
            # every rank's slice changes every step; all ranks can compute what the whole vector must be
            x_host = (x_host * np.float32(0.5) + np.float32(step)).astype(np.float32)
            op.my_slice.copy_(to(x_host[s0:s1]))
            y.copy_(to(c["y"][r0:r1]))
            op.step(c["alpha"], c["beta"])
            torch.cuda.synchronize()
            gold = oracle.spmv(rp, ci, v, x_host, c["y"][r0:r1], c["alpha"], c["beta"])
            scale = abs(c["alpha"]) * oracle.spmv_abs_rowsum(rp, ci, v, x_host) + np.abs(c["beta"] * c["y"][r0:r1])
            err = np.abs(y.cpu().numpy().astype(np.float64) - gold)
            ok = ok and bool(np.all(err <= 1e-5 * scale + 1e-30))
        # the compiled loop: three steps with beta = 0 give the product of the last exchange, whatever ran before
        op.steps(c["alpha"], 0.0, 3)
        torch.cuda.synchronize()
        gold = oracle.spmv(rp, ci, v, x_host, c["y"][r0:r1], c["alpha"], 0.0)
        scale = abs(c["alpha"]) * oracle.spmv_abs_rowsum(rp, ci, v, x_host)
        err = np.abs(y.cpu().numpy().astype(np.float64) - gold)
        ok = ok and bool(np.all(err <= 1e-5 * scale + 1e-30)) and op.exchange.seq == 8
        ok = ok and op.replication_error() == 0
        dist.barrier()
        op.close()
    finally:
        dist.destroy_process_group()
    Path(out_dir, f"rank{rank}.ok").write_text("1" if ok else "0")


def test_two_ranks_peer_exchange(pkg, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert [Path(tmp_path, f"rank{r}.ok").read_text() for r in range(world)] == ["1", "1"]
