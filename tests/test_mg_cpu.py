"""CPU: the multi-GPU layer's host logic -- nnz-balanced row partition, row slicing, and the
broadcast / shard bookkeeping with two gloo ranks (the device product is replaced by the
oracle inside this test only; the product path itself has no CPU implementation)."""
from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_partition_balances_nnz(pkg):
    from ops_sparse_b200 import mg, synth
    A = synth.config2(rows=1 << 15)["A"]
    for parts in (1, 2, 4, 8):
        cuts = mg.partition_rows(A.row_ptr, parts)
        assert cuts[0] == 0 and cuts[-1] == A.rows and np.all(np.diff(cuts) >= 0)
        per = np.array([A.row_ptr[cuts[g + 1]] - A.row_ptr[cuts[g]] for g in range(parts)])
        assert per.sum() == A.nnz
        # no part exceeds its fair share by more than one (longest) row
        assert per.max() <= A.nnz / parts + A.lengths().max()
        assert abs(mg.imbalance(A.row_ptr, cuts) - per.max() * parts / A.nnz) < 1e-12


def test_partition_edge_cases(pkg):
    from ops_sparse_b200 import mg
    empty = np.zeros(11, np.int32)  # 10 empty rows
    cuts = mg.partition_rows(empty, 4)
    assert cuts[0] == 0 and cuts[-1] == 10 and np.all(np.diff(cuts) >= 0)
    one = np.array([0, 1000], np.int32)  # a single row cannot be split
    assert list(mg.partition_rows(one, 3)) == [0, 0, 0, 1] or list(mg.partition_rows(one, 3))[-1] == 1
    with pytest.raises(ValueError):
        mg.partition_rows(np.array([0, 1], np.int32), 0)
    more_parts_than_rows = mg.partition_rows(np.array([0, 2, 4], np.int32), 8)
    assert more_parts_than_rows[-1] == 2 and np.all(np.diff(more_parts_than_rows) >= 0)


def test_slices_reassemble(pkg, oracle):
    from ops_sparse_b200 import mg, synth
    c = synth.config2(rows=4096)
    A = c["A"]
    full = oracle.spmv(A.row_ptr, A.col_ind, A.values, c["x"], c["y"], 1.5, 0.5)
    cuts = mg.partition_rows(A.row_ptr, 3)
    parts = []
    for g in range(3):
        r0, r1 = mg.local_rows(cuts, g)
        rp, ci, v = mg.slice_csr(A.row_ptr, A.col_ind, A.values, r0, r1)
        assert rp[0] == 0 and rp[-1] == ci.size == v.size
        parts.append(oracle.spmv(rp, ci, v, c["x"], c["y"][r0:r1], 1.5, 0.5))
    assert np.array_equal(np.concatenate(parts), full)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    oracle = entry.load_oracle()
    from ops_sparse_b200 import mg, synth

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = synth.config2(seed=21, rows=6000)  # every rank draws the same matrix from the same seed
        A = c["A"]
        cuts = mg.partition_rows(A.row_ptr, world)
        r0, r1 = mg.local_rows(cuts, rank)
        rp, ci, v = mg.slice_csr(A.row_ptr, A.col_ind, A.values, r0, r1)
        # x lives on rank 0 only; the other ranks start from garbage and receive it by broadcast
        x = torch.from_numpy(c["x"].copy()) if rank == 0 else torch.full((A.cols,), float("nan"))
        mg.broadcast_(x, src=0)
        y_local = oracle.spmv(rp, ci, v, x.numpy(), c["y"][r0:r1], c["alpha"], c["beta"])
        # SpMM flavour: B replicated, C sharded
        B = torch.from_numpy(np.random.default_rng(5).standard_normal((A.cols, 8)).astype(np.float32)) if rank == 0 \
            else torch.zeros(A.cols, 8)
        mg.broadcast_(B, src=0)
        C_local = oracle.spmm_f32(rp, ci, v, B.numpy(), np.zeros((r1 - r0, 8), np.float32), 1.0, 0.0)
        # all-gather form: x is held in slices, one per rank (slice_cuts), and gathered into a full copy
        xc = mg.slice_cuts(A.cols, world, 4)
        assert xc[0] == 0 and xc[-1] == A.cols
        mine = torch.from_numpy(c["x"][int(xc[rank]):int(xc[rank + 1])].copy())
        gathered = torch.full((A.cols,), float("nan"))
        if len(set(np.diff(xc).tolist())) == 1:
            dist.all_gather_into_tensor(gathered, mine)
        else:
            parts = [torch.empty(int(xc[g + 1] - xc[g])) for g in range(world)]
            dist.all_gather(parts, mine)
            gathered = torch.cat(parts)
        assert np.array_equal(gathered.numpy(), c["x"])
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), y=y_local, C=C_local, rows=np.array([r0, r1]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo(pkg, oracle, tmp_path):
    import torch.multiprocessing as mp
    from ops_sparse_b200 import synth

    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    c = synth.config2(seed=21, rows=6000)
    A = c["A"]
    full_y = oracle.spmv(A.row_ptr, A.col_ind, A.values, c["x"], c["y"], c["alpha"], c["beta"])
    B = np.random.default_rng(5).standard_normal((A.cols, 8)).astype(np.float32)
    full_C = oracle.spmm_f32(A.row_ptr, A.col_ind, A.values, B, np.zeros((A.rows, 8), np.float32), 1.0, 0.0)
    got = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    assert got[0]["rows"][0] == 0 and got[0]["rows"][1] == got[1]["rows"][0] and got[1]["rows"][1] == A.rows
    assert np.array_equal(np.concatenate([g["y"] for g in got]), full_y)
    assert np.array_equal(np.concatenate([g["C"] for g in got]), full_C)


def test_slice_cuts(pkg):
    from ops_sparse_b200 import mg
    for n, parts, align in ((1 << 20, 8, 4), (1000, 3, 4), (10, 3, 4), (7, 8, 1), (0, 4, 4), (2097152, 8, 1)):
        cuts = mg.slice_cuts(n, parts, align)
        assert cuts.size == parts + 1 and cuts[0] == 0 and cuts[-1] == n and np.all(np.diff(cuts) >= 0)
        assert np.all(cuts[:-1] % align == 0)  # every slice starts on the alignment the push kernel needs
        if n >= parts * align:
            assert np.diff(cuts).max() - np.diff(cuts).min() <= 2 * align
    with pytest.raises(ValueError):
        mg.slice_cuts(10, 0)
