"""Seeded synthetic CSR inputs: the five benchmark configurations and small test shapes.

No public matrix collection is used anywhere: every matrix is drawn here from a seeded
numpy generator with the shapes, row-length laws and value distributions the benchmark
configurations name.  The same arrays feed the CPU oracle and the GPU path, so both see
identical bytes.  Row-length generators follow the shapes of the reference harnesses'
own generators (fixed rows: test/spmm/arch22/spmm_test.cpp:73-92; skewed rows: :94-131;
unique sorted columns per row: test/spmv/arch22/spmv_test.cpp:72-86).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Csr:
    rows: int
    cols: int
    row_ptr: np.ndarray  # int32 [rows + 1]
    col_ind: np.ndarray  # int32 [nnz], ascending inside each row
    values: np.ndarray   # float32 [nnz] (callers round to 16 bit where the config says so)
    meta: dict = field(default_factory=dict)

    @property
    def nnz(self) -> int:
        return int(self.col_ind.size)

    def lengths(self) -> np.ndarray:
        return np.diff(self.row_ptr)

    def row_slice(self, r0: int, r1: int) -> "Csr":
        """Rows [r0, r1) as a matrix of their own (offsets rebased, columns stay global)."""
        a, b = int(self.row_ptr[r0]), int(self.row_ptr[r1])
        return Csr(r1 - r0, self.cols, (self.row_ptr[r0:r1 + 1] - a).astype(np.int32), self.col_ind[a:b],
                   self.values[a:b], dict(self.meta))


def columns_for_lengths(rng: np.random.Generator, lengths: np.ndarray, cols: int) -> np.ndarray:
    """`lengths[i]` distinct columns per row, uniform without replacement, ascending."""
    lengths = np.asarray(lengths, dtype=np.int64)
    if lengths.size and lengths.max() > cols:
        raise ValueError("a row cannot hold more distinct columns than the matrix has")
    nnz = int(lengths.sum())
    if nnz == 0:
        return np.zeros(0, dtype=np.int32)
    if cols <= 4096 or lengths.max() * 4 > cols:
        # dense-ish rows: draw each row as a partial permutation
        out = np.empty(nnz, dtype=np.int32)
        pos = 0
        for L in lengths:
            if L:
                out[pos:pos + L] = np.sort(rng.choice(cols, size=int(L), replace=False))
                pos += int(L)
        return out
    rows = np.repeat(np.arange(lengths.size, dtype=np.int64), lengths)
    key = rows * cols + rng.integers(0, cols, size=nnz, dtype=np.int64)
    while True:  # redraw collisions until every (row, column) pair is unique
        key.sort()
        dup = np.flatnonzero(key[1:] == key[:-1]) + 1
        if dup.size == 0:
            break
        key[dup] = (key[dup] // cols) * cols + rng.integers(0, cols, size=dup.size, dtype=np.int64)
    return (key % cols).astype(np.int32)


def csr_from_lengths(rng: np.random.Generator, lengths: np.ndarray, cols: int, value_fn) -> Csr:
    lengths = np.asarray(lengths, dtype=np.int64)
    row_ptr = np.zeros(lengths.size + 1, dtype=np.int64)
    np.cumsum(lengths, out=row_ptr[1:])
    if row_ptr[-1] >= 2**31:
        raise ValueError("nnz does not fit 32-bit offsets")
    col = columns_for_lengths(rng, lengths, cols)
    val = value_fn(rng, int(row_ptr[-1])).astype(np.float32)
    return Csr(int(lengths.size), int(cols), row_ptr.astype(np.int32), col, val)


def zipf_lengths(rng: np.random.Generator, rows: int, s: float, kmax: int, mean: float) -> np.ndarray:
    """Row lengths L = clamp(floor(c * k), 1, kmax), k ~ truncated Zipf P(k) ~ k^-s on [1, kmax],
    with c chosen so that the mean of c * k equals `mean`."""
    k = np.arange(1, kmax + 1, dtype=np.float64)
    w = k ** (-s)
    cdf = np.cumsum(w) / w.sum()
    ek = float((k * w).sum() / w.sum())
    draws = np.searchsorted(cdf, rng.random(rows), side="left") + 1
    return np.clip(np.floor(draws * (mean / ek)), 1, kmax).astype(np.int64)


def uniform(rng, n):
    return rng.uniform(-1.0, 1.0, size=n)


def normal(rng, n):
    return rng.standard_normal(size=n)


def fixed_rows_csr(seed: int, rows: int, cols: int, per_row: int, value_fn=uniform) -> Csr:
    rng = np.random.default_rng(seed)
    return csr_from_lengths(rng, np.full(rows, per_row, dtype=np.int64), cols, value_fn)


def stencil27_csr(seed: int, n: int) -> Csr:
    """27-point stencil on an n^3 grid, lexicographic node order, non-periodic boundary:
    centre 26.0, neighbours -1.0, every entry jittered by U(-0.01, 0.01)."""
    rng = np.random.default_rng(seed)
    N = n ** 3
    idx = np.arange(N, dtype=np.int32)
    x, y, z = idx % n, (idx // n) % n, idx // (n * n)
    cols = np.empty((N, 27), dtype=np.int32)
    valid = np.empty((N, 27), dtype=bool)
    centre = np.zeros(27, dtype=bool)
    s = 0
    for dz in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dx in (-1, 0, 1):  # ascending (dz, dy, dx) = ascending column index
                ok = ((x + dx >= 0) & (x + dx < n) & (y + dy >= 0) & (y + dy < n) & (z + dz >= 0) & (z + dz < n))
                valid[:, s] = ok
                cols[:, s] = idx + (dz * n + dy) * n + dx
                centre[s] = (dx == 0 and dy == 0 and dz == 0)
                s += 1
    lengths = valid.sum(axis=1).astype(np.int64)
    row_ptr = np.zeros(N + 1, dtype=np.int64)
    np.cumsum(lengths, out=row_ptr[1:])
    col = cols[valid]
    base = np.where(np.broadcast_to(centre, (N, 27))[valid], 26.0, -1.0)
    val = (base + rng.uniform(-0.01, 0.01, size=col.size)).astype(np.float32)
    return Csr(N, N, row_ptr.astype(np.int32), col.astype(np.int32), val, {"grid": n})


# ---------------------------------------------------------------- the five configurations

def config1(seed: int = 1) -> dict:
    """SpMV fp32, 4096 x 4096, exactly 16 nnz per row, values and x U(-1,1), alpha=1 beta=0."""
    A = fixed_rows_csr(seed, 4096, 4096, 16, uniform)
    rng = np.random.default_rng(seed + 1000)
    return {"name": "c1_spmv_f32_4096_16", "A": A, "x": uniform(rng, 4096).astype(np.float32),
            "y": uniform(rng, 4096).astype(np.float32), "alpha": 1.0, "beta": 0.0, "val": "f32", "out": "f32"}


def config2(seed: int = 2, rows: int = 1 << 20) -> dict:
    """SpMV fp32, power-law rows (Zipf s=1.8, mean 32, cap 16384), values / x / y N(0,1),
    alpha=1.5 beta=0.5.  `rows` scales the case down for tests."""
    rng = np.random.default_rng(seed)
    cap = min(16384, rows)
    A = csr_from_lengths(rng, zipf_lengths(rng, rows, 1.8, cap, 32.0), rows, normal)
    return {"name": f"c2_spmv_f32_powerlaw_{rows}", "A": A, "x": normal(rng, rows).astype(np.float32),
            "y": normal(rng, rows).astype(np.float32), "alpha": 1.5, "beta": 0.5, "val": "f32", "out": "f32"}


def config3(seed: int = 3, grid: int = 128) -> dict:
    """SpMV fp16 values and x, fp32 accumulate and y, 27-point stencil on grid^3, alpha=1 beta=0."""
    A = stencil27_csr(seed, grid)
    rng = np.random.default_rng(seed + 1000)
    return {"name": f"c3_spmv_f16_stencil27_{grid}", "A": A, "x": rng.uniform(0.0, 1.0, size=A.cols).astype(np.float32),
            "y": np.zeros(A.rows, dtype=np.float32), "alpha": 1.0, "beta": 0.0, "val": "f16", "out": "f32"}


def config4(seed: int = 4, rows: int = 1 << 18, n: int = 64) -> dict:
    """SpMM fp32, 64 nnz per row, B and C rows x n row-major N(0,1), alpha=1 beta=0.5."""
    A = fixed_rows_csr(seed, rows, rows, min(64, rows), uniform)
    rng = np.random.default_rng(seed + 1000)
    return {"name": f"c4_spmm_f32_{rows}_n{n}", "A": A, "B": rng.standard_normal((rows, n), dtype=np.float32),
            "C": rng.standard_normal((rows, n), dtype=np.float32), "alpha": 1.0, "beta": 0.5, "val": "f32",
            "out": "f32"}


def config5(seed: int = 5, rows: int = 1 << 21, n: int = 256) -> dict:
    """SpMM bf16 values and B, fp32 accumulate and C: graph adjacency with power-law degrees
    (Zipf s=2.0, mean 16, cap 65536), a_ij = 1/sqrt(deg_i * deg_j), features N(0,1), alpha=1 beta=0."""
    rng = np.random.default_rng(seed)
    cap = min(65536, rows)
    deg = zipf_lengths(rng, rows, 2.0, cap, 16.0)
    A = csr_from_lengths(rng, deg, rows, lambda r, k: np.zeros(k))
    row_of = np.repeat(np.arange(rows, dtype=np.int64), deg)
    A.values = (1.0 / np.sqrt(deg[row_of].astype(np.float64) * deg[A.col_ind].astype(np.float64))).astype(np.float32)
    return {"name": f"c5_spmm_bf16_graph_{rows}_n{n}", "A": A, "B": rng.standard_normal((rows, n), dtype=np.float32),
            "C": np.zeros((rows, n), dtype=np.float32), "alpha": 1.0, "beta": 0.0, "val": "bf16", "out": "f32"}


def algorithmic_bytes_spmv(rows: int, cols: int, nnz: int, val_bytes: int, out_bytes: int, beta: float) -> int:
    """Every input byte once + every output byte once (+ y read when beta != 0), int32 indices."""
    return 4 * (rows + 1) + (4 + val_bytes) * nnz + val_bytes * cols + out_bytes * rows * (2 if beta != 0 else 1)


def algorithmic_bytes_spmm(rows: int, cols: int, nnz: int, n: int, val_bytes: int, out_bytes: int, beta: float) -> int:
    return (4 * (rows + 1) + (4 + val_bytes) * nnz + val_bytes * cols * n
            + out_bytes * rows * n * (2 if beta != 0 else 1))
