"""GPU: aclsparseXcoo2csr against counting + prefix sum (what the reference computes,
sparse/coo2csr/arch35/coo2csr_kernel.cpp), bit-exact."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def count_and_scan(rows_idx, m, base):
    counts = np.bincount(rows_idx - base, minlength=m)[:m] if rows_idx.size else np.zeros(m, np.int64)
    out = np.zeros(m + 1, np.int64)
    out[1:] = np.cumsum(counts)
    return (out + base).astype(np.int32)


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("m,nnz,empty", [(1, 1, 0.0), (7, 30, 0.0), (1000, 5000, 0.5), (4096, 0, 0.0), (0, 0, 0.0),
                                          (300000, 2000000, 0.2), (5, 100000, 0.6)])
def test_coo2csr(pkg, handle, device, m, nnz, empty, base):
    rng = np.random.default_rng(m * 31 + nnz + base)
    if m and nnz:
        live = np.flatnonzero(rng.random(m) >= empty)
        if live.size == 0:
            live = np.array([m - 1])
        rows_idx = np.sort(rng.choice(live, size=nnz)).astype(np.int32) + base
    else:
        rows_idx = np.zeros(0, np.int32)
    want = count_and_scan(rows_idx.astype(np.int64), m, base)
    d_in = torch.from_numpy(rows_idx).to(device)
    d_out = torch.full((m + 1,), -7, dtype=torch.int32, device=device)
    from ctypes import c_void_p
    rc = pkg.lib().aclsparseXcoo2csr(handle.raw, c_void_p(d_in.data_ptr()) if nnz else None, rows_idx.size, m,
                                     c_void_p(d_out.data_ptr()), base)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy(), want)


def test_coo2csr_feeds_spmv(pkg, handle, device, oracle):
    """Triplets -> row offsets -> product: the converter's output is a valid row_ptr for aclsparseSpMV."""
    from ctypes import c_void_p
    from ops_sparse_b200 import api, synth
    rng = np.random.default_rng(3)
    lengths = synth.zipf_lengths(rng, 3000, 1.8, 2000, 12.0)
    A = synth.csr_from_lengths(rng, lengths, 5000, synth.normal)
    coo_rows = np.repeat(np.arange(A.rows, dtype=np.int32), np.diff(A.row_ptr))
    d_rows = torch.from_numpy(coo_rows).to(device)
    d_rp = torch.empty(A.rows + 1, dtype=torch.int32, device=device)
    assert pkg.lib().aclsparseXcoo2csr(handle.raw, c_void_p(d_rows.data_ptr()), int(A.nnz), A.rows,
                                       c_void_p(d_rp.data_ptr()), 0) == 0
    x = rng.standard_normal(A.cols).astype(np.float32)
    y = rng.standard_normal(A.rows).astype(np.float32)
    M = api.CsrMatrix(d_rp, torch.from_numpy(A.col_ind).to(device), torch.from_numpy(A.values).to(device), A.rows,
                      A.cols)
    dx, dy = api.DnVec(torch.from_numpy(x).to(device)), api.DnVec(torch.from_numpy(y).to(device))
    buf = api.spmv_preprocess(handle, M, dx, dy)
    api.spmv(handle, M, dx, dy, 2.0, -1.0, buffer=buf)
    torch.cuda.synchronize()
    gold = oracle.spmv(A.row_ptr, A.col_ind, A.values, x, y, 2.0, -1.0)
    scale = 2.0 * oracle.spmv_abs_rowsum(A.row_ptr, A.col_ind, A.values, x) + np.abs(y)
    import helpers
    helpers.assert_rowwise(dy.values.cpu().numpy().astype(np.float64), gold.astype(np.float64), scale,
                           helpers.TOL["f32"], "coo2csr -> spmv")
