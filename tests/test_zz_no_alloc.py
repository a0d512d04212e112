"""GPU: the SpMV entry point for callers that cannot allocate device memory.

`b200sp_spmv_f32_noalloc` keeps its tile table, counters and partial sums in an array that is
part of the library image on the device, so a caller that is only handed pointers (code under a
framework allocator that owns all memory, a solver with a frozen memory budget) can still get a
product.  The test calls it through the C ABI twice in a row on different inputs -- the second
call finds the first call's contents in the shared array -- and compares each result with the
regular path (aclsparseSpMV with a Preprocess'ed buffer).  It also checks that an oversized
matrix is refused before anything is launched.  The file name sorts last so a run that stops at
the first failure has already been through every other test.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _fn(pkg):
    f = pkg.lib().b200sp_spmv_f32_noalloc
    f.restype = c_int
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_float,
                  c_void_p]
    return f


def _case(seed, rows, cols, device):
    from ops_sparse_b200 import synth
    rng = np.random.default_rng(seed)
    lengths = synth.zipf_lengths(rng, rows, 1.8, min(cols, 9000), 24.0)
    lengths[rng.random(rows) < 0.1] = 0
    A = synth.csr_from_lengths(rng, lengths, cols, synth.normal)
    x = rng.standard_normal(cols).astype(np.float32)
    y = rng.standard_normal(rows).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return A, x, y, dev(A.row_ptr), dev(A.col_ind), dev(A.values), dev(x)


def test_matches_regular_path_on_two_calls_in_a_row(pkg, handle, device, oracle):
    from ops_sparse_b200 import api
    noalloc = _fn(pkg)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, rows, cols, alpha, beta in ((1, 30000, 20000, 1.5, 0.5), (2, 9000, 50000, -0.75, 0.0)):
        A, x, y, d_rp, d_ci, d_v, d_x = _case(seed, rows, cols, device)
        # regular path
        dA = api.CsrMatrix(d_rp, d_ci, d_v, rows, cols)
        dx, dy = api.DnVec(d_x), api.DnVec(torch.from_numpy(y).to(device))
        buf = api.spmv_preprocess(handle, dA, dx, dy)
        api.spmv(handle, dA, dx, dy, alpha, beta, buffer=buf)
        # entry point under test: inputs and output only, no handle, no buffer
        y2 = torch.from_numpy(y).to(device)
        rc = noalloc(c_void_p(d_rp.data_ptr()), c_void_p(d_ci.data_ptr()), c_void_p(d_v.data_ptr()),
                     c_void_p(d_x.data_ptr()), c_void_p(y2.data_ptr()), rows, cols, A.nnz, alpha, beta, stream)
        assert rc == 0
        torch.cuda.synchronize()
        want = dy.values.cpu().numpy().astype(np.float64)
        got = y2.cpu().numpy().astype(np.float64)
        scale = abs(alpha) * oracle.spmv_abs_rowsum(A.row_ptr, A.col_ind, A.values, x) + np.abs(beta * y)
        helpers.assert_rowwise(got, want, scale, helpers.TOL["f32"], f"noalloc vs regular path, seed {seed}")
        gold = oracle.spmv(A.row_ptr, A.col_ind, A.values, x, y, alpha, beta)
        helpers.assert_rowwise(got, gold, scale, helpers.TOL["f32"], f"noalloc vs oracle, seed {seed}")


def test_refuses_a_matrix_beyond_its_fixed_scratch(pkg, device):
    noalloc = _fn(pkg)
    one = torch.zeros(4, dtype=torch.int32, device=device)
    f = torch.zeros(4, dtype=torch.float32, device=device)
    p = lambda t: c_void_p(t.data_ptr())
    too_many = (1 << 26) + 1  # rows + nnz beyond B200SP_NOALLOC_MAX_ITEMS: refused before any launch
    rc = noalloc(p(one), p(one), p(f), p(f), p(f), 1, 1, too_many, 1.0, 0.0, None)
    assert rc != 0
    torch.cuda.synchronize()  # the context is still healthy
    assert float(f.sum().item()) == 0.0


def test_unaligned_arrays_and_empty_matrix(pkg, device, oracle):
    """col_ind / val that start one element past a 16-byte boundary take the scalar-load form of the kernel;
    a matrix without entries must still give y = beta * y."""
    noalloc = _fn(pkg)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    A, x, y, d_rp, d_ci, d_v, d_x = _case(3, 12000, 15000, device)
    shifted_ci = torch.empty(A.nnz + 1, dtype=torch.int32, device=device)
    shifted_v = torch.empty(A.nnz + 1, dtype=torch.float32, device=device)
    shifted_ci[1:].copy_(d_ci)
    shifted_v[1:].copy_(d_v)
    assert shifted_ci[1:].data_ptr() % 16 == 4
    y2 = torch.from_numpy(y).to(device)
    rc = noalloc(c_void_p(d_rp.data_ptr()), c_void_p(shifted_ci[1:].data_ptr()), c_void_p(shifted_v[1:].data_ptr()),
                 c_void_p(d_x.data_ptr()), c_void_p(y2.data_ptr()), A.rows, A.cols, A.nnz, 2.0, -0.5, stream)
    assert rc == 0
    torch.cuda.synchronize()
    gold = oracle.spmv(A.row_ptr, A.col_ind, A.values, x, y, 2.0, -0.5)
    scale = 2.0 * oracle.spmv_abs_rowsum(A.row_ptr, A.col_ind, A.values, x) + np.abs(0.5 * y)
    helpers.assert_rowwise(y2.cpu().numpy().astype(np.float64), gold, scale, helpers.TOL["f32"], "noalloc, unaligned")

    rows = 5000
    zero_rp = torch.zeros(rows + 1, dtype=torch.int32, device=device)
    pad = torch.zeros(4, dtype=torch.float32, device=device)
    y3 = torch.from_numpy(y[:rows].copy()).to(device)
    rc = noalloc(c_void_p(zero_rp.data_ptr()), c_void_p(zero_rp.data_ptr()), c_void_p(pad.data_ptr()),
                 c_void_p(d_x.data_ptr()), c_void_p(y3.data_ptr()), rows, A.cols, 0, 1.0, 0.25, stream)
    assert rc == 0
    torch.cuda.synchronize()
    np.testing.assert_array_equal(y3.cpu().numpy(), (np.float32(0.25) * y[:rows]).astype(np.float32))
    rc = noalloc(c_void_p(zero_rp.data_ptr()), c_void_p(zero_rp.data_ptr()), c_void_p(pad.data_ptr()),
                 c_void_p(d_x.data_ptr()), c_void_p(y3.data_ptr()), 0, A.cols, 0, 1.0, 0.25, stream)
    assert rc == 0  # no rows: nothing to do, nothing launched
    torch.cuda.synchronize()
