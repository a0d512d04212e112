"""GPU: the CSR producers (aclsparseXcoo2csr, aclsparseXcsrsort, aclsparseCsr2cscEx2), bit for bit against the
oracle's restatements of the reference's goldens (Coo2CsrGolden, csrsortGolden, Csr2CscGolden: oracle/oracle.cpp,
pinned to the reference headers by tests/test_oracle_pins.py) and against the committed fixtures those goldens
produced (tests/golden/convert.npz)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("m,nnz,empty", [(1, 1, 0.0), (7, 30, 0.0), (1000, 5000, 0.5), (4096, 0, 0.0), (0, 0, 0.0),
                                          (300000, 2000000, 0.2), (5, 100000, 0.6)])
def test_coo2csr(pkg, handle, device, oracle, m, nnz, empty, base):
    rng = np.random.default_rng(m * 31 + nnz + base)
    if m and nnz:
        live = np.flatnonzero(rng.random(m) >= empty)
        if live.size == 0:
            live = np.array([m - 1])
        rows_idx = np.sort(rng.choice(live, size=nnz)).astype(np.int32) + base
    else:
        rows_idx = np.zeros(0, np.int32)
    want = oracle.coo2csr(rows_idx, m, base)
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


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("m,n,mean_len,dups", [(1, 1, 1, False), (50, 40, 12, True), (3000, 5000, 30, False),
                                                (200, 100000, 3000, False), (20000, 300, 4, True), (64, 64, 0, False),
                                                (3, 200000, 70000, False), (5, 50, 9000, True)])
def test_csrsort(pkg, handle, device, oracle, m, n, mean_len, dups, base):
    from ctypes import byref, c_size_t, c_void_p
    L = pkg.lib()
    rng = np.random.default_rng(m + 7 * n + base)
    lengths = rng.poisson(mean_len, size=m).astype(np.int64) if mean_len else np.zeros(m, np.int64)
    if not dups:
        lengths = np.minimum(lengths, n)
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    nnz = int(rp[-1])
    cols = [rng.integers(0, n, size=int(k)) if dups else rng.permutation(n)[:int(k)] for k in lengths]
    ci = (np.concatenate(cols) if nnz else np.zeros(0)).astype(np.int32) + base
    rp = rp + base
    want_ci, want_p = oracle.csrsort(rp, ci, np.arange(nnz, dtype=np.int32), base)

    d_rp, d_ci = torch.from_numpy(rp).to(device), torch.from_numpy(ci).to(device)
    d_p = torch.arange(nnz, dtype=torch.int32, device=device)
    descr = c_void_p()
    assert L.aclsparseCreateMatDescr(byref(descr)) == 0
    L.aclsparseSetMatIndexBase(descr, base)
    size = c_size_t()
    ptr = lambda t: c_void_p(t.data_ptr()) if t.numel() else None
    assert L.aclsparseXcsrsort_bufferSizeExt(handle.raw, m, n, nnz, ptr(d_rp), ptr(d_ci), byref(size)) == 0
    assert (size.value >= 8 * nnz) if nnz else size.value == 0
    buf = torch.empty(max(size.value, 1), dtype=torch.uint8, device=device)
    assert L.aclsparseXcsrsort(handle.raw, m, n, nnz, descr, ptr(d_rp), ptr(d_ci), ptr(d_p), ptr(buf)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(d_ci.cpu().numpy(), want_ci)
    assert np.array_equal(d_p.cpu().numpy(), want_p)     # stable: equal columns keep their order
    assert np.array_equal(d_rp.cpu().numpy(), rp)        # untouched
    assert L.aclsparseDestroyMatDescr(descr) == 0


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("n,dups", [(200, True), (70000, False), (1 << 25, False), (2**31 - 2, False)])
def test_csrsort_every_tier_boundary(pkg, handle, device, oracle, n, dups, base):
    """Rows whose lengths sit on every boundary of the segmented sort (one key per lane, 2 / 4 / 8 keys per lane,
    the CTA radix sort in shared memory, the same in global memory), with column ranges that need one to four
    radix passes, duplicates (stability) and a permutation P that is not the identity."""
    from ctypes import byref, c_size_t, c_void_p
    L = pkg.lib()
    rng = np.random.default_rng(n % 1000 + base)
    lengths = np.array([0, 1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 511, 2047, 2048, 2049,
                        4097, 9000, 5, 0, 64, 33, 256, 2048], dtype=np.int64)
    if not dups:
        lengths = np.minimum(lengths, n)
    m = lengths.size
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    nnz = int(rp[-1])
    if dups:
        cols = [rng.integers(0, n, size=int(k)) for k in lengths]
    else:  # distinct columns without materialising a permutation of n
        cols = [np.unique(rng.integers(0, n, size=int(2 * k) + 8))[:int(k)] if k else np.zeros(0, np.int64) for k in lengths]
        cols = [rng.permutation(c) for c in cols]
        assert all(c.size == k for c, k in zip(cols, lengths))
    ci = np.concatenate(cols).astype(np.int32) + base
    rp = rp + base
    p0 = rng.permutation(nnz).astype(np.int32)
    want_ci, want_p = oracle.csrsort(rp, ci, p0, base)
    d_rp, d_ci, d_p = torch.from_numpy(rp).to(device), torch.from_numpy(ci).to(device), torch.from_numpy(p0).to(device)
    descr = c_void_p()
    assert L.aclsparseCreateMatDescr(byref(descr)) == 0
    L.aclsparseSetMatIndexBase(descr, base)
    size = c_size_t()
    ptr = lambda t: c_void_p(t.data_ptr())
    assert L.aclsparseXcsrsort_bufferSizeExt(handle.raw, m, n, nnz, ptr(d_rp), ptr(d_ci), byref(size)) == 0
    buf = torch.empty(max(size.value, 1), dtype=torch.uint8, device=device)
    assert L.aclsparseXcsrsort(handle.raw, m, n, nnz, descr, ptr(d_rp), ptr(d_ci), ptr(d_p), ptr(buf)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(d_ci.cpu().numpy(), want_ci)
    assert np.array_equal(d_p.cpu().numpy(), want_p)
    assert L.aclsparseDestroyMatDescr(descr) == 0


def test_csrsort_lets_the_blocked_long_row_kernel_in(pkg, handle, device, oracle):
    """Unsorted long rows keep aclsparseSpMV on a CTA per long row; after csrsort (values gathered through P) the
    analysis cuts them at the column blocks of x, and the product is the same within tolerance."""
    from ctypes import byref, c_int32, c_int64, c_size_t, c_void_p
    from ops_sparse_b200 import api, synth
    import helpers
    L = pkg.lib()
    rng = np.random.default_rng(12)
    M, N = 600, 60000
    lengths = rng.integers(0, 10, size=M)
    lengths[rng.choice(M, 200, replace=False)] = rng.integers(1024, 4000, 200)
    A = synth.csr_from_lengths(rng, lengths, N, synth.normal)
    ci = A.col_ind.copy()
    for r in range(M):  # shuffle every row
        s, e = A.row_ptr[r], A.row_ptr[r + 1]
        ci[s:e] = rng.permutation(ci[s:e])
    x, y = rng.standard_normal(N).astype(np.float32), rng.standard_normal(M).astype(np.float32)
    gold = oracle.spmv(A.row_ptr, ci, A.values, x, y, 1.25, 0.5)
    scale = 1.25 * oracle.spmv_abs_rowsum(A.row_ptr, ci, A.values, x) + np.abs(0.5 * y)

    L.b200sp_spmv_plan_bytes.restype = c_size_t
    L.b200sp_spmv_plan_bytes.argtypes = [c_int64, c_int64, c_int64]
    L.b200sp_spmv_analyze.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]
    d_rp, d_ci = torch.from_numpy(A.row_ptr).to(device), torch.from_numpy(ci).to(device)
    d_v = torch.from_numpy(A.values).to(device)

    def kind():
        nb = L.b200sp_spmv_plan_bytes(M, N, A.nnz)
        plan = torch.empty(nb, dtype=torch.uint8, device=device)
        info = (c_int32 * 8)()  # B200SP_SPMV_PLAN_INFO_INTS
        assert L.b200sp_spmv_analyze(c_void_p(d_rp.data_ptr()), c_void_p(d_ci.data_ptr()), M, N, A.nnz,
                                     c_void_p(plan.data_ptr()), nb, info, None) == 0
        return info[0]

    def product(values):
        Mx = api.CsrMatrix(d_rp, d_ci, values, M, N)
        dx, dy = api.DnVec(torch.from_numpy(x).to(device)), api.DnVec(torch.from_numpy(y).to(device))
        buf = api.spmv_preprocess(handle, Mx, dx, dy)
        api.spmv(handle, Mx, dx, dy, 1.25, 0.5, buffer=buf)
        torch.cuda.synchronize()
        return dy.values.cpu().numpy().astype(np.float64)

    assert kind() == 1
    helpers.assert_rowwise(product(d_v), gold.astype(np.float64), scale, helpers.TOL["f32"], "unsorted")
    descr, size = c_void_p(), c_size_t()
    assert L.aclsparseCreateMatDescr(byref(descr)) == 0
    assert L.aclsparseXcsrsort_bufferSizeExt(handle.raw, M, N, A.nnz, c_void_p(d_rp.data_ptr()),
                                             c_void_p(d_ci.data_ptr()), byref(size)) == 0
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    d_p = torch.arange(A.nnz, dtype=torch.int32, device=device)
    assert L.aclsparseXcsrsort(handle.raw, M, N, A.nnz, descr, c_void_p(d_rp.data_ptr()), c_void_p(d_ci.data_ptr()),
                               c_void_p(d_p.data_ptr()), c_void_p(buf.data_ptr())) == 0
    torch.cuda.synchronize()
    assert kind() == 2
    helpers.assert_rowwise(product(d_v[d_p.long()]), gold.astype(np.float64), scale, helpers.TOL["f32"], "sorted")
    L.aclsparseDestroyMatDescr(descr)


@pytest.mark.parametrize("vt", ["f32", "f16", "bf16", "i8"])
@pytest.mark.parametrize("base,numeric", [(0, True), (1, True), (0, False)])
def test_csr2csc(pkg, handle, device, oracle, vt, base, numeric):
    """Entries of a column keep their row order (the golden drops them into their columns row by row): bit for bit."""
    from ctypes import byref, c_size_t, c_void_p
    from ops_sparse_b200 import synth
    L, S = pkg.lib(), pkg
    rng = np.random.default_rng(5 + base)
    m, n = 4000, 2500
    lengths = synth.zipf_lengths(rng, m, 1.7, 2000, 9.0)
    lengths[rng.random(m) < 0.1] = 0
    A = synth.csr_from_lengths(rng, lengths, n, synth.normal)
    nnz = A.nnz
    if vt == "i8":
        val, acl = rng.integers(-100, 100, nnz).astype(np.int8), S.ACL_INT8
    elif vt == "f32":
        val, acl = A.values.astype(np.float32), S.ACL_FLOAT
    else:
        val, acl = oracle.to_storage(A.values.astype(np.float32), vt), (S.ACL_FLOAT16 if vt == "f16" else S.ACL_BF16)
    raw = val.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[val.dtype.itemsize])
    want_cp, want_ri, want_raw = oracle.csr2csc(m, n, A.row_ptr + base, A.col_ind + base, raw, base)
    want_val = want_raw.view(val.dtype)

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    d_rp, d_ci, d_v = dev(A.row_ptr + base), dev(A.col_ind + base), dev(val.view(np.uint8).reshape(nnz, -1))
    o_v = torch.full_like(d_v, 0x5A)
    o_cp = torch.full((n + 1,), -3, dtype=torch.int32, device=device)
    o_ri = torch.full((nnz,), -3, dtype=torch.int32, device=device)
    P = lambda t: c_void_p(t.data_ptr())
    size = c_size_t()
    action = 1 if numeric else 0
    assert L.aclsparseCsr2cscEx2_bufferSize(handle.raw, m, n, nnz, None, None, None, None, None, None, acl, action, base,
                                            0, byref(size)) == 0 and size.value >= 12 * nnz
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    assert L.aclsparseCsr2cscEx2(handle.raw, m, n, nnz, P(d_v), P(d_rp), P(d_ci), P(o_v), P(o_cp), P(o_ri), acl, action,
                                 base, 0, P(buf)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(o_cp.cpu().numpy(), want_cp)
    assert np.array_equal(o_ri.cpu().numpy(), want_ri)
    got_v = o_v.cpu().numpy()
    if numeric:
        assert np.array_equal(got_v, want_val.view(np.uint8).reshape(nnz, -1))
    else:
        assert np.all(got_v == 0x5A)  # SYMBOLIC leaves cscVal alone


def test_csr2csc_every_tier_boundary(pkg, handle, device, oracle):
    """Columns whose lengths sit on every boundary of the segmented sort (see the csrsort test above): the matrix is
    the transpose of one whose ROWS have those lengths."""
    from ctypes import byref, c_size_t, c_void_p
    from ops_sparse_b200 import synth
    L, S = pkg.lib(), pkg
    rng = np.random.default_rng(77)
    lengths = np.array([0, 1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 511, 2047, 2048, 2049,
                        4097, 9000, 5, 0, 64, 33, 256, 2048], dtype=np.int64)
    n, m = lengths.size, 12000                                  # n columns of those lengths, m rows
    T = synth.csr_from_lengths(rng, lengths, m, synth.normal)   # n x m: its rows are the columns wanted
    raw_t = T.values.astype(np.float32).view(np.uint32)
    rp, ci, raw = oracle.csr2csc(n, m, T.row_ptr, T.col_ind, raw_t, 0)   # A = T^T as CSR (m x n)
    nnz = ci.size
    want_cp, want_ri, want_raw = oracle.csr2csc(m, n, rp, ci, raw, 0)
    assert np.array_equal(want_cp, T.row_ptr) and np.array_equal(want_ri, T.col_ind)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    d_rp, d_ci, d_v = dev(rp), dev(ci), dev(raw.view(np.int32))
    o_v = torch.zeros(nnz, dtype=torch.int32, device=device)
    o_cp = torch.full((n + 1,), -3, dtype=torch.int32, device=device)
    o_ri = torch.full((nnz,), -3, dtype=torch.int32, device=device)
    P = lambda t: c_void_p(t.data_ptr())
    size = c_size_t()
    assert L.aclsparseCsr2cscEx2_bufferSize(handle.raw, m, n, nnz, None, None, None, None, None, None, S.ACL_FLOAT, 1, 0,
                                            0, byref(size)) == 0
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    for _ in range(2):  # the second run finds the workspace dirty
        assert L.aclsparseCsr2cscEx2(handle.raw, m, n, nnz, P(d_v), P(d_rp), P(d_ci), P(o_v), P(o_cp), P(o_ri), S.ACL_FLOAT,
                                     1, 0, 0, P(buf)) == 0
        torch.cuda.synchronize()
        assert np.array_equal(o_cp.cpu().numpy(), want_cp)
        assert np.array_equal(o_ri.cpu().numpy(), want_ri)
        assert np.array_equal(o_v.cpu().numpy().view(np.uint32), want_raw)


def test_csr2csc_empty_matrix_and_transposed_product(pkg, handle, device, oracle):
    """nnz = 0 fills the column offsets with the base; the CSC arrays of A, read as the CSR arrays of A^T, give
    y = A^T x through the non-transposed (atomic-free) product."""
    from ctypes import byref, c_size_t, c_void_p
    from ops_sparse_b200 import api, synth
    import helpers
    L, S = pkg.lib(), pkg
    P = lambda t: c_void_p(t.data_ptr())
    cp = torch.full((8,), -1, dtype=torch.int32, device=device)
    assert L.aclsparseCsr2cscEx2(handle.raw, 5, 7, 0, None, P(cp), None, None, P(cp), None, S.ACL_FLOAT, 1, 1, 0,
                                 None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(cp.cpu().numpy(), np.ones(8, np.int32))

    rng = np.random.default_rng(8)
    m, n = 3000, 2000
    A = synth.csr_from_lengths(rng, synth.zipf_lengths(rng, m, 1.8, 1500, 10.0), n, synth.normal)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    d_rp, d_ci, d_v = dev(A.row_ptr), dev(A.col_ind), dev(A.values)
    t_rp = torch.empty(n + 1, dtype=torch.int32, device=device)
    t_ci = torch.empty(A.nnz, dtype=torch.int32, device=device)
    t_v = torch.empty(A.nnz, dtype=torch.float32, device=device)
    size = c_size_t()
    assert L.aclsparseCsr2cscEx2_bufferSize(handle.raw, m, n, A.nnz, None, None, None, None, None, None, S.ACL_FLOAT, 1, 0,
                                            0, byref(size)) == 0
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    assert L.aclsparseCsr2cscEx2(handle.raw, m, n, A.nnz, P(d_v), P(d_rp), P(d_ci), P(t_v), P(t_rp), P(t_ci), S.ACL_FLOAT,
                                 1, 0, 0, P(buf)) == 0
    x, y = rng.standard_normal(m).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    At = api.CsrMatrix(t_rp, t_ci, t_v, n, m)
    dx, dy = api.DnVec(dev(x)), api.DnVec(dev(y))
    pbuf = api.spmv_preprocess(handle, At, dx, dy)
    api.spmv(handle, At, dx, dy, 1.5, 0.5, buffer=pbuf)
    torch.cuda.synchronize()
    gold = oracle.spmv_typed(A.row_ptr, A.col_ind, A.values, x, y, 1.5, 0.5, "f32", "f32", "f32", trans=True, cols=n)
    prod = np.abs(A.values.astype(np.float64) * np.repeat(x.astype(np.float64), np.diff(A.row_ptr)))
    scale = 1.5 * np.bincount(A.col_ind, weights=prod, minlength=n)[:n] + np.abs(0.5 * y)
    helpers.assert_rowwise(dy.values.cpu().numpy().astype(np.float64), gold.astype(np.float64), scale,
                           helpers.TOL["f32"], "A^T x through csr2csc")


def test_fixtures_of_the_reference_goldens(pkg, handle, device, golden_dir):
    """tests/golden/convert.npz: outputs of the reference's own golden functions, reproduced on the device."""
    from ctypes import byref, c_size_t, c_void_p
    L, S = pkg.lib(), pkg
    z = np.load(golden_dir / "convert.npz")
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    P = lambda t: c_void_p(t.data_ptr()) if t.numel() else None
    for name in z["coo_names"]:
        for base in (0, 1):
            k = f"coo/{name}/{base}"
            rows, m = z[f"{k}/rows"], int(z[f"{k}/m"][0])
            d_in, d_out = dev(rows), torch.full((m + 1,), -7, dtype=torch.int32, device=device)
            assert L.aclsparseXcoo2csr(handle.raw, P(d_in), rows.size, m, c_void_p(d_out.data_ptr()), base) == 0
            torch.cuda.synchronize()
            assert np.array_equal(d_out.cpu().numpy(), z[f"{k}/row_ptr"]), k
    for name in z["sort_names"]:
        for base in (0, 1):
            k = f"sort/{name}/{base}"
            rp, ci, n = z[f"{k}/row_ptr"], z[f"{k}/col_ind"], int(z[f"{k}/n"][0])
            m, nnz = rp.size - 1, ci.size
            d_rp, d_ci = dev(rp), dev(ci)
            d_p = torch.arange(nnz, dtype=torch.int32, device=device)
            descr = c_void_p()
            assert L.aclsparseCreateMatDescr(byref(descr)) == 0
            L.aclsparseSetMatIndexBase(descr, base)
            size = c_size_t()
            assert L.aclsparseXcsrsort_bufferSizeExt(handle.raw, m, n, nnz, P(d_rp), P(d_ci), byref(size)) == 0
            buf = torch.empty(max(size.value, 1), dtype=torch.uint8, device=device)
            assert L.aclsparseXcsrsort(handle.raw, m, n, nnz, descr, P(d_rp), P(d_ci), P(d_p), P(buf)) == 0
            torch.cuda.synchronize()
            assert np.array_equal(d_ci.cpu().numpy(), z[f"{k}/col_out"]), k
            assert np.array_equal(d_p.cpu().numpy(), z[f"{k}/perm_out"]), k
            L.aclsparseDestroyMatDescr(descr)
    for name in z["csc_names"]:
        for base in (0, 1):
            k = f"csc/{name}/{base}"
            m, n = (int(v) for v in z[f"{k}/shape"])
            rp, ci, val = z[f"{k}/row_ptr"], z[f"{k}/col_ind"], z[f"{k}/val"]
            nnz = ci.size
            d_rp, d_ci, d_v = dev(rp), dev(ci), dev(val.view(np.int32))
            o_v = torch.zeros(max(nnz, 1), dtype=torch.int32, device=device)
            o_cp = torch.full((n + 1,), -3, dtype=torch.int32, device=device)
            o_ri = torch.full((max(nnz, 1),), -3, dtype=torch.int32, device=device)
            size = c_size_t()
            assert L.aclsparseCsr2cscEx2_bufferSize(handle.raw, m, n, nnz, None, None, None, None, None, None, S.ACL_FLOAT,
                                                    1, base, 0, byref(size)) == 0
            buf = torch.empty(max(size.value, 1), dtype=torch.uint8, device=device)
            assert L.aclsparseCsr2cscEx2(handle.raw, m, n, nnz, P(d_v), c_void_p(d_rp.data_ptr()), P(d_ci),
                                         c_void_p(o_v.data_ptr()), c_void_p(o_cp.data_ptr()),
                                         c_void_p(o_ri.data_ptr()), S.ACL_FLOAT, 1, base, 0,
                                         c_void_p(buf.data_ptr())) == 0
            torch.cuda.synchronize()
            assert np.array_equal(o_cp.cpu().numpy(), z[f"{k}/col_ptr"]), k
            assert np.array_equal(o_ri.cpu().numpy()[:nnz], z[f"{k}/row_ind"]), k
            assert np.array_equal(o_v.cpu().numpy()[:nnz].view(np.uint32), z[f"{k}/val_out"]), k


def test_csr2csc_hot_columns(pkg, handle, device, oracle):
    """Columns that almost every row touches: their segments (9000 and 5000 entries) are longer than one
    shared-memory chunk of the sort, so the chunk sort + merge passes run, with a run left over."""
    from ctypes import byref, c_size_t, c_void_p
    L, S = pkg.lib(), pkg
    rng = np.random.default_rng(77)
    m, n = 9000, 400
    rows = []
    for r in range(m):
        extra = rng.choice(np.arange(2, n), size=int(rng.integers(0, 4)), replace=False)
        cols = np.concatenate([[0], [1] if r % 9 < 5 else [], extra]).astype(np.int32)
        rows.append(np.sort(cols))
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum([c.size for c in rows])
    ci = np.concatenate(rows).astype(np.int32)
    val = rng.integers(0, 1 << 30, size=ci.size).astype(np.uint32)
    want_cp, want_ri, want_v = oracle.csr2csc(m, n, rp, ci, val, 0)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    P = lambda t: c_void_p(t.data_ptr())
    d_rp, d_ci, d_v = dev(rp), dev(ci), dev(val.view(np.int32))
    o_v, o_ri = torch.zeros_like(d_v), torch.zeros_like(d_ci)
    o_cp = torch.zeros(n + 1, dtype=torch.int32, device=device)
    size = c_size_t()
    assert L.aclsparseCsr2cscEx2_bufferSize(handle.raw, m, n, ci.size, None, None, None, None, None, None, S.ACL_FLOAT, 1,
                                            0, 0, byref(size)) == 0
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    assert L.aclsparseCsr2cscEx2(handle.raw, m, n, ci.size, P(d_v), P(d_rp), P(d_ci), P(o_v), P(o_cp), P(o_ri),
                                 S.ACL_FLOAT, 1, 0, 0, P(buf)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(o_cp.cpu().numpy(), want_cp) and np.array_equal(o_ri.cpu().numpy(), want_ri)
    assert np.array_equal(o_v.cpu().numpy().view(np.uint32), want_v)
