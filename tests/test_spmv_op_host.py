"""CPU: argument checks and status codes of the SpMVOp plan API that return before any device work
(order and codes follow sparse/spmv_op/arch35/spmv_op_host.cpp:65-297, 496-745 of the reference), and the
oracle's restatement of the reference's compensated row sum against an exact product."""
from __future__ import annotations

from ctypes import byref, c_float, c_size_t, c_void_p

import numpy as np

FAKE = c_void_p(0x1000)  # descriptors only store pointers; nothing here dereferences them
H = c_void_p(0x10)       # a handle that is never dereferenced before the checks below return


def make(pkg, rows=6, cols=5, nnz=9, off_type=None, idx_type=None, base=0, vtype=None):
    L, S = pkg.lib(), pkg
    A = c_void_p()
    assert L.aclsparseCreateCsr(byref(A), rows, cols, nnz, FAKE, FAKE, FAKE,
                                S.ACL_SPARSE_INDEX_32I if off_type is None else off_type,
                                S.ACL_SPARSE_INDEX_32I if idx_type is None else idx_type, base,
                                S.ACL_FLOAT if vtype is None else vtype) == 0
    return A


def vec(pkg, n, vtype=None, values=FAKE):
    d = c_void_p()
    assert pkg.lib().aclsparseCreateDnVec(byref(d), n, values, pkg.ACL_FLOAT if vtype is None else vtype) == 0
    return d


def test_buffer_size_checks(pkg):
    L, S = pkg.lib(), pkg
    A, x, y = make(pkg), vec(pkg, 5), vec(pkg, 6)
    size = c_size_t(123)
    N, T = S.ACL_SPARSE_OP_NON_TRANSPOSE, S.ACL_SPARSE_OP_TRANSPOSE
    f = L.aclsparseSpMVOp_bufferSize
    assert f(None, N, A, x, y, y, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert f(H, T, A, x, y, y, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert f(H, N, A, x, y, y, S.ACL_FLOAT16, 0, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert f(H, N, None, x, y, y, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert f(H, N, A, x, y, y, S.ACL_FLOAT, 7, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert f(H, N, A, x, y, y, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    # opA / computeType are looked at before matA, matA before alg, alg before the out-pointer
    assert f(H, T, None, x, y, y, S.ACL_FLOAT, 7, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert f(H, N, None, x, y, y, S.ACL_FLOAT, 7, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    for alg, want_zero in ((S.ACL_SPARSE_SPMVOP_ALG_DEFAULT, True), (S.ACL_SPARSE_SPMVOP_ALG1, True),
                           (S.ACL_SPARSE_SPMVOP_ALG2, False)):
        assert f(H, N, A, x, y, y, S.ACL_FLOAT, alg, byref(size)) == 0
        assert (size.value == 0) == want_zero
        if not want_zero:
            assert size.value >= 4 * 6  # one int32 per row at least
    # matrix kinds: fp16 values, 64-bit column indices are refused; 64-bit row offsets and base 1 are fine
    for kw, want in ((dict(vtype=S.ACL_FLOAT16), S.ACL_SPARSE_STATUS_NOT_SUPPORTED),
                     (dict(idx_type=S.ACL_SPARSE_INDEX_64I), S.ACL_SPARSE_STATUS_NOT_SUPPORTED),
                     (dict(off_type=S.ACL_SPARSE_INDEX_64I), 0), (dict(base=1), 0)):
        B = make(pkg, **kw)
        assert f(H, N, B, x, y, y, S.ACL_FLOAT, 0, byref(size)) == want
        L.aclsparseDestroySpMat(B)
    big = make(pkg, rows=(1 << 31), cols=5, nnz=0)
    assert f(H, N, big, x, y, y, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    for d, kill in ((big, L.aclsparseDestroySpMat), (A, L.aclsparseDestroySpMat), (x, L.aclsparseDestroyDnVec),
                    (y, L.aclsparseDestroyDnVec)):
        assert kill(d) == 0


def test_descr_plan_life_cycle_and_execute_checks(pkg):
    L, S = pkg.lib(), pkg
    N = S.ACL_SPARSE_OP_NON_TRANSPOSE
    A, x, y, z = make(pkg), vec(pkg, 5), vec(pkg, 6), vec(pkg, 6)
    D, P = c_void_p(), c_void_p()
    mk = L.aclsparseSpMVOp_createDescr
    assert mk(None, byref(D), N, A, x, y, z, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert mk(H, None, N, A, x, y, z, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert mk(H, byref(D), N, None, x, y, z, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert mk(H, byref(D), N, A, x, y, z, S.ACL_FLOAT, 9, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    # ALG2 needs its workspace; the check comes before opA / computeType
    assert mk(H, byref(D), S.ACL_SPARSE_OP_TRANSPOSE, A, x, y, z, S.ACL_FLOAT, S.ACL_SPARSE_SPMVOP_ALG2,
              None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert mk(H, byref(D), S.ACL_SPARSE_OP_TRANSPOSE, A, x, y, z, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert mk(H, byref(D), N, A, x, y, z, S.ACL_INT32, 0, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    odd = make(pkg, base=3)
    assert mk(H, byref(D), N, odd, x, y, z, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert D.value is None
    assert mk(H, byref(D), N, A, x, y, z, S.ACL_FLOAT, S.ACL_SPARSE_SPMVOP_ALG1, None) == 0 and D.value

    plan = L.aclsparseSpMVOp_createPlan
    assert plan(None, D, byref(P), None, 0) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert plan(H, None, byref(P), None, 0) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert plan(H, D, None, None, 0) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert plan(H, D, byref(P), FAKE, 0) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED   # no epilogue modules
    assert plan(H, D, byref(P), None, 8) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert plan(H, D, byref(P), None, 0) == 0 and P.value

    sud = L.aclsparseSpMVOp_setGlobalUserData
    assert sud(None, P, b"k", None, 0) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert sud(H, None, b"k", None, 0) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert sud(H, P, b"k", FAKE, 0) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert sud(H, P, b"k", None, 4) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert sud(H, P, b"k", FAKE, 4) == 0 and sud(H, P, None, None, 0) == 0

    one = c_float(1.0)
    a = b = c_void_p(__import__("ctypes").addressof(one))
    run = L.aclsparseSpMVOp
    assert run(None, P, a, b, x, y, z) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert run(H, None, a, b, x, y, z) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(H, P, None, b, x, y, z) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(H, P, a, None, x, y, z) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(H, P, a, b, None, y, z) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(H, P, a, b, x, None, z) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(H, P, a, b, x, y, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    xh = vec(pkg, 5, S.ACL_FLOAT16)
    assert run(H, P, a, b, xh, y, z) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED

    assert L.aclsparseSpMVOp_destroyPlan(P) == 0 and L.aclsparseSpMVOp_destroyPlan(None) == 0
    assert L.aclsparseSpMVOp_destroyDescr(D) == 0 and L.aclsparseSpMVOp_destroyDescr(None) == 0
    for d in (x, y, z, xh):
        assert L.aclsparseDestroyDnVec(d) == 0
    for d in (A, odd):
        assert L.aclsparseDestroySpMat(d) == 0


def test_oracle_compensated_rows_against_an_exact_product(oracle):
    """The reference states |result - exact| <= 2 eps |exact| per row for its compensated dot product; the
    final alpha / beta combination adds two more roundings.  Ill-conditioned rows included."""
    rng = np.random.default_rng(5)
    rows, cols = 400, 700
    lengths = rng.integers(0, 300, rows)
    lengths[:5] = (0, 1, 2, 3, 5000)
    rp = np.zeros(rows + 1, np.int64)
    rp[1:] = np.cumsum(lengths)
    ci = rng.integers(0, cols, rp[-1]).astype(np.int32)
    val = (rng.standard_normal(rp[-1]) * 10.0 ** rng.integers(-3, 4, rp[-1])).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    y = rng.standard_normal(rows).astype(np.float32)
    eps = 2.0 ** -24
    for alpha, beta in ((1.0, 0.0), (1.5, -0.5), (0.0, 2.0), (-3.0, 1.0)):
        z = oracle.spmv_op(rp, ci, val, x, y, alpha, beta).astype(np.float64)
        exact, mag = oracle.spmv_exact(rp, ci, val, x, y, alpha, beta)
        bound = 4 * eps * (np.abs(exact) + np.abs(beta * y.astype(np.float64))) + 64 * eps * eps * abs(alpha) * mag * np.maximum(lengths, 1) + 1e-45
        assert np.all(np.abs(z - exact) <= bound), (alpha, beta, np.max(np.abs(z - exact) / bound))
    # int32 offsets, index base 1: same bits
    z0 = oracle.spmv_op(rp, ci, val, x, y, 1.5, -0.5)
    z1 = oracle.spmv_op((rp + 1).astype(np.int32), ci + 1, val, x, y, 1.5, -0.5, index_base=1)
    assert np.array_equal(z0.view(np.uint32), z1.view(np.uint32))
    # beta == 0 never reads y
    zn = oracle.spmv_op(rp, ci, val, x, np.full(rows, np.nan, np.float32), 2.0, 0.0)
    assert np.all(np.isfinite(zn))
