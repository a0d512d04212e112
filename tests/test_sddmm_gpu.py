"""GPU: aclsparseSDDMM through the C ABI against an fp64 product sampled on the pattern of C (what the
reference's test golden computes, test/sddmm/sddmm_golden.h as used by test/sddmm/sddmm/arch35/sddmm_test.cpp:
162-193, with fp16 cases fed the fp16-rounded inputs and scalars).  Tolerance per entry:
tol * (|alpha| * sum_k |x_ik y_kj| + |beta c_ij|), tol = 1e-5 (fp32) or 2e-3 (fp16 storage, fp32 accumulation)
plus half an ulp of the fp16 result."""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_size_t, c_uint16, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dense_operand(rng, rows, cols, order, pad, dtype):
    """Logical rows x cols matrix stored row- or column-major with `pad` extra leading-dimension elements."""
    a = rng.uniform(-1.0, 1.0, (rows, cols)).astype(np.float32)
    if dtype == "f16":
        a = a.astype(np.float16).astype(np.float32)
    if order == "row":
        ld = cols + pad
        store = np.full((rows, ld), 7.0, np.float32)
        store[:, :cols] = a
    else:
        ld = rows + pad
        store = np.full((cols, ld), 7.0, np.float32)
        store[:, :rows] = a.T
    return a, store.reshape(-1), ld


def run_sddmm(pkg, handle, device, rp, ci, cvals, Xs, Ys, alpha, beta, m, n, opx, opy, ox, oy, dtype, device_scalars=False):
    S, L = pkg, pkg.lib()
    tdt = torch.float16 if dtype == "f16" else torch.float32
    acl = S.ACL_FLOAT16 if dtype == "f16" else S.ACL_FLOAT
    dev = lambda a, t=None: (torch.from_numpy(np.ascontiguousarray(a)).to(device) if t is None
                             else torch.from_numpy(np.ascontiguousarray(a)).to(device).to(t))
    (xs, xr, xc, ldx), (ys, yr, yc, ldy) = Xs, Ys
    d_x, d_y, d_c = dev(xs, tdt), dev(ys, tdt), dev(cvals, tdt)
    d_rp, d_ci = dev(rp), dev(ci)
    X, Y, C = c_void_p(), c_void_p(), c_void_p()
    order = lambda o: S.ACL_SPARSE_ORDER_ROW if o == "row" else S.ACL_SPARSE_ORDER_COL
    assert L.aclsparseCreateDnMat(byref(X), xr, xc, ldx, c_void_p(d_x.data_ptr()), acl, order(ox)) == 0
    assert L.aclsparseCreateDnMat(byref(Y), yr, yc, ldy, c_void_p(d_y.data_ptr()), acl, order(oy)) == 0
    assert L.aclsparseCreateCsr(byref(C), m, n, ci.size, c_void_p(d_rp.data_ptr()), c_void_p(d_ci.data_ptr()),
                                c_void_p(d_c.data_ptr()), 0, 0, 0, acl) == 0
    if device_scalars:
        keep = (torch.tensor([alpha], dtype=tdt, device=device), torch.tensor([beta], dtype=tdt, device=device))
        a, b = c_void_p(keep[0].data_ptr()), c_void_p(keep[1].data_ptr())
    elif dtype == "f16":
        keep = (c_uint16(int(np.float16(alpha).view(np.uint16))), c_uint16(int(np.float16(beta).view(np.uint16))))
        a, b = c_void_p(ctypes.addressof(keep[0])), c_void_p(ctypes.addressof(keep[1]))
    else:
        keep = (c_float(alpha), c_float(beta))
        a, b = c_void_p(ctypes.addressof(keep[0])), c_void_p(ctypes.addressof(keep[1]))
    opX = S.ACL_SPARSE_OP_TRANSPOSE if opx else S.ACL_SPARSE_OP_NON_TRANSPOSE
    opY = S.ACL_SPARSE_OP_TRANSPOSE if opy else S.ACL_SPARSE_OP_NON_TRANSPOSE
    handle.set_pointer_mode_device(device_scalars)
    try:
        size = c_size_t()
        assert L.aclsparseSDDMMBufferSize(handle.raw, opX, opY, a, X, Y, b, C, acl, 0, byref(size)) == 0 and size.value > 0
        buf = torch.empty(size.value, dtype=torch.uint8, device=device)
        assert L.aclsparseSDDMMPreprocess(handle.raw, opX, opY, a, X, Y, b, C, acl, 0, c_void_p(buf.data_ptr())) == 0
        assert L.aclsparseSDDMM(handle.raw, opX, opY, a, X, Y, b, C, acl, 0, c_void_p(buf.data_ptr())) == 0
        torch.cuda.synchronize()
    finally:
        handle.set_pointer_mode_device(False)
    out = d_c.to(torch.float32).cpu().numpy()
    for d, kill in ((X, L.aclsparseDestroyDnMat), (Y, L.aclsparseDestroyDnMat), (C, L.aclsparseDestroySpMat)):
        kill(d)
    return out


def golden(rp, ci, cvals, X, Y, alpha, beta):
    rows = np.repeat(np.arange(rp.size - 1), np.diff(rp))
    Xd, Yd = X.astype(np.float64), Y.astype(np.float64)   # X: m x k, Y: k x n (logical)
    dots = np.einsum("pk,kp->p", Xd[rows], Yd[:, ci])
    mags = np.einsum("pk,kp->p", np.abs(Xd[rows]), np.abs(Yd[:, ci]))
    c = cvals.astype(np.float64)
    return alpha * dots + beta * c, abs(alpha) * mags + np.abs(beta * c)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("opx,ox", [(False, "row"), (False, "col"), (True, "row"), (True, "col")])
@pytest.mark.parametrize("opy,oy", [(False, "row"), (False, "col"), (True, "row"), (True, "col")])
def test_ops_orders_and_padding(pkg, handle, device, dtype, opx, ox, opy, oy):
    from ops_sparse_b200 import synth
    rng = np.random.default_rng(hash((dtype, opx, ox, opy, oy)) % (1 << 31))
    m, n, k = 300, 260, 75
    lengths = synth.zipf_lengths(rng, m, 1.6, n, 12.0)
    lengths[rng.random(m) < 0.15] = 0
    A = synth.csr_from_lengths(rng, lengths, n, synth.uniform)
    cvals = A.values.astype(np.float16).astype(np.float32) if dtype == "f16" else A.values.astype(np.float32)
    X, xs, ldx = dense_operand(rng, m, k, ox, 3, dtype) if not opx else (None, None, None)
    if opx:   # stored k x m, logical op(X) = stored^T
        Xt, xs, ldx = dense_operand(rng, k, m, ox, 3, dtype)
        X, xr, xc = Xt.T, k, m
    else:
        xr, xc = m, k
    if opy:   # stored n x k
        Yt, ys, ldy = dense_operand(rng, n, k, oy, 5, dtype)
        Y, yr, yc = Yt.T, n, k
    else:
        Y, ys, ldy = dense_operand(rng, k, n, oy, 5, dtype)
        yr, yc = k, n
    alpha, beta = (1.5, -0.5)
    got = run_sddmm(pkg, handle, device, A.row_ptr, A.col_ind, cvals, (xs, xr, xc, ldx), (ys, yr, yc, ldy), alpha, beta,
                    m, n, opx, opy, ox, oy, dtype)
    want, scale = golden(A.row_ptr, A.col_ind, cvals, X, Y, alpha, beta)
    tol = 1e-5 if dtype == "f32" else 2e-3
    slack = np.abs(want) * 2.0 ** -11 if dtype == "f16" else 0.0
    assert np.all(np.abs(got - want) <= tol * scale + slack + 1e-30), np.max(np.abs(got - want) / (tol * scale + slack + 1e-30))


@pytest.mark.parametrize("k", [128, 328])  # rows of 16 / 32 / 41 / 82 sixteen-byte pieces: one per lane, or a loop
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_graph_shape_device_scalars_and_beta_zero(pkg, handle, device, dtype, k):
    """The shape of the backward step of a graph layer: X m x k row-major, Y n x k row-major used transposed;
    scalars on the device; beta = 0 must not read C (NaN in C)."""
    from ops_sparse_b200 import synth
    rng = np.random.default_rng(17)
    m = n = 5000
    A = synth.csr_from_lengths(rng, synth.zipf_lengths(rng, m, 2.0, 4000, 10.0), n, synth.uniform)
    X, xs, ldx = dense_operand(rng, m, k, "row", 0, dtype)
    Yt, ys, ldy = dense_operand(rng, n, k, "row", 0, dtype)
    nan_c = np.full(A.nnz, np.nan, np.float32)
    got = run_sddmm(pkg, handle, device, A.row_ptr, A.col_ind, nan_c, (xs, m, k, ldx), (ys, n, k, ldy), 0.75, 0.0, m, n,
                    False, True, "row", "row", dtype, device_scalars=True)
    want, scale = golden(A.row_ptr, A.col_ind, np.zeros(A.nnz, np.float32), X, Yt.T, 0.75, 0.0)
    tol = 1e-5 if dtype == "f32" else 2e-3
    slack = np.abs(want) * 2.0 ** -11 if dtype == "f16" else 0.0
    assert np.all(np.isfinite(got)) and np.all(np.abs(got - want) <= tol * scale + slack + 1e-30)


def test_fp16_result_saturates(pkg, handle, device):
    """alpha large enough to overflow fp16: +-65504, not inf (reference sddmm_kernel.cpp:424-437)."""
    rng = np.random.default_rng(2)
    m, n, k = 16, 16, 64
    rp = np.arange(m + 1, dtype=np.int32) * 2
    ci = np.tile(np.array([1, 9], np.int32), m)
    X = np.ones((m, k), np.float32)
    Y = np.ones((k, n), np.float32)
    Y[:, 9] = -1.0
    got = run_sddmm(pkg, handle, device, rp, ci, np.zeros(2 * m, np.float32), (X.reshape(-1), m, k, k),
                    (Y.reshape(-1), k, n, n), 60000.0, 0.0, m, n, False, False, "row", "row", "f16")
    assert np.array_equal(got[0::2], np.full(m, 65504.0, np.float32))
    assert np.array_equal(got[1::2], np.full(m, -65504.0, np.float32))


def test_empty_pattern_and_status_codes(pkg, handle, device):
    S, L = pkg, pkg.lib()
    t = torch.zeros(64, device=device)
    i = torch.zeros(8, dtype=torch.int32, device=device)
    P = lambda x: c_void_p(x.data_ptr())
    X, Y, C, Ch = c_void_p(), c_void_p(), c_void_p(), c_void_p()
    assert L.aclsparseCreateDnMat(byref(X), 4, 8, 8, P(t), S.ACL_FLOAT, 0) == 0
    assert L.aclsparseCreateDnMat(byref(Y), 8, 4, 4, P(t), S.ACL_FLOAT, 0) == 0
    assert L.aclsparseCreateCsr(byref(C), 4, 4, 0, P(i), None, None, 0, 0, 0, S.ACL_FLOAT) == 0
    assert L.aclsparseCreateCsr(byref(Ch), 4, 4, 0, P(i), None, None, 0, 0, 0, S.ACL_FLOAT16) == 0
    one = c_float(1.0)
    a = c_void_p(ctypes.addressof(one))
    size = c_size_t()
    N = S.ACL_SPARSE_OP_NON_TRANSPOSE
    f = L.aclsparseSDDMM
    assert L.aclsparseSDDMMBufferSize(handle.raw, N, N, a, X, Y, a, C, S.ACL_FLOAT, 0, byref(size)) == 0
    assert f(handle.raw, N, N, a, X, Y, a, C, S.ACL_FLOAT, 0, P(t)) == 0                # nothing to do
    assert f(None, N, N, a, X, Y, a, C, S.ACL_FLOAT, 0, P(t)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert f(handle.raw, N, N, a, None, Y, a, C, S.ACL_FLOAT, 0, P(t)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert f(handle.raw, 2, N, a, X, Y, a, C, S.ACL_FLOAT, 0, P(t)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED      # conj. transpose
    assert f(handle.raw, N, N, a, X, Y, a, Ch, S.ACL_FLOAT, 0, P(t)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED     # mixed types
    assert f(handle.raw, N, S.ACL_SPARSE_OP_TRANSPOSE, a, X, Y, a, C, S.ACL_FLOAT, 0, P(t)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert f(handle.raw, N, N, a, X, Y, a, C, S.ACL_FLOAT, 3, P(t)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED      # algorithm
    assert f(handle.raw, N, N, None, X, Y, a, C, S.ACL_FLOAT, 0, P(t)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert f(handle.raw, N, N, a, X, Y, a, C, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseSDDMMPreprocess(handle.raw, N, N, a, X, Y, a, C, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES
    assert L.aclsparseSDDMMBufferSize(handle.raw, N, N, a, X, Y, a, C, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    for d, kill in ((X, L.aclsparseDestroyDnMat), (Y, L.aclsparseDestroyDnMat), (C, L.aclsparseDestroySpMat),
                    (Ch, L.aclsparseDestroySpMat)):
        kill(d)


def test_fixtures_of_the_reference_golden(pkg, handle, device, oracle, golden_dir):
    """tests/golden/sddmm.npz: rows of the reference's own SDDMM case table (its pattern generator, its seeds, its
    fp64 golden with inputs quantised through fp16 where the case is fp16), judged as its test judges the device:
    golden cast to fp32 (clamped to +-65504 for fp16), then the frame's mixed tolerance (test/sddmm/sddmm/arch35/
    sddmm_test.cpp:262-292)."""
    z = np.load(golden_dir / "sddmm.npz")
    for name in z["names"]:
        m, k, n = (int(v) for v in z[f"{name}/shape"])
        alpha, beta = (float(v) for v in z[f"{name}/scalars"])
        dtype = str(z[f"{name}/dtype"][0])
        ro, ci = z[f"{name}/row_offsets"], z[f"{name}/col_ind"]
        if ci.size == 0:
            continue  # the reference test skips the value check of its empty case too
        np_t = np.float32 if dtype == "f32" else np.float16
        X = z[f"{name}/X"].astype(np.float32).astype(np_t).reshape(m, k)       # what the test uploads: fp64 -> fp32 (-> fp16)
        Yt = z[f"{name}/Yt"].astype(np.float32).astype(np_t).reshape(n, k)
        c0 = z[f"{name}/c_init"].astype(np.float32).astype(np_t).astype(np.float32)
        flat = lambda a: a.astype(np.float32).reshape(-1)
        got = run_sddmm(pkg, handle, device, ro, ci, c0, (flat(X), m, k, k), (flat(Yt), n, k, k), alpha, beta, m, n,
                        False, True, "row", "row", dtype)
        gold = z[f"{name}/gold"].astype(np.float32)
        if dtype == "f16":
            gold = np.clip(gold, -65504.0, 65504.0)
        ok, st = oracle.verify_mixed_tolerance(got, gold, dtype)
        assert ok, (name, st)
