"""GPU: products with host-resident dense operands, pipelined over row panels, against one call on the whole
matrix with device-resident operands (panels are analysed on their own, so a row may be summed in another
order: the comparison is within the fp32 tolerance, and bit for bit between repeated runs and graph replays)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _upload(device, A):
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return dev(A.row_ptr), dev(A.col_ind), dev(A.values)


@pytest.mark.parametrize("panels", [1, 3, 4])
@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_spmv_panels_match_one_call(pkg, handle, device, oracle, panels, beta):
    from ops_sparse_b200 import api, hostio, synth
    cfg = synth.config2(rows=1 << 15)
    A = cfg["A"]
    d_rp, d_ci, d_v = _upload(device, A)
    x_h = torch.from_numpy(cfg["x"]).pin_memory()
    y_h = torch.from_numpy(cfg["y"]).pin_memory()
    # one call, operands on the device
    M = api.CsrMatrix(d_rp, d_ci, d_v, A.rows, A.cols)
    dx, dy = api.DnVec(x_h.to(device)), api.DnVec(y_h.to(device))
    buf = api.spmv_preprocess(handle, M, dx, dy)
    api.spmv(handle, M, dx, dy, 1.5, beta, buffer=buf)
    torch.cuda.synchronize()
    want = dy.values.cpu()
    # panels, operands on the host
    x_d, y_d = torch.empty_like(x_h, device=device), torch.full_like(y_h, float("nan"), device=device)
    res_h = torch.empty_like(y_h).pin_memory()
    pipe = hostio.HostOperandProduct(A.row_ptr, d_ci, d_v, A.cols, x_d, y_d, panels=panels)
    scale = 1.5 * oracle.spmv_abs_rowsum(A.row_ptr, A.col_ind, A.values, cfg["x"]) + np.abs(beta * cfg["y"])
    first = None
    for _ in range(2):
        pipe.step(x_h, y_h, res_h, 1.5, beta)
        torch.cuda.synchronize()
        helpers.assert_rowwise(res_h.numpy().astype(np.float64), want.numpy().astype(np.float64), scale,
                               helpers.TOL["f32"], f"{panels} panels")
        first = res_h.clone() if first is None else first
        assert torch.equal(res_h.view(torch.int32), first.view(torch.int32))
    graph = pipe.capture(x_h, y_h, res_h, 1.5, beta)
    res_h.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(res_h.view(torch.int32), first.view(torch.int32))
    assert pipe.cuts[0] == 0 and pipe.cuts[-1] == A.rows and np.all(np.diff(pipe.cuts) >= 0)
    assert all(int(A.row_ptr[c]) % 4 == 0 for c in pipe.cuts[1:-1])
    pipe.close()


def test_spmm_panels_match_one_call(pkg, handle, device):
    from ops_sparse_b200 import api, hostio, synth
    cfg = synth.config4(rows=1 << 13, n=64)
    A = cfg["A"]
    d_rp, d_ci, d_v = _upload(device, A)
    B_h = torch.from_numpy(cfg["B"]).pin_memory()
    C_h = torch.from_numpy(cfg["C"]).pin_memory()
    M = api.CsrMatrix(d_rp, d_ci, d_v, A.rows, A.cols)
    dB, dC = api.DnMat.row_major(B_h.to(device)), api.DnMat.row_major(C_h.to(device))
    buf = api.spmm_preprocess(handle, M, dB, dC)
    api.spmm(handle, M, dB, dC, 1.0, 0.5, buffer=buf)
    torch.cuda.synchronize()
    want = dC.values.cpu()
    B_d, C_d = torch.empty_like(B_h, device=device), torch.empty_like(C_h, device=device)
    res_h = torch.empty_like(C_h).pin_memory()
    pipe = hostio.HostOperandProduct(A.row_ptr, d_ci, d_v, A.cols, B_d, C_d, panels=4)
    pipe.step(B_h, C_h, res_h, 1.0, 0.5)
    torch.cuda.synchronize()
    # every row has 64 entries: the lane-group kernel sums each in CSR order whatever the panel, same bits
    assert torch.equal(res_h.view(torch.int32), want.view(torch.int32))
    pipe.close()


def test_c_entry_points_allocate_their_own_staging(pkg, device, oracle):
    """include/b200sp_host.h straight through ctypes, with NULL staging buffers (the object allocates them), a
    recorded step, a second set of scalars (a second recording) and the result written over the old y."""
    import ctypes
    from ctypes import POINTER, byref, c_float, c_int, c_int32, c_int64, c_void_p
    from ops_sparse_b200 import synth, ACL_FLOAT
    L = pkg.lib()
    P = c_void_p
    L.b200spHostProductCreate.argtypes = [POINTER(P), c_int64, c_int64, c_int64, POINTER(c_int32), P, P, c_int, c_int64,
                                          c_int, c_int, P, P, c_int, c_int]
    L.b200spHostProductRun.argtypes = [P, P, P, P, P, P, c_int]
    L.b200spHostProductSynchronize.argtypes = [P]
    L.b200spHostProductDestroy.argtypes = [P]
    cfg = synth.config2(rows=1 << 14, seed=9)
    A = cfg["A"]
    _, d_ci, d_v = _upload(device, A)
    rp = np.ascontiguousarray(A.row_ptr, dtype=np.int32)
    x_h = torch.from_numpy(cfg["x"]).pin_memory()
    y_h = torch.from_numpy(cfg["y"].copy()).pin_memory()
    obj = P()
    assert L.b200spHostProductCreate(byref(obj), A.rows, A.cols, A.nnz, rp.ctypes.data_as(POINTER(c_int32)),
                                     d_ci.data_ptr(), d_v.data_ptr(), ACL_FLOAT, 0, ACL_FLOAT, ACL_FLOAT, None, None,
                                     3, 2) == 0
    try:
        y_now = cfg["y"].astype(np.float32).copy()
        for alpha, beta in ((1.5, 0.5), (1.5, 0.5), (-2.0, 0.0), (1.5, 0.5)):
            a, b = c_float(alpha), c_float(beta)
            assert L.b200spHostProductRun(obj, byref(a), x_h.data_ptr(), byref(b), y_h.data_ptr(), y_h.data_ptr(), 1) == 0
            assert L.b200spHostProductSynchronize(obj) == 0
            gold = oracle.spmv(A.row_ptr, A.col_ind, A.values, cfg["x"], y_now, alpha, beta)
            scale = abs(alpha) * oracle.spmv_abs_rowsum(A.row_ptr, A.col_ind, A.values, cfg["x"]) + np.abs(beta * y_now)
            helpers.assert_rowwise(y_h.numpy().astype(np.float64), gold, scale, helpers.TOL["f32"], f"alpha {alpha}")
            y_now = y_h.numpy().copy()
        assert L.b200spHostProductRun(obj, None, None, None, None, y_h.data_ptr(), 0) != 0  # no x: refused
    finally:
        assert L.b200spHostProductDestroy(obj) == 0
