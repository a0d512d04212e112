"""GPU: the five benchmark configurations at their full size, every output against the CPU oracle.

Each test builds the configuration exactly as the benchmark does (same seeds, same sizes), runs it through the
aclsparse C API with a Preprocess'ed buffer, and hands the whole result to the oracle's threaded checker, which
forms the golden row by row (the arithmetic of SpmvCpu, test/spmv/arch22/spmv_test.cpp:156-173, and SpmmCpuFp32,
test/spmm/arch35/spmm_test.cpp:125-161, of the reference) and applies the per-row tolerance
|got - gold| <= tol * (|alpha| * sum |a_ij b_j| + |beta * old|), tol = 1e-5 for fp32 data and 2e-3 for 16-bit
values with fp32 accumulation.  The plan the analysis chose is asserted too, so that the kernels checked here are
the ones the benchmark times.
"""
from __future__ import annotations

from ctypes import c_int32, c_int64, c_size_t, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def _plan_info(pkg, d_rp, d_ci, rows, cols, nnz, device):
    L = pkg.lib()
    L.b200sp_spmv_plan_bytes.restype = c_size_t
    L.b200sp_spmv_plan_bytes.argtypes = [c_int64, c_int64, c_int64]
    L.b200sp_spmv_analyze.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p,
                                      c_void_p]
    nb = L.b200sp_spmv_plan_bytes(rows, cols, nnz)
    plan = torch.empty(nb, dtype=torch.uint8, device=device)
    info = (c_int32 * 8)()
    assert L.b200sp_spmv_analyze(c_void_p(d_rp.data_ptr()), c_void_p(d_ci.data_ptr()), rows, cols, nnz,
                                 c_void_p(plan.data_ptr()), nb, info, None) == 0
    torch.cuda.synchronize()
    return list(info)


def _launches(pkg):
    f = pkg.lib().b200sp_kernel_launches
    f.restype = __import__("ctypes").c_ulonglong
    return int(f())


def _run_spmv(cfg, handle, device, oracle, pkg, expect_kind=None, expect_launches=None):
    from ops_sparse_b200 import api
    A = cfg["A"]
    vt, ot = TORCH[cfg["val"]], TORCH[cfg["out"]]
    d_rp, d_ci = torch.from_numpy(A.row_ptr).to(device), torch.from_numpy(A.col_ind).to(device)
    d_v = torch.from_numpy(A.values).to(device).to(vt)
    d_x = torch.from_numpy(cfg["x"]).to(device).to(vt)
    d_y = torch.from_numpy(cfg["y"]).to(device).to(ot)
    info = _plan_info(pkg, d_rp, d_ci, A.rows, A.cols, A.nnz, device)
    if expect_kind is not None:
        assert info[0] == expect_kind, info
    dA, dx, dy = api.CsrMatrix(d_rp, d_ci, d_v, A.rows, A.cols), api.DnVec(d_x), api.DnVec(d_y)
    buf = api.spmv_preprocess(handle, dA, dx, dy)
    before = _launches(pkg)
    api.spmv(handle, dA, dx, dy, cfg["alpha"], cfg["beta"], buffer=buf)
    torch.cuda.synchronize()
    if expect_launches is not None:
        assert _launches(pkg) - before == expect_launches
    vw = d_v.to(torch.float32).cpu().numpy()
    xw = d_x.to(torch.float32).cpu().numpy()
    y0 = torch.from_numpy(cfg["y"]).to(ot).to(torch.float32).numpy()
    got = dy.values.to(torch.float32).cpu().numpy()
    tol = 1e-5 if cfg["val"] == "f32" else 2e-3
    bad, worst = oracle.check_spmv_f32(A.row_ptr, A.col_ind, vw, xw, y0, got, cfg["alpha"], cfg["beta"], tol)
    assert bad == 0, f"{bad} of {A.rows} rows outside tolerance {tol}; worst err / scale {worst:.3g}"
    return info


def _run_spmm(cfg, handle, device, oracle, pkg, expect_launches=None, expect_blocks=None):
    import ctypes
    from ops_sparse_b200 import api
    A = cfg["A"]
    vt, ot = TORCH[cfg["val"]], TORCH[cfg["out"]]
    d_rp, d_ci = torch.from_numpy(A.row_ptr).to(device), torch.from_numpy(A.col_ind).to(device)
    d_v = torch.from_numpy(A.values).to(device).to(vt)
    d_B = torch.from_numpy(cfg["B"]).to(device).to(vt)
    d_C = torch.from_numpy(cfg["C"]).to(device).to(ot)
    dA = api.CsrMatrix(d_rp, d_ci, d_v, A.rows, A.cols)
    dB, dC = api.DnMat.row_major(d_B), api.DnMat.row_major(d_C)
    buf = api.spmm_preprocess(handle, dA, dB, dC)
    plan = (ctypes.c_int32 * 4)()
    assert pkg.lib().b200spSpMMPlanInfo(dA.raw, plan) == 0 and plan[3] == 1
    if expect_blocks is not None:  # long rows by column blocks of B (units > 0) or by segments (units == 0)
        assert (plan[1] > 0) == expect_blocks, list(plan)
    before = _launches(pkg)
    api.spmm(handle, dA, dB, dC, cfg["alpha"], cfg["beta"], buffer=buf)
    torch.cuda.synchronize()
    if expect_launches is not None:
        assert _launches(pkg) - before == expect_launches
    assert pkg.lib().b200sp_spmm_stream_error() == 0
    vw = d_v.to(torch.float32).cpu().numpy()
    Bw = d_B.to(torch.float32).cpu().numpy()
    del d_B
    C0 = torch.from_numpy(cfg["C"]).to(ot).to(torch.float32).numpy()
    got = dC.values.to(torch.float32).cpu().numpy()
    tol = 1e-5 if cfg["val"] == "f32" else 2e-3
    bad, worst = oracle.check_spmm_f32(A.row_ptr, A.col_ind, vw, Bw, C0, got, cfg["alpha"], cfg["beta"], tol)
    assert bad == 0, f"{bad} of {got.size} outputs outside tolerance {tol}; worst err / scale {worst:.3g}"


def test_c1_spmv_f32_4096(handle, device, oracle, pkg):
    from ops_sparse_b200 import synth
    cfg = synth.config1()
    info = _run_spmv(cfg, handle, device, oracle, pkg, expect_kind=1, expect_launches=1)
    assert info[1] == 0 and info[2] == 0  # sixteen entries per row: the short-row kernel alone


def test_c2_spmv_f32_powerlaw_1m(handle, device, oracle, pkg):
    """Long rows (512+ entries, up to 16384) must go through SpmvLongBlockKernel with 32 blocks of x beside
    SpmvMediumShortKernel: two launches per product."""
    from ops_sparse_b200 import synth
    cfg = synth.config2()
    lengths = cfg["A"].lengths()
    info = _run_spmv(cfg, handle, device, oracle, pkg, expect_kind=2, expect_launches=2)
    assert info[4] == 32 and info[5] == 32768
    assert info[2] == int((lengths >= info[6]).sum()) and info[1] == int(((lengths > 32) & (lengths < info[6])).sum())
    assert int(lengths.max()) == 16384


def test_c3_spmv_f16_stencil_128(handle, device, oracle, pkg):
    from ops_sparse_b200 import synth
    cfg = synth.config3()
    assert cfg["A"].rows == 128 ** 3 and cfg["A"].nnz == (3 * 128 - 2) ** 3
    info = _run_spmv(cfg, handle, device, oracle, pkg, expect_kind=1, expect_launches=1)
    assert info[1] == 0 and info[2] == 0 and info[3] == 4


def test_c4_spmm_f32_262144_n64(handle, device, oracle, pkg):
    from ops_sparse_b200 import synth
    cfg = synth.config4()
    assert cfg["A"].rows == 262144 and cfg["B"].shape == (262144, 64)
    _run_spmm(cfg, handle, device, oracle, pkg, expect_launches=1, expect_blocks=False)  # SpmmFastKernel alone


def test_c5_spmm_bf16_graph_2m_n256(handle, device, oracle, pkg):
    """512-byte rows of B: SpmmRowStreamKernel for the rows of up to 1024 entries and, for the longer ones (up to
    65536 entries, ascending columns, B of 1 GB), SpmmLongBlockKernel: two launches per product."""
    from ops_sparse_b200 import synth
    cfg = synth.config5()
    A = cfg["A"]
    assert A.rows == 1 << 21 and cfg["B"].shape == (1 << 21, 256) and int(A.lengths().max()) > 4096
    _run_spmm(cfg, handle, device, oracle, pkg, expect_launches=2, expect_blocks=True)
