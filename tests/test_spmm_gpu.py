"""GPU: CSR SpMM through the aclsparse C API against the CPU oracle and the golden fixtures."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def formula(n):
    i = (np.arange(n, dtype=np.int64) % 10001).astype(np.float32)
    return (np.float32(-5.0) + np.float32(10.0) * i / np.float32(10000.0)).astype(np.float32)


def run_spmm(h, device, rp, ci, val, vt, B_store, C_store, ot, m, k, n, ldb, ldc, alpha, beta, op_b=False,
             b_order="row", c_order="row", alg=0, preprocess=True):
    """Flat storage arrays in, new C storage out."""
    from ops_sparse_b200 import api, ACL_SPARSE_OP_TRANSPOSE, ACL_SPARSE_OP_NON_TRANSPOSE

    A = helpers.make_csr(device, rp, ci, val, vt, m, k)
    dB = api.DnMat(helpers.to_device(B_store, vt, device), k, n, ldb, b_order)
    dC = api.DnMat(helpers.to_device(C_store, ot, device), m, n, ldc, c_order)
    op = ACL_SPARSE_OP_TRANSPOSE if op_b else ACL_SPARSE_OP_NON_TRANSPOSE
    if preprocess:
        buf = api.spmm_preprocess(h, A, dB, dC, op, alg)
    else:  # buffer of the right size that Preprocess never saw: SpMM analyses into it itself
        buf = torch.empty(api.spmm_buffer_size(h, A, dB, dC, op, alg), dtype=torch.uint8, device=device)
    api.spmm(h, A, dB, dC, alpha, beta, op_b=op, alg=alg, buffer=buf)
    torch.cuda.synchronize()
    first = dC.values.clone()
    if preprocess:  # a second run on the same plan gives the same bits
        dC2 = api.DnMat(helpers.to_device(C_store, ot, device), m, n, ldc, c_order)
        api.spmm(h, A, dB, dC2, alpha, beta, op_b=op, alg=alg, buffer=buf)
        torch.cuda.synchronize()
        assert torch.equal(first.view(torch.uint8), dC2.values.view(torch.uint8)), "second run differs"
    return helpers.to_host(first, ot)


def compact_case(oracle, rng, m, k, n, lengths, vt, ot, alpha, beta):
    from ops_sparse_b200 import synth
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    ci = synth.columns_for_lengths(rng, np.asarray(lengths), k)
    val = oracle.to_storage(rng.uniform(-1, 1, rp[-1]).astype(np.float32), vt)
    B = oracle.to_storage(rng.standard_normal((k, n)).astype(np.float32), vt)
    C = oracle.to_storage(rng.standard_normal((m, n)).astype(np.float32), ot)
    return rp, ci, val, B, C


def check_compact(oracle, rp, ci, val, B, C, vt, ot, alpha, beta, got, what):
    m, n = C.shape
    if vt == "f32":
        gold = oracle.spmm_f32(rp, ci, val, B, C, alpha, beta)
    else:
        gold = oracle.from_storage(oracle.spmm_16(rp, ci, val, B, C, alpha, beta, vt, ot), ot).astype(np.float64)
    scale = abs(alpha) * oracle.spmm_abs_sum(rp, ci, val, B, vt) + np.abs(beta * oracle.from_storage(C, ot).astype(np.float64))
    tol = helpers.TOL[vt]
    if ot in ("f16", "bf16"):
        scale = scale + np.abs(gold) * (2.0 ** -11 if ot == "f16" else 2.0 ** -8) / tol
    helpers.assert_rowwise(oracle.from_storage(got, ot).astype(np.float64).reshape(m, n), gold, scale, tol, what)


def test_known_answer_4x3(handle, device):
    """sparse/spmm/README.md:276-305, 404-412 of the reference."""
    rp = np.array([0, 2, 3, 4, 5], np.int32)
    ci = np.array([0, 2, 1, 0, 2], np.int32)
    v = np.array([1, 2, 3, 4, 5], np.float32)
    B = np.array([[1, 0], [0, 1], [1, 1]], np.float32)
    got = run_spmm(handle, device, rp, ci, v, "f32", B, np.zeros((4, 2), np.float32), "f32", 4, 3, 2, 2, 2, 1.0, 0.0)
    assert np.array_equal(got, np.array([[3, 2], [0, 3], [4, 0], [5, 5]], np.float32))


@pytest.mark.parametrize("preprocess", [True, False])
def test_config4_scaled(handle, device, oracle, preprocess):
    from ops_sparse_b200 import synth
    c = synth.config4(rows=8192, n=64)
    A = c["A"]
    got = run_spmm(handle, device, A.row_ptr, A.col_ind, A.values, "f32", c["B"], c["C"], "f32", A.rows, A.cols, 64,
                   64, 64, c["alpha"], c["beta"], preprocess=preprocess)
    check_compact(oracle, A.row_ptr, A.col_ind, A.values, c["B"], c["C"], "f32", "f32", c["alpha"], c["beta"], got,
                  "config4")


@pytest.mark.parametrize("ot", ["f32", "bf16"])
def test_config5_scaled(handle, device, oracle, ot):
    """bf16 graph adjacency with power-law degrees (rows up to 16384 entries at this scale)."""
    from ops_sparse_b200 import synth
    c = synth.config5(rows=1 << 14, n=256)
    A = c["A"]
    assert A.lengths().max() > 4096  # multi-segment rows are exercised
    val, B = oracle.to_storage(A.values, "bf16"), oracle.to_storage(c["B"], "bf16")
    C = oracle.to_storage(c["C"], ot)
    got = run_spmm(handle, device, A.row_ptr, A.col_ind, val, "bf16", B, C, ot, A.rows, A.cols, 256, 256, 256, 1.0,
                   0.0)
    check_compact(oracle, A.row_ptr, A.col_ind, val, B, C, "bf16", ot, 1.0, 0.0, got, f"config5/{ot}")


@pytest.mark.parametrize("vt,ot", [("f32", "f32"), ("f16", "f16"), ("bf16", "bf16"), ("bf16", "f32")])
@pytest.mark.parametrize("n", [1, 4, 8, 24, 32, 64, 72, 128, 200, 256, 264, 512])
def test_widths_and_types(handle, device, oracle, vt, ot, n):
    rng = np.random.default_rng(n * 7 + len(vt))
    m, k = 700, 900
    lengths = rng.integers(0, 48, size=m)
    lengths[3] = 0
    lengths[10] = 850
    rp, ci, val, B, C = compact_case(oracle, rng, m, k, n, lengths, vt, ot, 1.5, -0.5)
    got = run_spmm(handle, device, rp, ci, val, vt, B, C, ot, m, k, n, n, n, 1.5, -0.5)
    check_compact(oracle, rp, ci, val, B, C, vt, ot, 1.5, -0.5, got, f"{vt}->{ot} n={n}")


@pytest.mark.parametrize("vt,ot,n", [("f32", "f32", 64), ("f32", "f32", 8), ("f32", "f32", 200), ("bf16", "f32", 256),
                                     ("bf16", "bf16", 64), ("f16", "f16", 40)])
def test_bit_identical_to_golden_for_rows_up_to_1024(handle, device, oracle, vt, ot, n):
    """Rows of at most 1024 entries are summed in CSR order with unfused multiply-add: same bits as the golden."""
    rng = np.random.default_rng(n + len(vt))
    m, k = 500, 3000
    lengths = rng.integers(0, 70, size=m)
    lengths[7], lengths[77], lengths[400] = 1024, 1000, 0
    rp, ci, val, B, C = compact_case(oracle, rng, m, k, n, lengths, vt, ot, 1.25, 0.5)
    got = run_spmm(handle, device, rp, ci, val, vt, B, C, ot, m, k, n, n, n, 1.25, 0.5)
    if vt == "f32":
        gold = oracle.spmm_f32_layout(m, n, rp, ci, val, B, n, True, False, C, n, True, 1.25, 0.5).reshape(m, n)
        assert np.array_equal(got.view(np.uint32), gold.view(np.uint32))
    else:
        gold = oracle.spmm_16(rp, ci, val, B, C, 1.25, 0.5, vt, ot)
        assert np.array_equal(got.view(np.uint8), gold.view(np.uint8))


def test_long_rows_segments(handle, device, oracle):
    """Rows of 1024, 1025, 4096, 4097, 9000 and 20000 entries next to short ones."""
    rng = np.random.default_rng(11)
    m, k, n = 600, 30000, 32
    lengths = rng.integers(0, 8, size=m)
    for r, L in zip((1, 100, 200, 300, 400, 599), (1024, 1025, 4096, 4097, 9000, 20000)):
        lengths[r] = L
    rp, ci, val, B, C = compact_case(oracle, rng, m, k, n, lengths, "f32", "f32", 1.0, 0.5)
    for beta in (0.0, 0.5):
        got = run_spmm(handle, device, rp, ci, val, "f32", B, C, "f32", m, k, n, n, n, 1.0, beta)
        check_compact(oracle, rp, ci, val, B, C, "f32", "f32", 1.0, beta, got, f"long rows beta={beta}")


def test_kahan_algorithm(handle, device, oracle):
    from ops_sparse_b200 import ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG as KAHAN
    rng = np.random.default_rng(12)
    m, k, n = 300, 5000, 16
    lengths = np.full(m, 900)
    rp, ci, val, B, C = compact_case(oracle, rng, m, k, n, lengths, "f32", "f32", 1.0, 0.0)
    got = run_spmm(handle, device, rp, ci, val, "f32", B, C, "f32", m, k, n, n, n, 1.0, 0.0, alg=KAHAN)
    check_compact(oracle, rp, ci, val, B, C, "f32", "f32", 1.0, 0.0, got, "kahan")
    # compensated sums sit closer to the exact product than the plain fp32 golden does
    exact = np.zeros((m, n))
    for r in range(m):
        s, e = rp[r], rp[r + 1]
        exact[r] = val[s:e].astype(np.float64) @ B[ci[s:e]].astype(np.float64)
    plain = oracle.spmm_f32(rp, ci, val, B, C, 1.0, 0.0)
    assert np.abs(got - exact).mean() <= np.abs(plain - exact).mean()


@pytest.mark.parametrize("opb", [False, True])
@pytest.mark.parametrize("b_order", ["row", "col"])
@pytest.mark.parametrize("c_order", ["row", "col"])
def test_layouts_with_padding(handle, device, oracle, opb, b_order, c_order):
    rng = np.random.default_rng(13)
    m, k, n = 150, 170, 40
    lengths = rng.integers(0, 30, size=m)
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    from ops_sparse_b200 import synth
    ci = synth.columns_for_lengths(rng, lengths, k)
    val = rng.uniform(-1, 1, rp[-1]).astype(np.float32)
    brow, crow = b_order == "row", c_order == "row"
    # The B descriptor is always k x n with ld >= n (row) or >= k (col); padding of 8 keeps
    # vector alignment so both the fast and the generic kernels are hit across the parameters.
    ldb = (n if brow else k) + 8
    ldc = (n if crow else m) + 8
    nb = max(k, n) * ldb
    nc = (m if crow else n) * ldc
    B = rng.standard_normal(nb).astype(np.float32)
    C = rng.standard_normal(nc).astype(np.float32)
    got = run_spmm(handle, device, rp, ci, val, "f32", B, C, "f32", m, k, n, ldb, ldc, 0.75, 1.25, op_b=opb,
                   b_order=b_order, c_order=c_order)
    gold = oracle.spmm_f32_layout(m, n, rp, ci, val, B, ldb, brow, opb, C, ldc, crow, 0.75, 1.25)
    # op(B) as a compact k x n array, through the same index rule the golden uses
    cc, jj = np.arange(k)[:, None], np.arange(n)[None, :]
    if not opb:
        bidx = cc * ldb + jj if brow else jj * ldb + cc
    else:
        bidx = jj * ldb + cc if brow else cc * ldb + jj
    opB = B[bidx]
    idx = (np.arange(m)[:, None] * ldc + np.arange(n)[None, :]) if crow else (np.arange(n)[None, :] * ldc + np.arange(m)[:, None])
    scale = 0.75 * oracle.spmm_abs_sum(rp, ci, val, opB) + np.abs(1.25 * C[idx].astype(np.float64))
    helpers.assert_rowwise(got.ravel()[idx].astype(np.float64), gold[idx].astype(np.float64), scale, 1e-5,
                           f"layout opB={opb} B={b_order} C={c_order}")
    # padding between rows / columns of C is untouched
    mask = np.ones(nc, bool)
    mask[idx.ravel()] = False
    assert np.array_equal(got.ravel()[mask], C[mask])


def test_int8(handle, device, oracle):
    rng = np.random.default_rng(14)
    m, k, n = 200, 300, 24
    lengths = rng.integers(0, 60, size=m)
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    from ops_sparse_b200 import synth
    ci = synth.columns_for_lengths(rng, lengths, k)
    val = rng.integers(-128, 128, rp[-1]).astype(np.int8)
    B = rng.integers(-128, 128, k * n).astype(np.int8)
    C = rng.integers(-2**31, 2**31, m * n).astype(np.int32)  # large C: the saturating epilogue matters
    got = run_spmm(handle, device, rp, ci, val, "i8", B, C, "i32", m, k, n, n, n, 70000, 3)
    gold = oracle.spmm_i8(m, n, rp, ci, val, B, n, True, False, C, n, True, 70000, 3, saturate=True)
    assert np.array_equal(got.ravel(), gold)
    assert (gold == 2**31 - 1).any() or (gold == -2**31).any()


def test_fp16_output_saturates(handle, device, oracle):
    m = k = 64
    n = 8
    rp = np.arange(0, m + 1, dtype=np.int32)
    ci = np.arange(m, dtype=np.int32)
    val = oracle.to_storage(np.full(m, 300.0, np.float32), "f16")
    B = oracle.to_storage(np.full((k, n), 300.0, np.float32), "f16")
    C = np.zeros((m, n), np.uint16)
    got = run_spmm(handle, device, rp, ci, val, "f16", B, C, "f16", m, k, n, n, n, 1.0, 0.0)
    assert np.all(oracle.from_storage(got, "f16") == 65504.0)


def test_golden_fixtures_spmm35(handle, device, oracle, golden_dir):
    """The reference harness's own five fp32 cases, its fp16 case and its int8 case, with its own
    pass criteria (MERE < 2^-13, MARE < 10 * 2^-13; fp16 2^-10; int8 exact)."""
    z = np.load(golden_dir / "spmm35_fp32.npz")
    for name in z["names"]:
        m, k, n, ldb, ldc, opb, bcol, ccol = (int(v) for v in z[f"{name}/shape"])
        alpha, beta = (float(v) for v in z[f"{name}/scalars"])
        B = formula(k * ldb)
        C = formula(m * ldc) if beta != 0 else np.zeros(m * ldc, np.float32)
        got = run_spmm(handle, device, z[f"{name}/row_ptr"], z[f"{name}/col_ind"], z[f"{name}/val"], "f32", B, C,
                       "f32", m, k, n, ldb, ldc, alpha, beta, op_b=bool(opb), b_order="col" if bcol else "row",
                       c_order="col" if ccol else "row", alg=1)
        ok, st = oracle.verify_mere_mare(got, z[f"{name}/gold"], m, n, ldc, not ccol)
        assert ok, (name, st)
        assert np.array_equal(got.ravel().view(np.uint32), z[f"{name}/gold"].view(np.uint32)), name  # every layout
    z = np.load(golden_dir / "spmm35_f16_i8.npz")
    m, k, n = (int(v) for v in z["shape"])
    got = run_spmm(handle, device, z["row_ptr"], z["col_ind"], z["f16_val"], "f16", z["f16_B"],
                   np.zeros(m * n, np.uint16), "f16", m, k, n, n, n, 1.0, 0.0)
    ok, st = oracle.verify_mere_mare(oracle.from_storage(got, "f16"), oracle.from_storage(z["f16_gold"], "f16"), m, n, n,
                                     True, 2.0 ** -10, 10 * 2.0 ** -10)
    assert ok, st
    assert np.array_equal(got.ravel(), z["f16_gold"])
    got = run_spmm(handle, device, z["row_ptr"], z["col_ind"], z["i8_val"], "i8", z["i8_B"],
                   np.zeros(m * n, np.int32), "i32", m, k, n, n, n, 1, 0)
    assert np.array_equal(got.ravel(), z["i8_gold"])
    got = run_spmm(handle, device, z["row_ptr"], z["col_ind"], z["i8_val"], "i8", z["i8_B"], z["i8_C2"], "i32", m, k,
                   n, n, n, 3, -2)
    assert np.array_equal(got.ravel(), z["i8_gold2"])


def test_golden_fixtures_spmm22(handle, device, oracle, golden_dir):
    z = np.load(golden_dir / "spmm22.npz")
    for i in range(int(z["count"][0])):
        M, K, N, _ = (int(v) for v in z[f"{i}/shape"])
        alpha, beta = (float(v) for v in z[f"{i}/scalars"])
        B = (np.float32(0.5) + np.float32(0.0001) * (np.arange(K * N) % 1000).astype(np.float32))
        C = (np.float32(0.01) * (np.arange(M * N) % 100).astype(np.float32))
        got = run_spmm(handle, device, z[f"{i}/row_ptr"], z[f"{i}/col_ind"], z[f"{i}/val"], "f32", B, C, "f32", M, K,
                       N, N, N, alpha, beta)
        assert oracle.verify_abs_and_rel(got, z[f"{i}/gold"], 1e-3, 1e-3) == 0, i  # the harness's own rule
        ok, st = oracle.verify_mere_mare(got, z[f"{i}/gold"].ravel(), M, N, N)
        assert ok, (i, st)


def test_status_codes(handle, device, pkg):
    """Error paths of the three SpMM entry points (spmm_host.cpp:152-191, 349-351, 373-383)."""
    from ctypes import byref, c_float, c_size_t, c_void_p, cast
    from ops_sparse_b200 import api
    L, S = pkg.lib(), pkg
    rp = torch.tensor([0, 1, 2], dtype=torch.int32, device=device)
    ci = torch.tensor([0, 1], dtype=torch.int32, device=device)
    v = torch.ones(2, dtype=torch.float32, device=device)
    A = api.CsrMatrix(rp, ci, v, 2, 2)
    B = api.DnMat.row_major(torch.ones(2, 4, device=device))
    C = api.DnMat.row_major(torch.zeros(2, 4, device=device))
    one = c_float(1.0)
    al = cast(byref(one), c_void_p)
    size = c_size_t()
    args = (al, A.raw, B.raw, al, C.raw, S.ACL_FLOAT, 0)
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 0, *args, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 0, al, None, B.raw, al, C.raw, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 1, 0, *args, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 2, *args, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 0, al, A.raw, B.raw, al, C.raw, S.ACL_INT32, 0, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 0, al, A.raw, B.raw, al, C.raw, S.ACL_FLOAT, 7, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    Bbad = api.DnMat.row_major(torch.ones(3, 4, device=device))
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 0, al, A.raw, Bbad.raw, al, C.raw, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseSpMMGetBufferSize(handle.raw, 0, 0, *args, byref(size)) == 0 and size.value > 0
    assert L.aclsparseSpMMPreprocess(handle.raw, 0, 0, *args, None) == S.ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES
    assert L.aclsparseSpMM(handle.raw, 0, 0, *args, None) == S.ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES
    buf = torch.empty(size.value, dtype=torch.uint8, device=device)
    assert L.aclsparseSpMM(None, 0, 0, *args, c_void_p(buf.data_ptr())) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    # NULL alpha reads as 0: C = 0 * A B + 1 * C
    C.values.fill_(7.0)
    assert L.aclsparseSpMM(handle.raw, 0, 0, None, A.raw, B.raw, al, C.raw, S.ACL_FLOAT, 0, c_void_p(buf.data_ptr())) == 0
    torch.cuda.synchronize()
    assert torch.all(C.values == 7.0)


def test_row_stream_wait_that_runs_out(pkg, handle, device, oracle):
    """Failure detection without a fault: the row-stream kernel is told to expect 16 bytes more than it copies on
    every barrier and to wait two milliseconds at most.  Every wait runs out; the kernel must raise the flag,
    write nothing of C (beta = 1 leaves the rows without entries as they were) and return with the GPU usable;
    the next Preprocess reports it; with the normal settings the same product is correct again."""
    from ops_sparse_b200 import api, synth
    L = pkg.lib()
    L.b200sp_spmm_stream_wait_test.argtypes = [ctypes.c_longlong, ctypes.c_uint]
    L.b200sp_spmm_stream_wait_test.restype = None
    rng = np.random.default_rng(41)
    m, k, n = 3000, 2500, 256
    lengths = synth.zipf_lengths(rng, m, 1.9, 900, 10.0)   # rows of up to 900 entries: the row-stream kernel alone
    lengths[rng.random(m) < 0.2] = 0
    A = synth.csr_from_lengths(rng, lengths, k, synth.uniform)
    Bq = torch.from_numpy(rng.standard_normal((k, n)).astype(np.float32)).to(torch.bfloat16)
    C0 = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32))
    dA = api.CsrMatrix(torch.from_numpy(A.row_ptr).to(device), torch.from_numpy(A.col_ind).to(device),
                       torch.from_numpy(A.values).to(device).to(torch.bfloat16), m, k)
    dB, dC = api.DnMat.row_major(Bq.to(device)), api.DnMat.row_major(C0.to(device))
    buf = api.spmm_preprocess(handle, dA, dB, dC)
    torch.cuda.synchronize()
    assert L.b200sp_spmm_stream_error() == 0
    try:
        L.b200sp_spmm_stream_wait_test(1 << 22, 16)
        api.spmm(handle, dA, dB, dC, 1.0, 1.0, buffer=buf)
        torch.cuda.synchronize()                              # returns: nothing hangs
        assert L.b200sp_spmm_stream_error() == 1
        assert torch.equal(dC.values.cpu(), C0)               # not one row of C was written with a partial sum
    finally:
        L.b200sp_spmm_stream_wait_test(0, 0)
    # the failure surfaces at the next synchronising entry point, once
    from ops_sparse_b200 import ACL_FLOAT
    args = (handle.raw, 0, 0, None, dA.raw, dB.raw, None, dC.raw, ACL_FLOAT, 0, api._ptr(buf))
    assert L.aclsparseSpMMPreprocess(*args) == pkg.ACL_SPARSE_STATUS_EXECUTION_FAILED
    assert L.b200sp_spmm_stream_error() == 0
    assert L.aclsparseSpMMPreprocess(*args) == 0
    api.spmm(handle, dA, dB, dC, 1.0, 1.0, buffer=buf)
    torch.cuda.synchronize()
    assert L.b200sp_spmm_stream_error() == 0
    vw = torch.from_numpy(A.values).to(torch.bfloat16).to(torch.float32).numpy()
    bad, worst = oracle.check_spmm_f32(A.row_ptr, A.col_ind, vw, Bq.to(torch.float32).numpy(), C0.numpy(),
                                       dC.values.cpu().numpy(), 1.0, 1.0, 2e-3)
    assert bad == 0, worst


def _block_case(rng, m, k, long_rows, lo, hi):
    """A few long rows with ascending columns among short ones."""
    from ops_sparse_b200 import synth
    lengths = rng.integers(0, 40, m)
    lengths[rng.choice(m, long_rows, replace=False)] = rng.integers(lo, hi, long_rows)
    return synth.csr_from_lengths(rng, lengths, k, synth.uniform)


def _analysed_blocks(pkg, dA, n, row_bytes):
    """What the two kernel-level analysis passes decide for this matrix: (units of the column-block path, long rows)."""
    L = pkg.lib()
    c64, P = ctypes.c_int64, ctypes.c_void_p
    L.b200sp_spmm_plan_bytes.restype = ctypes.c_size_t
    L.b200sp_spmm_plan_bytes.argtypes = [c64, c64, c64]
    L.b200sp_spmm_analyze.argtypes = [P, c64, c64, c64, P, ctypes.c_size_t, ctypes.POINTER(ctypes.c_int32), P]
    L.b200sp_spmm_analyze_blocks.argtypes = [P, P, c64, c64, c64, c64, c64, P, ctypes.c_size_t,
                                             ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32), P]
    nbytes = L.b200sp_spmm_plan_bytes(dA.rows, dA.nnz, n)
    plan = torch.empty(nbytes, dtype=torch.uint8, device=dA.row_ptr.device)
    seg, blocks, longs = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    assert L.b200sp_spmm_analyze(dA.row_ptr.data_ptr(), dA.rows, dA.nnz, n, plan.data_ptr(), nbytes,
                                 ctypes.byref(seg), None) == 0
    assert L.b200sp_spmm_analyze_blocks(dA.row_ptr.data_ptr(), dA.col_ind.data_ptr(), dA.rows, dA.cols, dA.nnz, n,
                                        row_bytes, plan.data_ptr(), nbytes, ctypes.byref(blocks), ctypes.byref(longs),
                                        None) == 0
    torch.cuda.synchronize()
    return blocks.value, longs.value


@pytest.mark.parametrize("vt,n", [("bf16", 256), ("f16", 256), ("f32", 128), ("f32", 264)])
def test_long_rows_by_column_blocks(pkg, handle, device, oracle, vt, n):
    """B far larger than L2 and rows of more than 1024 entries with ascending columns: the long rows are summed
    block by block of B (SpmmLongBlockKernel).  The result must satisfy the usual tolerance, be the same bits on
    every run, and the analysis must have chosen that path; with one long row's columns out of order it must not."""
    from ops_sparse_b200 import api
    rng = np.random.default_rng(97)
    esize = 4 if vt == "f32" else 2
    k = (120 << 20) // (n * esize)              # B of about 120 MB
    m = 1500
    A = _block_case(rng, m, k, 40, 1025, 9000)
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[vt]
    cdt = torch.float16 if vt == "f16" else torch.float32       # the reference's fp16 SpMM writes fp16
    Bq = torch.from_numpy(rng.standard_normal((k, n)).astype(np.float32)).to(tdt)
    C0 = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(cdt)
    vq = torch.from_numpy(A.values).to(tdt)
    dB = api.DnMat.row_major(Bq.to(device))
    tol = 1e-5 if vt == "f32" else 2e-3

    def product(col_ind):
        dA = api.CsrMatrix(torch.from_numpy(A.row_ptr).to(device), torch.from_numpy(col_ind).to(device),
                           vq.to(device), m, k)
        outs = []
        for _ in range(2):
            dC = api.DnMat.row_major(C0.to(device))
            buf = api.spmm_preprocess(handle, dA, dB, dC)
            api.spmm(handle, dA, dB, dC, 0.75, -0.5, buffer=buf)
            api.spmm(handle, dA, dB, dC, 0.75, 0.0, buffer=buf)   # the arrival counters must have been reset
            torch.cuda.synchronize()
            outs.append(dC.values.clone())
        assert torch.equal(outs[0], outs[1]), "two runs differ"
        bad, worst = oracle.check_spmm_f32(A.row_ptr, col_ind, vq.to(torch.float32).numpy(),
                                           Bq.to(torch.float32).numpy(), C0.to(torch.float32).numpy(),
                                           outs[0].to(torch.float32).cpu().numpy(), 0.75, 0.0, tol)
        assert bad == 0, worst
        return _analysed_blocks(pkg, dA, n, n * esize)

    blocks, longs = product(A.col_ind)
    assert longs == 40 and blocks >= 2 * 40
    # one long row with two columns swapped: not ascending any more, the segment CTAs take the long rows
    ci = A.col_ind.copy()
    r = int(np.argmax(np.diff(A.row_ptr)))
    s = A.row_ptr[r]
    ci[s + 5], ci[s + 700] = ci[s + 700], ci[s + 5]
    blocks, longs = product(ci)
    assert longs == 40 and blocks == 0


def test_no_wait_ran_out_in_the_row_stream_kernel(pkg, device):
    """The row-stream kernel bounds its waits on the copy engine and raises a flag when one runs out;
    after everything above it must still be clear.  (Runs last in this file.)"""
    torch.cuda.synchronize()
    f = pkg.lib().b200sp_spmm_stream_error
    f.restype = ctypes.c_int
    assert f() == 0
