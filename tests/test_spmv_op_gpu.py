"""GPU: the SpMVOp plan API (Z = alpha A X + beta Y, fp32, compensated row sums) through the C ABI.

Cases cover the axes of the reference's own test table (test/spmv_op/arch35/spmv_op_test.csv: shape,
sparsity, empty rows, alpha / beta, pointer mode, row-offset width, Z aliasing Y, unsorted columns,
algorithm, diagonal pattern, empty operands) with inputs drawn here.  Every result is checked three ways:
against the oracle's restatement of the reference's row recurrence, against an exact (fp64) product
within a few fp32 roundings, and with the reference table's own criteria (test/frame/verify.h:112-160 with
the table's thresholds: mean relative error < 1e-6, largest < 5e-6, relative to |gold| + 2^-14).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

EPS = 2.0 ** -24


def make_case(seed, m, k, sparsity, empty_prob=0.0, unsorted=False, pattern="random"):
    rng = np.random.default_rng(seed)
    if pattern == "diag":
        n = min(m, k)
        lengths = np.zeros(m, np.int64)
        lengths[:n] = 1
        ci = np.arange(n, dtype=np.int32)
    else:
        dens = 1.0 - sparsity
        lengths = rng.binomial(k, dens, size=m).astype(np.int64) if k > 0 else np.zeros(m, np.int64)
        lengths[rng.random(m) < empty_prob] = 0
        cols = [np.sort(rng.choice(k, size=int(n), replace=False)) for n in lengths] if m * k <= 1 << 22 else None
        if cols is None:  # large and very sparse: draw with replacement, then make each row unique
            cols = [np.unique(rng.integers(0, k, size=int(n))) for n in lengths]
            lengths = np.array([c.size for c in cols], np.int64)
        if unsorted:
            cols = [rng.permutation(c) for c in cols]
        ci = (np.concatenate(cols) if cols else np.zeros(0)).astype(np.int32)
    rp = np.zeros(m + 1, np.int64)
    rp[1:] = np.cumsum(lengths)
    val = rng.uniform(-1.0, 1.0, int(rp[-1])).astype(np.float32)
    x = rng.uniform(-1.0, 1.0, k).astype(np.float32)
    y = rng.uniform(-1.0, 1.0, m).astype(np.float32)
    return rp, ci, val, x, y


def run_op(pkg, handle, device, rp, ci, val, x, y, alpha, beta, k, *, offsets="i32", base=0, alias=False,
           alg=0, device_scalars=False, runs=1):
    from ops_sparse_b200 import api
    m = rp.size - 1
    ro = (rp + base).astype(np.int64 if offsets == "i64" else np.int32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    d_ro, d_ci, d_v = dev(ro), dev(ci + base if ci.size else ci), dev(val)
    A = api.CsrMatrix(d_ro, d_ci, d_v, m, k, nnz=int(rp[-1]), index_base=base)
    dx, dy = api.DnVec(dev(x), size=k), api.DnVec(dev(y), size=m)
    dz = dy if alias else api.DnVec(torch.full((max(m, 1),), float("nan"), device=device)[:m], size=m)
    plan = api.SpMVOpPlan(handle, A, dx, dy, dz, alg=alg)
    handle.set_pointer_mode_device(device_scalars)
    try:
        a = torch.tensor([alpha], dtype=torch.float32, device=device) if device_scalars else alpha
        b = torch.tensor([beta], dtype=torch.float32, device=device) if device_scalars else beta
        outs = []
        for _ in range(runs):
            if alias:
                dy.values.copy_(dev(y))
            plan.run(dx, dy, dz, a, b)
            torch.cuda.synchronize()
            outs.append(dz.values.cpu().numpy().copy())
    finally:
        handle.set_pointer_mode_device(False)
        plan.close()
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint32), outs[0].view(np.uint32)), "runs differ"
    return outs[0]


def check(oracle, got, rp, ci, val, x, y, alpha, beta, what):
    m = rp.size - 1
    if m == 0:
        assert got.size == 0
        return
    exact, mag = oracle.spmv_exact(rp, ci, val, x, y, alpha, beta)
    gold = exact.astype(np.float32)
    lengths = np.diff(rp)
    bound = 4 * EPS * (np.abs(exact) + np.abs(np.float64(np.float32(beta)) * y)) \
        + 64 * EPS * EPS * abs(alpha) * mag * np.maximum(lengths, 1) + 1e-45
    err = np.abs(got.astype(np.float64) - exact)
    assert np.all(err <= bound), f"{what}: exact-product bound exceeded by {np.max(err / bound):.2f}x"
    ref = oracle.spmv_op(rp, ci, val, x, y, alpha, beta)
    err_ref = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err_ref <= 2 * bound), f"{what}: differs from the oracle's row recurrence"
    # reference table criteria; they divide by |gold|, so rows in which alpha*A*x and beta*y cancel to less
    # than a sixteenth of their size are left to the bound above (no fp32 result can meet 1e-6 there: the
    # reference's own final two roundings are relative to the uncancelled terms)
    assert np.all(np.isfinite(got)), what
    size = abs(alpha) * mag + np.abs(np.float64(np.float32(beta)) * y)
    well = np.abs(exact) >= size / 16
    differs = (got != gold) & well
    rel = np.abs(got.astype(np.float64) - gold) / (np.abs(gold.astype(np.float64)) + 0.00006103515625)
    mere = rel[differs].mean() if differs.any() else 0.0
    mare = rel[well].max(initial=0.0)
    assert mere < 1e-6 and mare < 5e-6, f"{what}: MERE {mere:.2e} MARE {mare:.2e}"


SMALL = [
    # name, m, k, sparsity, empty_prob, seed, alpha, beta, device_scalars, offsets, alias, unsorted, alg, pattern
    ("basic_4x4", 4, 4, 0.5, 0.0, 42, 1.0, 0.0, True, "i32", False, False, 0, "random"),
    ("alpha2_beta1", 4, 4, 0.5, 0.0, 43, 2.0, 1.0, True, "i32", False, False, 0, "random"),
    ("alpha_half_beta_neg1", 4, 4, 0.5, 0.0, 44, 0.5, -1.0, True, "i32", False, False, 0, "random"),
    ("alpha0", 4, 4, 0.5, 0.0, 45, 0.0, 1.0, True, "i32", False, False, 0, "random"),
    ("alpha0_beta0", 4, 4, 0.5, 0.0, 47, 0.0, 0.0, True, "i32", False, False, 0, "random"),
    ("unsorted_16", 16, 16, 0.5, 0.0, 61, 1.0, 1.0, True, "i32", False, True, 0, "random"),
    ("dense_32", 32, 32, 0.1, 0.0, 53, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("single_1x1", 1, 1, 0.0, 0.0, 54, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("zero_1x1", 1, 1, 1.0, 0.0, 55, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("all_empty_4x4", 4, 4, 1.0, 0.0, 0, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("host_scalars", 4, 4, 0.5, 0.0, 57, 3.0, -2.0, False, "i32", False, False, 0, "random"),
    ("wide_4x16", 4, 16, 0.5, 0.0, 58, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("tall_16x4", 16, 4, 0.5, 0.0, 59, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("diag_8", 8, 8, 0.0, 0.0, 0, 1.0, 1.0, True, "i32", False, False, 0, "diag"),
    ("empty_rows_8", 8, 8, 0.5, 0.5, 60, 1.0, 1.0, True, "i32", False, False, 0, "random"),
]
LARGE = [
    ("2048_5pct", 2048, 2048, 0.95, 0.0, 101, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("4096_5pct_alg1", 4096, 4096, 0.95, 0.0, 102, 1.0, 1.0, True, "i32", False, False, 1, "random"),
    ("2048_half_dense", 2048, 2048, 0.50, 0.0, 105, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("wide_1024x4096", 1024, 4096, 0.95, 0.0, 107, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("tall_4096x1024", 4096, 1024, 0.95, 0.0, 108, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("i64_scaled", 2048, 2048, 0.95, 0.0, 111, 2.5, -1.5, True, "i64", False, False, 0, "random"),
    ("alias_scaled", 2048, 2048, 0.95, 0.0, 115, 3.0, -2.0, True, "i32", True, False, 0, "random"),
    ("alias_i64", 2048, 2048, 0.95, 0.0, 114, 1.0, 1.0, True, "i64", True, False, 0, "random"),
    ("alpha_1e6_beta_1e-6", 2048, 2048, 0.95, 0.0, 119, 1e6, 1e-6, True, "i32", False, False, 0, "random"),
    ("alpha_1e-6_beta_1e6", 2048, 2048, 0.95, 0.0, 120, 1e-6, 1e6, True, "i32", False, False, 0, "random"),
    ("unsorted_2048", 2048, 2048, 0.95, 0.0, 121, 1.0, 1.0, True, "i32", False, True, 0, "random"),
    ("diag_4096", 4096, 4096, 0.0, 0.0, 0, 1.0, 1.0, True, "i32", False, False, 0, "diag"),
    ("empty_rows_most", 2048, 2048, 0.95, 0.9, 123, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("nnz0_4096", 4096, 4096, 1.0, 0.0, 0, 2.0, 1.5, True, "i32", False, False, 0, "random"),
    ("host_4096", 4096, 4096, 0.95, 0.0, 124, 1.0, 1.0, False, "i32", False, False, 0, "random"),
    ("alg2_2048", 2048, 2048, 0.95, 0.0, 125, 1.0, 1.0, True, "i32", False, False, 2, "random"),
    ("alg2_alias", 2048, 2048, 0.95, 0.0, 127, 1.0, 1.0, True, "i32", True, False, 2, "random"),
    ("alg2_i64", 2048, 2048, 0.95, 0.0, 128, 1.0, 1.0, True, "i64", False, False, 2, "random"),
    ("row_1x100000", 1, 100000, 0.99, 0.0, 132, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("col_100000x1", 100000, 1, 0.0, 0.0, 133, 1.0, 1.0, True, "i32", False, False, 0, "random"),
    ("col_i64_100000x1", 100000, 1, 0.0, 0.0, 137, 1.0, 1.0, True, "i64", False, False, 2, "random"),
    ("full_1024", 1024, 1024, 0.0, 0.0, 138, 1.0, 1.0, True, "i32", False, False, 2, "random"),
]


@pytest.mark.parametrize("case", SMALL + LARGE, ids=[c[0] for c in SMALL + LARGE])
def test_table_axes(pkg, handle, device, oracle, case):
    name, m, k, sp, ep, seed, alpha, beta, dev_scalars, offsets, alias, unsorted, alg, pattern = case
    rp, ci, val, x, y = make_case(seed, m, k, sp, ep, unsorted, pattern)
    got = run_op(pkg, handle, device, rp, ci, val, x, y, alpha, beta, k, offsets=offsets, alias=alias, alg=alg,
                 device_scalars=dev_scalars, runs=2)
    check(oracle, got, rp, ci, val, x, y, alpha, beta, name)


@pytest.mark.parametrize("m,k", [(0, 4), (4, 0), (0, 0), (0, 1024), (1024, 0)])
def test_empty_operands(pkg, handle, device, oracle, m, k):
    rp, ci, val, x, y = make_case(0, m, k, 1.0, pattern="random")
    got = run_op(pkg, handle, device, rp, ci, val, x, y, 1.0, 1.0, k)
    assert got.size == m
    if m:
        assert np.array_equal(got, y)  # A has no entries: Z = beta * Y


@pytest.mark.parametrize("alg", [1, 2])
@pytest.mark.parametrize("offsets", ["i32", "i64"])
def test_index_base_one_and_power_law_rows(pkg, handle, device, oracle, alg, offsets):
    """One-based offsets and columns; row lengths from 0 to 20000 so that every lane-group width and the
    longest-first ordering of ALG2 are used."""
    from ops_sparse_b200 import synth
    rng = np.random.default_rng(77)
    m, k = 6000, 30000
    lengths = synth.zipf_lengths(rng, m, 1.6, 20000, 40.0)
    lengths[rng.random(m) < 0.05] = 0
    A = synth.csr_from_lengths(rng, lengths, k, synth.normal)
    rp = A.row_ptr.astype(np.int64)
    x, y = rng.standard_normal(k).astype(np.float32), rng.standard_normal(m).astype(np.float32)
    got = run_op(pkg, handle, device, rp, A.col_ind, A.values, x, y, -1.25, 0.75, k, offsets=offsets, base=1, alg=alg,
                 runs=2)
    check(oracle, got, rp, A.col_ind, A.values, x, y, -1.25, 0.75, f"base1 alg{alg} {offsets}")


def test_cancelling_rows_keep_their_digits(pkg, handle, device, oracle):
    """Rows whose large terms cancel: a plain fp32 sum loses every digit, the compensated one must not."""
    rng = np.random.default_rng(9)
    m, k, nb, ns = 512, 4096, 300, 10
    n = 2 * nb + ns
    rp = np.arange(m + 1, dtype=np.int64) * n
    ci = np.concatenate([np.sort(rng.choice(k, n, replace=False)) for _ in range(m)]).astype(np.int32)
    x = np.ones(k, np.float32)
    big = (rng.uniform(1e4, 1e6, (m, nb))).astype(np.float32)
    small = rng.uniform(-1.0, 1.0, (m, ns)).astype(np.float32)
    val = np.concatenate([big, -big, small], axis=1)
    val = np.take_along_axis(val, rng.permuted(np.tile(np.arange(val.shape[1]), (m, 1)), axis=1), axis=1)
    val = val.astype(np.float32).reshape(-1)
    y = np.zeros(m, np.float32)
    for alg in (1, 2):
        got = run_op(pkg, handle, device, rp, ci, val, x, y, 1.0, 0.0, k, alg=alg)
        exact, mag = oracle.spmv_exact(rp, ci, val, x, y, 1.0, 0.0)
        err = np.abs(got.astype(np.float64) - exact)
        assert np.all(err <= 4 * EPS * np.abs(exact) + 8 * EPS * EPS * mag * n), f"alg {alg}"
        plain = np.abs(np.add.reduceat(val, rp[:-1]).astype(np.float64) - exact)  # a plain fp32 sum, for contrast
        assert np.median(plain) > 100 * np.median(err + 1e-12)


def test_nan_in_y_is_ignored_when_beta_is_zero_and_values_may_change(pkg, handle, device, oracle):
    """beta == 0 never reads Y; the values of A may be updated in place between runs of one plan."""
    from ops_sparse_b200 import api
    rp, ci, val, x, y = make_case(31, 3000, 3000, 0.97)
    m = k = 3000
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    d_v = dev(val)
    A = api.CsrMatrix(dev(rp.astype(np.int32)), dev(ci), d_v, m, k, nnz=int(rp[-1]))
    dx = api.DnVec(dev(x), size=k)
    dy = api.DnVec(torch.full((m,), float("nan"), device=device), size=m)
    dz = api.DnVec(torch.zeros(m, device=device), size=m)
    for alg in (1, 2):
        plan = api.SpMVOpPlan(handle, A, dx, dy, dz, alg=alg)
        plan.run(dx, dy, dz, 2.0, 0.0)
        torch.cuda.synchronize()
        check(oracle, dz.values.cpu().numpy(), rp, ci, val, x, np.zeros(m, np.float32), 2.0, 0.0, f"nan y alg{alg}")
        val2 = (val * np.float32(-0.5) + np.float32(0.25)).astype(np.float32)
        d_v.copy_(dev(val2))
        plan.run(dx, dy, dz, 2.0, 0.0)
        torch.cuda.synchronize()
        check(oracle, dz.values.cpu().numpy(), rp, ci, val2, x, np.zeros(m, np.float32), 2.0, 0.0, f"new values alg{alg}")
        d_v.copy_(dev(val))
        plan.close()


def test_execute_checks_on_device(pkg, handle, device):
    """Checks that read the handle: vector sizes must equal the matrix dimensions; Y may be absent only when
    beta == 0 is known on the host."""
    from ctypes import byref, c_float, c_void_p, addressof
    from ops_sparse_b200 import api
    S, L = pkg, pkg.lib()
    rp, ci, val, x, y = make_case(3, 64, 48, 0.8)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    A = api.CsrMatrix(dev(rp.astype(np.int32)), dev(ci), dev(val), 64, 48, nnz=int(rp[-1]))
    dx, dy, dz = api.DnVec(dev(x)), api.DnVec(dev(y)), api.DnVec(torch.zeros(64, device=device))
    plan = api.SpMVOpPlan(handle, A, dx, dy, dz)
    one, zero = c_float(1.0), c_float(0.0)
    a1, b1, b0 = c_void_p(addressof(one)), c_void_p(addressof(one)), c_void_p(addressof(zero))
    run = L.aclsparseSpMVOp
    long_x = api.DnVec(torch.zeros(49, device=device))
    short_y = api.DnVec(torch.zeros(63, device=device))
    assert run(handle.raw, plan._plan, a1, b1, long_x.raw, dy.raw, dz.raw) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(handle.raw, plan._plan, a1, b1, dx.raw, short_y.raw, dz.raw) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(handle.raw, plan._plan, a1, b1, dx.raw, dy.raw, short_y.raw) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert run(handle.raw, plan._plan, a1, b0, dx.raw, dy.raw, dz.raw) == 0
    torch.cuda.synchronize()
    plan.close()
