"""CPU: pins the oracle (oracle/oracle.cpp) to the reference.

1. the 4 x 3 known answer of the reference's SpMM README;
2. the committed golden fixtures, which were produced by the reference's own golden
   functions (tests/golden/make_golden.py): the oracle must reproduce them bit for bit;
3. where oracle/_ref was built (reference sources present), randomised bit-for-bit
   cross-checks against those functions directly, plus the 16-bit converters.
"""
from __future__ import annotations

import numpy as np
import pytest


def formula(n):
    i = (np.arange(n, dtype=np.int64) % 10001).astype(np.float32)
    return (np.float32(-5.0) + np.float32(10.0) * i / np.float32(10000.0)).astype(np.float32)


def test_known_answer_4x3(oracle):
    # sparse/spmm/README.md:276-305 (inputs) and :404-412 (expected C)
    rp = np.array([0, 2, 3, 4, 5], np.int32)
    ci = np.array([0, 2, 1, 0, 2], np.int32)
    v = np.array([1, 2, 3, 4, 5], np.float32)
    B = np.array([[1, 0], [0, 1], [1, 1]], np.float32)
    C = oracle.spmm_f32(rp, ci, v, B, np.zeros((4, 2), np.float32), 1.0, 0.0)
    assert np.array_equal(C, np.array([[3, 2], [0, 3], [4, 0], [5, 5]], np.float64))


def test_fixture_spmm35_fp32(oracle, golden_dir):
    z = np.load(golden_dir / "spmm35_fp32.npz")
    for name in z["names"]:
        m, k, n, ldb, ldc, opb, bcol, ccol = (int(v) for v in z[f"{name}/shape"])
        alpha, beta = (float(v) for v in z[f"{name}/scalars"])
        B = formula(k * ldb)
        C = formula(m * ldc) if beta != 0 else np.zeros(m * ldc, np.float32)
        got = oracle.spmm_f32_layout(m, n, z[f"{name}/row_ptr"], z[f"{name}/col_ind"], z[f"{name}/val"], B, ldb,
                                     not bcol, bool(opb), C, ldc, not ccol, alpha, beta)
        assert np.array_equal(got.view(np.uint32), z[f"{name}/gold"].view(np.uint32)), name


def test_fixture_spmm35_f16_i8(oracle, golden_dir):
    z = np.load(golden_dir / "spmm35_f16_i8.npz")
    m, k, n = (int(v) for v in z["shape"])
    got = oracle.spmm_16(z["row_ptr"], z["col_ind"], z["f16_val"], z["f16_B"], np.zeros((m, n), np.uint16), 1.0, 0.0,
                         "f16", "f16")
    assert np.array_equal(got.ravel(), z["f16_gold"])
    # input rounding itself: the oracle's converter reproduces the harness's fp16 bits
    assert np.array_equal(oracle.f32_to_f16(z["val_f32"]), z["f16_val"])
    for sat in (False, True):  # no overflow in these cases: both epilogues agree with the golden
        gi = oracle.spmm_i8(m, n, z["row_ptr"], z["col_ind"], z["i8_val"], z["i8_B"], n, True, False,
                            np.zeros(m * n, np.int32), n, True, 1, 0, saturate=sat)
        assert np.array_equal(gi, z["i8_gold"])
        gi2 = oracle.spmm_i8(m, n, z["row_ptr"], z["col_ind"], z["i8_val"], z["i8_B"], n, True, False, z["i8_C2"], n,
                             True, 3, -2, saturate=sat)
        assert np.array_equal(gi2, z["i8_gold2"])


def test_fixture_spmm22(oracle, golden_dir):
    z = np.load(golden_dir / "spmm22.npz")
    for i in range(int(z["count"][0])):
        M, K, N, _ = (int(v) for v in z[f"{i}/shape"])
        alpha, beta = (float(v) for v in z[f"{i}/scalars"])
        B = (np.float32(0.5) + np.float32(0.0001) * (np.arange(K * N) % 1000).astype(np.float32)).reshape(K, N)
        C = (np.float32(0.01) * (np.arange(M * N) % 100).astype(np.float32)).reshape(M, N)
        got = oracle.spmm_f32_layout(M, N, z[f"{i}/row_ptr"], z[f"{i}/col_ind"], z[f"{i}/val"], B, N, True, False, C,
                                     N, True, alpha, beta)
        assert np.array_equal(got.view(np.uint32), z[f"{i}/gold"].ravel().view(np.uint32)), i


def test_fixture_spmv(oracle, golden_dir):
    z = np.load(golden_dir / "spmv.npz")
    for i in range(int(z["count"][0])):
        comp, vt, ot = (str(s) for s in z[f"{i}/types"])
        M, N, trans = (int(v) for v in z[f"{i}/dims"])
        a, b = z[f"{i}/scalars"]
        if comp == "i32":
            a, b = int(a), int(b)
        got = oracle.spmv_typed(z[f"{i}/row_ptr"], z[f"{i}/col_ind"], z[f"{i}/val"], z[f"{i}/x"], z[f"{i}/y"], a, b,
                                comp, vt, ot, trans=bool(trans), cols=N, bf16_trunc=True)
        assert np.array_equal(got, z[f"{i}/gold"]), (i, comp, vt, ot, trans)


def test_threads_do_not_change_bits(oracle):
    rng = np.random.default_rng(5)
    M, K, N = 500, 400, 24
    L = rng.integers(0, 40, size=M)
    rp = np.zeros(M + 1, np.int32)
    rp[1:] = np.cumsum(L)
    ci = rng.integers(0, K, size=rp[-1]).astype(np.int32)
    v = rng.standard_normal(rp[-1]).astype(np.float32)
    x, y = rng.standard_normal(K).astype(np.float32), rng.standard_normal(M).astype(np.float32)
    assert np.array_equal(oracle.spmv(rp, ci, v, x, y, 1.5, 0.5, threads=1), oracle.spmv(rp, ci, v, x, y, 1.5, 0.5, threads=4))
    B, C = rng.standard_normal((K, N)).astype(np.float32), rng.standard_normal((M, N)).astype(np.float32)
    assert np.array_equal(oracle.spmm_f32(rp, ci, v, B, C, 1.0, 0.5, threads=1),
                          oracle.spmm_f32(rp, ci, v, B, C, 1.0, 0.5, threads=3))


def test_verifiers(oracle):
    gold = np.linspace(-3, 3, 1000).astype(np.float32)
    ok, st = oracle.verify_mixed(gold, gold * (1 + 2.0 ** -12), "f32")
    assert ok and st["matched"] == 1.0
    bad = gold.copy()
    bad[:20] += 0.5  # 2 % of the elements far off: matched ratio 0.98 < 0.99 and max error > 1e-2
    ok, st = oracle.verify_mixed(gold, bad, "f32")
    assert not ok and st["max_abs_err"] >= 0.49
    ok, _ = oracle.verify_mixed(gold, np.full_like(gold, np.nan), "f32")
    assert not ok
    g2 = gold.reshape(100, 10)
    ok, st = oracle.verify_mere_mare(g2 * (1 + 2.0 ** -15), g2, 100, 10, 10)
    assert ok
    ok, _ = oracle.verify_mere_mare(g2 * 1.01, g2, 100, 10, 10)
    assert not ok
    assert oracle.verify_abs_and_rel(gold + 1e-4, gold) == 0
    assert oracle.verify_abs_and_rel(gold + 1.0, gold) > 0


# ---- direct cross-checks against the reference's compiled golden (present in this checkout only)

def _need_ref(oracle, name):
    if not oracle.ref_available(name):
        pytest.skip(f"oracle/_ref/libref_{name}.so not built (reference sources absent)")


def test_ref_converters(oracle):
    _need_ref(oracle, "spmm35")
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(400000) * 10.0 ** rng.integers(-9, 6, 400000)).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65519.99, 65520.0, 1e-8, 6.1e-5], np.float32)])
    assert np.array_equal(oracle.f32_to_f16(x), oracle.ref_f32_to_f16(x))
    h = np.arange(65536, dtype=np.uint16)
    mine, ref = oracle.f16_to_f32(h).view(np.uint32), oracle.ref_f16_to_f32(h).view(np.uint32)
    sub = ((h & 0x7C00) == 0) & ((h & 0x03FF) != 0)
    assert np.array_equal(mine[~sub], ref[~sub])
    # The harness's fp16->fp32 routine mis-scales subnormal halves whose fp32 exponent field is
    # even (it ORs the hidden bit into the exponent); none occur in its own data.  The oracle
    # follows IEEE 754 there: every subnormal is mantissa * 2^-24 exactly.
    exact = (h[sub] & 0x3FF).astype(np.float64) * 2.0 ** -24 * np.where(h[sub] & 0x8000, -1.0, 1.0)
    assert np.array_equal(oracle.f16_to_f32(h[sub]).astype(np.float64), exact)
    assert int((mine[sub] != ref[sub]).sum()) == 1364


@pytest.mark.parametrize("seed", range(6))
def test_ref_spmm_random_layouts(oracle, seed):
    _need_ref(oracle, "spmm35")
    rng = np.random.default_rng(100 + seed)
    m, k, n = int(rng.integers(1, 70)), int(rng.integers(1, 90)), int(rng.integers(1, 40))
    L = rng.integers(0, min(k, 30) + 1, size=m)
    rp = np.zeros(m + 1, np.int32)
    rp[1:] = np.cumsum(L)
    ci = np.concatenate([rng.choice(k, size=int(x), replace=False) for x in L] + [np.zeros(0, np.int64)]).astype(np.int32)
    v = rng.uniform(-5, 5, rp[-1]).astype(np.float32)
    for opb in (False, True):
        for brow in (True, False):
            for crow in (True, False):
                # op(B) is k x n: its storage is k x ldb (N,row), n x ldb (N,col / T,row), k x ldb (T,col)
                pad_b, pad_c = int(rng.integers(0, 3)), int(rng.integers(0, 3))
                b_rows_contig = (not opb and brow) or (opb and not brow)
                ldb = (n if b_rows_contig else k) + pad_b
                nb = (k if b_rows_contig else n) * ldb
                ldc = (n if crow else m) + pad_c
                nc = (m if crow else n) * ldc
                B = rng.uniform(-5, 5, nb).astype(np.float32)
                C = rng.uniform(-5, 5, nc).astype(np.float32)
                alpha, beta = float(rng.uniform(-2, 2)), float(rng.choice([0.0, 0.5, -1.25]))
                mine = oracle.spmm_f32_layout(m, n, rp, ci, v, B, ldb, brow, opb, C, ldc, crow, alpha, beta)
                ref = oracle.ref_spmm_f32(m, n, rp, ci, v, B, ldb, brow, opb, C, ldc, crow, alpha, beta)
                assert np.array_equal(mine.view(np.uint32), ref.view(np.uint32))
                vi = rng.integers(-128, 128, rp[-1]).astype(np.int8)
                Bi = rng.integers(-128, 128, nb).astype(np.int8)
                Ci = rng.integers(-1000, 1000, nc).astype(np.int32)
                mine = oracle.spmm_i8(m, n, rp, ci, vi, Bi, ldb, brow, opb, Ci, ldc, crow, 3, -2, saturate=False)
                ref = oracle.ref_spmm_i8(m, n, rp, ci, vi, Bi, ldb, brow, opb, Ci, ldc, crow, 3, -2)
                assert np.array_equal(mine, ref)


@pytest.mark.parametrize("triple", [("f32", "f32", "f32"), ("f32", "f16", "f32"), ("f32", "f16", "f16"),
                                    ("f32", "bf16", "f32"), ("f32", "bf16", "bf16"), ("i32", "i32", "i32"),
                                    ("f32", "i32", "f32")])
@pytest.mark.parametrize("trans", [False, True])
def test_ref_spmv_random(oracle, triple, trans):
    _need_ref(oracle, "spmv")
    comp, vt, ot = triple
    rng = np.random.default_rng(hash((triple, trans)) % 2**32)
    M, N = int(rng.integers(1, 200)), int(rng.integers(1, 300))
    L = rng.binomial(N, 0.1, size=M)
    rp = np.zeros(M + 1, np.int32)
    rp[1:] = np.cumsum(L)
    ci = np.concatenate([np.sort(rng.choice(N, size=int(x), replace=False)) for x in L] + [np.zeros(0, np.int64)]).astype(np.int32)
    xs, ys = (M, N) if trans else (N, M)

    def draw(n, t):
        if t == "i32":
            return rng.integers(-1000, 1000, n).astype(np.int32)
        f = rng.uniform(-5, 5, n).astype(np.float32)
        return oracle.f32_to_bf16_trunc(f) if t == "bf16" else oracle.to_storage(f, t)

    val, x, y = draw(rp[-1], vt), draw(xs, vt), draw(ys, ot)
    a, b = (3, -2) if comp == "i32" else (1.5, 0.5)
    mine = oracle.spmv_typed(rp, ci, val, x, y, a, b, comp, vt, ot, trans=trans, cols=N, bf16_trunc=True)
    ref = oracle.ref_spmv(rp, ci, val, x, y, a, b, comp, vt, ot, trans=trans, cols=N)
    assert np.array_equal(mine, ref)


# ---- CSR producers and SDDMM: the restatements against the committed fixtures (everywhere) and against the
# reference's golden headers compiled in place (where oracle/_ref holds them) --------------------------------

def test_fixture_convert(oracle, golden_dir):
    z = np.load(golden_dir / "convert.npz")
    for name in z["sort_names"]:
        for base in (0, 1):
            k = f"sort/{name}/{base}"
            co, po = oracle.csrsort(z[f"{k}/row_ptr"], z[f"{k}/col_ind"], np.arange(z[f"{k}/col_ind"].size, dtype=np.int32), base)
            assert np.array_equal(co, z[f"{k}/col_out"]) and np.array_equal(po, z[f"{k}/perm_out"]), k
    for name in z["coo_names"]:
        for base in (0, 1):
            k = f"coo/{name}/{base}"
            assert np.array_equal(oracle.coo2csr(z[f"{k}/rows"], int(z[f"{k}/m"][0]), base), z[f"{k}/row_ptr"]), k
    for name in z["csc_names"]:
        for base in (0, 1):
            k = f"csc/{name}/{base}"
            m, n = (int(v) for v in z[f"{k}/shape"])
            cp, ri, vo = oracle.csr2csc(m, n, z[f"{k}/row_ptr"], z[f"{k}/col_ind"], z[f"{k}/val"], base)
            assert np.array_equal(cp, z[f"{k}/col_ptr"]) and np.array_equal(ri, z[f"{k}/row_ind"]), k
            assert np.array_equal(vo, z[f"{k}/val_out"]), k


def sddmm_case(oracle, z, name):
    """Inputs and golden of one fixture case, the golden's inputs quantised as the reference test does."""
    m, k, n = (int(v) for v in z[f"{name}/shape"])
    alpha, beta = (float(v) for v in z[f"{name}/scalars"])
    dtype = str(z[f"{name}/dtype"][0])
    X, Yt, c0 = z[f"{name}/X"], z[f"{name}/Yt"], z[f"{name}/c_init"]
    gx, gy, gc, ga, gb = X, Yt, c0, alpha, beta
    if dtype == "f16":
        q = lambda a: oracle.f16_to_f32(oracle.f32_to_f16(np.asarray(a, np.float64).astype(np.float32))).astype(np.float64)
        gx, gy, gc = q(X), q(Yt), q(c0)
        ga, gb = float(q([alpha])[0]), float(q([beta])[0])
    gold = oracle.sddmm_f64(m, n, k, gx, gy, z[f"{name}/row_offsets"], z[f"{name}/col_ind"], gc, ga, gb, False, True)
    return m, k, n, alpha, beta, dtype, X, Yt, c0, gold


def test_fixture_sddmm(oracle, golden_dir):
    z = np.load(golden_dir / "sddmm.npz")
    for name in z["names"]:
        gold = sddmm_case(oracle, z, name)[-1]
        assert np.array_equal(gold.view(np.uint64), z[f"{name}/gold"].view(np.uint64)), name


def test_convert_and_sddmm_against_reference_headers(oracle):
    if not (oracle.ref_available("convert") and oracle.ref_available("sddmm")):
        pytest.skip("oracle/_ref holds no golden headers of the reference on this machine")
    rng = np.random.default_rng(99)
    for trial in range(25):
        m, n = int(rng.integers(1, 300)), int(rng.integers(1, 400))
        base = int(rng.integers(0, 2))
        lengths = rng.integers(0, min(n, 60) + 1, size=m)
        rp = np.zeros(m + 1, np.int32)
        rp[1:] = np.cumsum(lengths)
        ci = rng.integers(0, n, size=int(rp[-1])).astype(np.int32)      # duplicates, unsorted
        perm = rng.permutation(ci.size).astype(np.int32)
        a, b = oracle.csrsort(rp + base, ci + base, perm, base), oracle.ref_csrsort(rp + base, ci + base, perm, base)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
        rows = np.sort(rng.integers(-2, m + 2, size=int(rng.integers(0, 500)))).astype(np.int32) + base  # some out of range
        assert np.array_equal(oracle.coo2csr(rows, m, base), oracle.ref_coo2csr(rows, m, base))
        for dt in (np.uint8, np.uint16, np.uint32):
            vals = rng.integers(0, 200, size=ci.size).astype(dt)
            x, y = oracle.csr2csc(m, n, rp + base, ci + base, vals, base), oracle.ref_csr2csc(m, n, rp + base, ci + base, vals, base)
            assert all(np.array_equal(p, q) for p, q in zip(x, y))
        mm, nn, kk = int(rng.integers(1, 40)), int(rng.integers(1, 40)), int(rng.integers(1, 70))
        ro, cc, cv = oracle.ref_sddmm_sparsity(mm, nn, float(rng.choice([0.0, 0.3, 1.0])), -1.0, 1.0, trial)
        for opx in (False, True):
            for opy in (False, True):
                X, Y = rng.standard_normal(mm * kk), rng.standard_normal(kk * nn)
                g1 = oracle.sddmm_f64(mm, nn, kk, X, Y, ro, cc, cv, 1.25, -0.5, opx, opy)
                g2 = oracle.ref_sddmm_f64(mm, nn, kk, X, Y, ro, cc, cv, 1.25, -0.5, opx, opy)
                assert np.array_equal(g1.view(np.uint64), g2.view(np.uint64))
    # the frame's mixed-tolerance verdict and the SDDMM test's fp16 converters
    allh = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(oracle.f16_to_f32(allh).view(np.uint32), oracle.ref_sddmm_f16_to_f32(allh).view(np.uint32))
    x = (rng.standard_normal(200000) * 10.0 ** rng.integers(-9, 6, 200000)).astype(np.float32)
    assert np.array_equal(oracle.f32_to_f16(x), oracle.ref_sddmm_f32_to_f16(x))
    for kind, noise in (("f32", 1e-6), ("f32", 1e-3), ("f16", 1e-3), ("f16", 1e-2), ("bf16", 1e-2), ("bf16", 1e-1)):
        g = rng.standard_normal(4000).astype(np.float32)
        out = (g + noise * rng.standard_normal(4000)).astype(np.float32)
        assert oracle.verify_mixed_tolerance(out, g, kind)[0] == oracle.ref_verify_mixed_tolerance(out, g, kind), (kind, noise)
