"""Generates the golden fixtures in this directory from the REFERENCE's own golden code.

Needs oracle/_ref/libref_*.so, i.e. a machine where the reference checkout is present and
`python oracle/build_oracle.py` has compiled its harness sources in place.  The fixtures it
writes are what the CPU oracle and the CUDA path are compared against on machines without
the reference.  Run from the repository root:  python tests/golden/make_golden.py

Fixture contents (all small):
  spmm35_fp32.npz   the five fp32 cases of test/spmm/arch35/spmm_test.cpp:964-975 (its seeds,
                    its srand/rand CSR generator, its index-formula B / C), golden = SpmmCpuFp32
  spmm35_f16_i8.npz the fp16 and int8 baseline cases (:978-1000), golden per the harness recipe
  spmm22.npz        a slice of the arch22 case table (test/spmm/arch22/spmm_test.cpp:445-646)
                    with its own uniform / power-law generators, golden = spmm_csr_cpu
  spmv.npz          SpmvCpu / SpmvTransCpu on seeded inputs for all seven type triples (the
                    harness itself is time-seeded, so only its functions are pinned, on inputs
                    drawn here with its distributions: values, x, y ~ U(-5, 5))
  convert.npz       csrsortGolden / Coo2CsrGolden / Csr2CscGolden (test/csrsort/arch35/csrsort_golden.h,
                    test/coo2csr/coo2csr_golden.h, test/csr2csc_ex2/csr2csc_ex2_golden.h) on seeded index
                    arrays, both index bases, duplicates and empty rows included
  sddmm.npz         a slice of the reference's SDDMM case table (test/sddmm/sddmm/arch35/sddmm_test.csv) with
                    its pattern generator, its seeds for X / Y / C and SddmmGolden's fp64 results
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

o = entry.load_oracle()
OUT = Path(__file__).resolve().parent


def formula(n: int) -> np.ndarray:
    """-5 + 10 * (i mod 10001) / 10000 in fp32, the harness's fill for B and C."""
    i = (np.arange(n, dtype=np.int64) % 10001).astype(np.float32)
    return (np.float32(-5.0) + np.float32(10.0) * i / np.float32(10000.0)).astype(np.float32)


def spmm35_fp32():
    cases = [  # name, m, k, n, nnz (0 = m*k/10), alpha, beta, opB_T, B col-major, C col-major, seed
        ("baseline_row_N_beta0", 256, 256, 64, 0, 1.0, 0.0, 0, 0, 0, 42),
        ("opB_transpose", 256, 256, 64, 0, 1.0, 0.0, 1, 0, 0, 43),
        ("B_C_col_major", 256, 256, 64, 0, 1.0, 0.0, 0, 1, 1, 44),
        ("beta_nonzero", 256, 256, 64, 0, 1.0, 0.5, 0, 0, 0, 45),
        ("small_shape", 32, 32, 16, 80, 1.0, 0.0, 0, 0, 0, 46),
    ]
    out = {"names": np.array([c[0] for c in cases])}
    for name, m, k, n, nnz, alpha, beta, opb, bcol, ccol, seed in cases:
        nnz = nnz or m * k // 10
        rp, ci, v = o.ref_generate_random_csr(seed, m, k, nnz)
        ldb = k if bcol else n
        ldc = m if ccol else n
        B = formula(k * ldb)
        C = formula(m * ldc) if beta != 0 else np.zeros(m * ldc, dtype=np.float32)
        gold = o.ref_spmm_f32(m, n, rp, ci, v, B, ldb, not bcol, bool(opb), C, ldc, not ccol, alpha, beta)
        out[f"{name}/shape"] = np.array([m, k, n, ldb, ldc, opb, bcol, ccol], dtype=np.int64)
        out[f"{name}/scalars"] = np.array([alpha, beta], dtype=np.float32)
        out[f"{name}/row_ptr"], out[f"{name}/col_ind"], out[f"{name}/val"] = rp, ci, v
        out[f"{name}/gold"] = gold
    np.savez_compressed(OUT / "spmm35_fp32.npz", **out)


def spmm35_f16_i8():
    m = k = 256
    n = 64
    rp, ci, v = o.ref_generate_random_csr(42, m, k, m * k // 10)
    nnz = ci.size
    out = {"shape": np.array([m, k, n], dtype=np.int64), "row_ptr": rp, "col_ind": ci, "val_f32": v}
    # fp16: round inputs with the harness's converter, fp32 golden loop, clamp, round the output
    vh, Bh = o.ref_f32_to_f16(v), o.ref_f32_to_f16(formula(k * n))
    Ch = o.ref_f32_to_f16(np.zeros(m * n, dtype=np.float32))
    g = o.ref_spmm_f32(m, n, rp, ci, o.ref_f16_to_f32(vh), o.ref_f16_to_f32(Bh), n, True, False,
                       o.ref_f16_to_f32(Ch), n, True, 1.0, 0.0)
    g = np.clip(g, -65504.0, 65504.0).astype(np.float32)
    out["f16_val"], out["f16_B"], out["f16_gold"] = vh, Bh, o.ref_f32_to_f16(g)
    # int8: the harness fills A, B (and C when beta != 0) with (i % 11) - 5  (spmm_test.cpp:780-792)
    va = ((np.arange(nnz) % 11) - 5).astype(np.int8)
    Bi = ((np.arange(k * n) % 11) - 5).astype(np.int8)
    gi = o.ref_spmm_i8(m, n, rp, ci, va, Bi, n, True, False, np.zeros(m * n, dtype=np.int32), n, True, 1, 0)
    out["i8_val"], out["i8_B"], out["i8_gold"] = va, Bi, gi
    # a second int8 case with alpha / beta and a non-zero C
    Ci = ((np.arange(m * n) % 11) - 5).astype(np.int32)
    out["i8_C2"] = Ci
    out["i8_gold2"] = o.ref_spmm_i8(m, n, rp, ci, va, Bi, n, True, False, Ci, n, True, 3, -2)
    np.savez_compressed(OUT / "spmm35_f16_i8.npz", **out)


def spmm22():
    # M, K, N, nnz, alpha, beta, dist (0 uniform, 1 power-law).  The first three are rows of the
    # arch22 case table; the last two add skewed rows (one of them longer than 1024 entries).
    cases = [
        (16, 128, 32, 512, 1.4, 2.0, 0),
        (511, 31, 64, 158, 4.8, 1.9, 0),
        (31, 16, 64, 124, 3.3, -0.5, 1),
        (257, 300, 8, 9000, 1.0, 0.0, 1),
        (64, 4096, 32, 20000, 0.5, 1.0, 1),
    ]
    out = {"count": np.array([len(cases)])}
    for i, (M, K, N, nnz, alpha, beta, dist) in enumerate(cases):
        rp, ci, v = o.ref_generate_csr22(dist, M, K, nnz)
        # the harness's fills (spmm_test.cpp:378-383): B[i] = 0.5 + 0.0001 * (i % 1000), C[i] = 0.01 * (i % 100)
        B = (np.float32(0.5) + np.float32(0.0001) * (np.arange(K * N) % 1000).astype(np.float32)).reshape(K, N)
        C = (np.float32(0.01) * (np.arange(M * N) % 100).astype(np.float32)).reshape(M, N)
        Y = o.ref_spmm_csr_cpu(M, K, N, rp, ci, v, B, C, alpha, beta)
        out[f"{i}/shape"] = np.array([M, K, N, dist], dtype=np.int64)
        out[f"{i}/scalars"] = np.array([alpha, beta], dtype=np.float32)
        out[f"{i}/row_ptr"], out[f"{i}/col_ind"], out[f"{i}/val"] = rp, ci, v
        out[f"{i}/gold"] = Y  # B and C are formulas: tests rebuild them
    np.savez_compressed(OUT / "spmm22.npz", **out)


def spmv():
    triples = [  # comp, val, out
        ("f32", "f32", "f32"), ("f32", "f16", "f32"), ("f32", "f16", "f16"), ("f32", "bf16", "f32"),
        ("f32", "bf16", "bf16"), ("i32", "i32", "i32"), ("f32", "i32", "f32"),
    ]
    shapes = [(120, 200, 0.9, 1.0, 0.0), (65, 33, 0.5, 2.5, -1.5), (16, 256, 0.5, -0.75, 0.25)]
    out = {}
    idx = 0
    for comp, vt, ot in triples:
        for (M, N, sparsity, alpha, beta) in shapes:
            for trans in (False, True):
                rng = np.random.default_rng(7000 + idx)
                lengths = rng.binomial(N, 1.0 - sparsity, size=M)
                lengths[rng.random(M) < 0.05] = 0  # a few empty rows
                rp = np.zeros(M + 1, dtype=np.int32)
                rp[1:] = np.cumsum(lengths)
                ci = np.concatenate([np.sort(rng.choice(N, size=int(L), replace=False)) for L in lengths] +
                                    [np.zeros(0, dtype=np.int64)]).astype(np.int32)
                xs, ys = (M, N) if trans else (N, M)
                if vt == "i32":
                    val = rng.integers(-5, 6, size=ci.size).astype(np.int32)
                    x = rng.integers(-5, 6, size=xs).astype(np.int32)
                    a, b = int(round(alpha)) or 1, int(round(beta))
                else:
                    # bf16 storage by truncation = the reference harness's own host type
                    conv = o.f32_to_bf16_trunc if vt == "bf16" else (lambda z: o.to_storage(z, vt))
                    val = conv(rng.uniform(-5, 5, size=ci.size).astype(np.float32))
                    x = conv(rng.uniform(-5, 5, size=xs).astype(np.float32))
                    a, b = alpha, beta
                if ot == "i32":
                    y = rng.integers(-5, 6, size=ys).astype(np.int32)
                else:
                    convo = o.f32_to_bf16_trunc if ot == "bf16" else (lambda z: o.to_storage(z, ot))
                    y = convo(rng.uniform(-5, 5, size=ys).astype(np.float32))
                gold = o.ref_spmv(rp, ci, val, x, y, a, b, comp, vt, ot, trans=trans, cols=N)
                key = f"{idx}"
                out[f"{key}/types"] = np.array([comp, vt, ot])
                out[f"{key}/dims"] = np.array([M, N, int(trans)], dtype=np.int64)
                out[f"{key}/scalars"] = np.array([a, b], dtype=np.float64)
                out[f"{key}/row_ptr"], out[f"{key}/col_ind"] = rp, ci
                out[f"{key}/val"], out[f"{key}/x"], out[f"{key}/y"], out[f"{key}/gold"] = val, x, y, gold
                idx += 1
    out["count"] = np.array([idx])
    np.savez_compressed(OUT / "spmv.npz", **out)


def convert():
    rng = np.random.default_rng(2026)
    out = {}
    sort_cases = [("tiny", 1, 1, 1.0, False), ("dups", 50, 40, 12.0, True), ("wide", 100, 5000, 30.0, False),
                  ("long", 6, 100000, 1500.0, False), ("many_short", 800, 300, 4.0, True), ("empty", 64, 64, 0.0, False)]
    out["sort_names"] = np.array([c[0] for c in sort_cases])
    for name, m, n, mean_len, dups in sort_cases:
        lengths = rng.poisson(mean_len, size=m).astype(np.int64) if mean_len else np.zeros(m, np.int64)
        if not dups:
            lengths = np.minimum(lengths, n)
        rp = np.zeros(m + 1, np.int32)
        rp[1:] = np.cumsum(lengths)
        cols = [rng.integers(0, n, size=int(k)) if dups else rng.permutation(n)[:int(k)] for k in lengths]
        ci = (np.concatenate(cols) if rp[-1] else np.zeros(0)).astype(np.int32)
        for base in (0, 1):
            perm = np.arange(ci.size, dtype=np.int32)
            co, po = o.ref_csrsort(rp + base, ci + base, perm, base)
            out[f"sort/{name}/{base}/row_ptr"], out[f"sort/{name}/{base}/col_ind"] = rp + base, ci + base
            out[f"sort/{name}/{base}/col_out"], out[f"sort/{name}/{base}/perm_out"] = co, po
            out[f"sort/{name}/{base}/n"] = np.array([n])
    coo_cases = [("one", 1, 1, 0.0), ("small", 7, 30, 0.0), ("half_empty", 1000, 5000, 0.5), ("no_entries", 4096, 0, 0.0),
                 ("no_rows", 0, 0, 0.0)]
    out["coo_names"] = np.array([c[0] for c in coo_cases])
    for name, m, nnz, empty in coo_cases:
        live = np.flatnonzero(rng.random(m) >= empty) if m else np.zeros(0, np.int64)
        rows = np.sort(rng.choice(live, size=nnz)) if (nnz and live.size) else np.zeros(0, np.int64)
        for base in (0, 1):
            r = (rows + base).astype(np.int32)
            out[f"coo/{name}/{base}/rows"], out[f"coo/{name}/{base}/m"] = r, np.array([m])
            out[f"coo/{name}/{base}/row_ptr"] = o.ref_coo2csr(r, m, base)
    csc_cases = [("square", 300, 300, 9.0), ("tall", 800, 50, 3.0), ("flat", 20, 6000, 150.0), ("empty", 10, 12, 0.0)]
    out["csc_names"] = np.array([c[0] for c in csc_cases])
    for name, m, n, mean_len in csc_cases:
        lengths = np.minimum(rng.poisson(mean_len, size=m), n).astype(np.int64) if mean_len else np.zeros(m, np.int64)
        rp = np.zeros(m + 1, np.int32)
        rp[1:] = np.cumsum(lengths)
        ci = (np.concatenate([np.sort(rng.permutation(n)[:int(k)]) for k in lengths]) if rp[-1] else np.zeros(0)).astype(np.int32)
        vals = rng.integers(0, 1 << 31, size=ci.size).astype(np.uint32)
        for base in (0, 1):
            cp, ri, vo = o.ref_csr2csc(m, n, rp + base, ci + base, vals, base)
            out[f"csc/{name}/{base}/shape"] = np.array([m, n])
            out[f"csc/{name}/{base}/row_ptr"], out[f"csc/{name}/{base}/col_ind"], out[f"csc/{name}/{base}/val"] = rp + base, ci + base, vals
            out[f"csc/{name}/{base}/col_ptr"], out[f"csc/{name}/{base}/row_ind"], out[f"csc/{name}/{base}/val_out"] = cp, ri, vo
    np.savez_compressed(OUT / "convert.npz", **out)


def sddmm():
    # name, m, k, n, ratio, alpha, beta, dtype, lo, hi, seed: rows of the reference's case table (op_x = N, op_y = T,
    # row-major operands, as in every row of that table)
    cases = [("L0_01", 128, 64, 128, 0.5, 1.0, 0.0, "f32", -1.0, 1.0, 1), ("L0_02", 64, 32, 64, 0.5, 1.0, 0.0, "f16", -0.5, 0.5, 6),
             ("L1_08", 100, 50, 100, 0.5, -1.0, 0.0, "f32", -1.0, 1.0, 13), ("L1_11", 48, 24, 48, 0.5, 1.0, 1.0, "f32", -1.0, 1.0, 17),
             ("L2_07", 64, 32, 64, 0.0, 1.0, 0.0, "f32", -1.0, 1.0, 21), ("WB_02", 1, 32, 64, 0.5, 1.0, 0.0, "f16", -0.5, 0.5, 23),
             ("WB_05", 64, 1, 64, 0.5, 1.0, 0.0, "f32", -1.0, 1.0, 26), ("WB_07", 1, 64, 100, 1.0, 1.0, 1.0, "f32", -1.0, 1.0, 28),
             ("WB_08", 16, 64, 16, 0.5, 2.0, 0.0, "f16", -50.0, 50.0, 29)]
    out = {"names": np.array([c[0] for c in cases])}
    for name, m, k, n, ratio, alpha, beta, dtype, lo, hi, seed in cases:
        ro, ci, cv = o.ref_sddmm_sparsity(m, n, ratio, lo, hi, seed)
        X = o.ref_sddmm_uniform(seed + 1, lo, hi, m * k)          # m x k row-major
        Yt = o.ref_sddmm_uniform(seed + 2, lo, hi, n * k)         # n x k row-major (op_y = T)
        gx, gy, gc, ga, gb = X, Yt, cv, alpha, beta
        if dtype == "f16":  # the test quantises the golden's inputs through fp16 (sddmm_test.cpp:171-181)
            q = lambda a: o.ref_sddmm_f16_to_f32(o.ref_sddmm_f32_to_f16(a.astype(np.float32))).astype(np.float64)
            gx, gy, gc = q(X), q(Yt), q(cv)
            ga, gb = float(q(np.array([alpha]))[0]), float(q(np.array([beta]))[0])
        gold = o.ref_sddmm_f64(m, n, k, gx, gy, ro, ci, gc, ga, gb, False, True)
        out[f"{name}/shape"] = np.array([m, k, n])
        out[f"{name}/scalars"] = np.array([alpha, beta])
        out[f"{name}/dtype"] = np.array([dtype])
        out[f"{name}/row_offsets"], out[f"{name}/col_ind"], out[f"{name}/c_init"] = ro, ci, cv
        out[f"{name}/X"], out[f"{name}/Yt"], out[f"{name}/gold"] = X, Yt, gold
    np.savez_compressed(OUT / "sddmm.npz", **out)


if __name__ == "__main__":
    for name in ("spmv", "spmm35", "spmm22"):
        if not o.ref_available(name):
            raise SystemExit(f"oracle/_ref/libref_{name}.so is missing: build it where the reference is present")
    spmm35_fp32()
    spmm35_f16_i8()
    spmm22()
    spmv()
    convert()
    sddmm()
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")
