"""ctypes view of the CPU oracle (oracle/_build/liboracle.so) and, when built, of the
reference's own golden functions (oracle/_ref/libref_*.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the CPU-baseline
legs of bench.py, never by the shipped package.  Arrays are numpy; 16-bit floats travel as
uint16 bit patterns.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "liboracle.so"
REF_DIR = HERE / "_ref"

F32, F16, BF16, I32, I8 = 0, 1, 2, 3, 4
_TYPE_OF = {"f32": F32, "f16": F16, "bf16": BF16, "i32": I32, "i8": I8}
_NP_OF = {F32: np.float32, F16: np.uint16, BF16: np.uint16, I32: np.int32, I8: np.int8}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python oracle/build_oracle.py`")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.oracle_hardware_threads.restype = c_int
        _lib.oracle_verify_abs_and_rel.restype = c_int64
    return _lib


def type_id(name) -> int:
    return name if isinstance(name, int) else _TYPE_OF[name]


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def hardware_threads() -> int:
    return int(lib().oracle_hardware_threads())


# ---- 16-bit conversions ------------------------------------------------------------------

def _convert(fn: str, a: np.ndarray, src, dst) -> np.ndarray:
    a = _c(a, src)
    out = np.empty(a.shape, dtype=dst)
    getattr(lib(), fn)(_p(a), _p(out), c_int64(a.size))
    return out


def f32_to_f16(a): return _convert("oracle_f32_to_f16", a, np.float32, np.uint16)
def f16_to_f32(a): return _convert("oracle_f16_to_f32", a, np.uint16, np.float32)
def f32_to_bf16(a): return _convert("oracle_f32_to_bf16_rne", a, np.float32, np.uint16)
def f32_to_bf16_trunc(a): return _convert("oracle_f32_to_bf16_trunc", a, np.float32, np.uint16)
def bf16_to_f32(a): return _convert("oracle_bf16_to_f32", a, np.uint16, np.float32)


def to_storage(a: np.ndarray, t) -> np.ndarray:
    """fp32 / int data -> the array the kernels read for element type t (bits for 16-bit floats)."""
    t = type_id(t)
    if t == F16:
        return f32_to_f16(a)
    if t == BF16:
        return f32_to_bf16(a)
    return _c(a, _NP_OF[t])


def from_storage(a: np.ndarray, t) -> np.ndarray:
    t = type_id(t)
    if t == F16:
        return f16_to_f32(a)
    if t == BF16:
        return bf16_to_f32(a)
    return np.asarray(a)


# ---- SpMV -----------------------------------------------------------------------------------

def spmv_typed(row_ptr, col_ind, val, x, y, alpha, beta, comp="f32", val_type="f32", out_type="f32",
               trans=False, cols=None, bf16_trunc=False, threads=1) -> np.ndarray:
    """Golden SpMV on storage-typed arrays; returns y_out in out_type storage."""
    comp, vt, ot = type_id(comp), type_id(val_type), type_id(out_type)
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, x, y = _c(val, _NP_OF[vt]), _c(x, _NP_OF[vt]), _c(y, _NP_OF[ot])
    rows = row_ptr.size - 1
    out = np.empty_like(y)
    sc = (c_int32 if comp == I32 else c_float)
    a, b = sc(alpha), sc(beta)
    if trans:
        assert cols is not None
        out = y.copy()
        rc = lib().oracle_spmv_trans(_p(row_ptr), _p(col_ind), _p(val), _p(x), _p(y), _p(out), c_int64(rows),
                                     c_int64(cols), comp, vt, ot, ctypes.byref(a), ctypes.byref(b), int(bf16_trunc))
    else:
        out = y.copy()
        rc = lib().oracle_spmv(_p(row_ptr), _p(col_ind), _p(val), _p(x), _p(y), _p(out), c_int64(rows), comp, vt, ot,
                               ctypes.byref(a), ctypes.byref(b), int(bf16_trunc), int(threads))
    if rc != 0:
        raise ValueError("type combination without a golden instantiation")
    return out


def spmv(row_ptr, col_ind, val, x, y, alpha=1.0, beta=0.0, threads=1) -> np.ndarray:
    """fp32 golden SpMV, result as float64 for error arithmetic."""
    return spmv_typed(row_ptr, col_ind, val, x, y, alpha, beta, threads=threads).astype(np.float64)


def spmv_abs_rowsum(row_ptr, col_ind, val, x, val_type="f32") -> np.ndarray:
    vt = type_id(val_type)
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, x = _c(val, _NP_OF[vt]), _c(x, _NP_OF[vt])
    out = np.empty(row_ptr.size - 1, dtype=np.float64)
    lib().oracle_spmv_abs_rowsum(_p(row_ptr), _p(col_ind), _p(val), _p(x), vt, c_int64(out.size), _p(out))
    return out


# ---- SpMM -----------------------------------------------------------------------------------

def spmm_f32_layout(m, n, row_ptr, col_ind, val, B, ldb, b_row_major, op_b_t, C, ldc, c_row_major, alpha, beta,
                    threads=1) -> np.ndarray:
    """Golden fp32 SpMM on flat storage arrays with explicit layout; returns the new C storage."""
    row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np.float32)
    B = _c(B, np.float32).ravel()
    out = _c(C, np.float32).ravel().copy()
    lib().oracle_spmm_f32(c_int64(m), c_int64(n), _p(row_ptr), _p(col_ind), _p(val), _p(B), c_int64(ldb),
                          int(b_row_major), int(op_b_t), _p(out), c_int64(ldc), int(c_row_major), c_float(alpha),
                          c_float(beta), int(threads))
    return out


def spmm_f32(row_ptr, col_ind, val, B, C, alpha=1.0, beta=0.0, threads=1) -> np.ndarray:
    """Compact row-major fp32 golden SpMM; result (m, n) as float64."""
    B, C = _c(B, np.float32), _c(C, np.float32)
    m, n = C.shape
    out = spmm_f32_layout(m, n, row_ptr, col_ind, val, B, n, True, False, C, n, True, alpha, beta, threads)
    return out.reshape(m, n).astype(np.float64)


def spmm_16(row_ptr, col_ind, val_bits, B_bits, C_store, alpha, beta, in_type, out_type, ldb=None, ldc=None,
            b_row_major=True, op_b_t=False, c_row_major=True, m=None, n=None, threads=1) -> np.ndarray:
    """Golden SpMM with 16-bit A / B storage; C_store is out_type storage; returns new C storage."""
    it, ot = type_id(in_type), type_id(out_type)
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val_bits, B_bits = _c(val_bits, np.uint16), _c(B_bits, np.uint16)
    out = _c(C_store, _NP_OF[ot]).copy()
    if m is None:
        m, n = out.shape
    ldb = ldb if ldb is not None else n
    ldc = ldc if ldc is not None else n
    rc = lib().oracle_spmm_16(c_int64(m), c_int64(n), c_int64(val_bits.size), _p(row_ptr), _p(col_ind), _p(val_bits),
                              _p(B_bits), c_int64(B_bits.size), c_int64(ldb), int(b_row_major), int(op_b_t), _p(out),
                              c_int64(out.size), c_int64(ldc), int(c_row_major), c_float(alpha), c_float(beta), it, ot,
                              int(threads))
    if rc != 0:
        raise ValueError("unsupported 16-bit type combination")
    return out


def spmm_i8(m, n, row_ptr, col_ind, val, B, ldb, b_row_major, op_b_t, C, ldc, c_row_major, alpha, beta,
            saturate=True) -> np.ndarray:
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, B = _c(val, np.int8), _c(B, np.int8).ravel()
    out = _c(C, np.int32).ravel().copy()
    lib().oracle_spmm_i8(c_int64(m), c_int64(n), _p(row_ptr), _p(col_ind), _p(val), _p(B), c_int64(ldb),
                         int(b_row_major), int(op_b_t), _p(out), c_int64(ldc), int(c_row_major), c_int32(alpha),
                         c_int32(beta), int(saturate))
    return out


def spmm_abs_sum(row_ptr, col_ind, val, B, val_type="f32") -> np.ndarray:
    vt = type_id(val_type)
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, B = _c(val, _NP_OF[vt]), _c(B, _NP_OF[vt])
    m, n = row_ptr.size - 1, B.shape[1]
    out = np.empty((m, n), dtype=np.float64)
    lib().oracle_spmm_abs_sum(_p(row_ptr), _p(col_ind), _p(val), _p(B), vt, c_int64(m), c_int64(n), _p(out))
    return out


# ---- CSR producers and SDDMM -------------------------------------------------------------------------

def csrsort(row_ptr, col_ind, perm, index_base=0):
    """(sorted col_ind, permuted perm): golden of aclsparseXcsrsort."""
    row_ptr, col_ind, perm = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(perm, np.int32)
    co, po = col_ind.copy(), perm.copy()
    lib().oracle_csrsort(_p(row_ptr), _p(col_ind), _p(perm), int(row_ptr.size - 1), int(index_base), _p(co), _p(po))
    return co, po


def coo2csr(coo_row, m, index_base=0):
    coo_row = _c(coo_row, np.int32)
    out = np.empty(m + 1, dtype=np.int32)
    lib().oracle_coo2csr(_p(coo_row), int(coo_row.size), int(m), int(index_base), _p(out))
    return out


def csr2csc(m, n, row_ptr, col_ind, values, index_base=0):
    """(col_ptr, row_ind, values in CSC order); values of any 1-, 2- or 4-byte dtype move as raw bytes."""
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    values = np.ascontiguousarray(values)
    cp, ri, vo = np.empty(n + 1, dtype=np.int32), np.empty(col_ind.size, dtype=np.int32), np.empty_like(values)
    lib().oracle_csr2csc(int(m), int(n), int(col_ind.size), _p(row_ptr), _p(col_ind), _p(values),
                         int(values.dtype.itemsize), int(index_base), _p(cp), _p(ri), _p(vo))
    return cp, ri, vo


def sddmm_f64(m, n, k, X, Y, row_offsets, col_ind, c_init, alpha, beta, op_x_t=False, op_y_t=False):
    X, Y, c_init = _c(X, np.float64).ravel(), _c(Y, np.float64).ravel(), _c(c_init, np.float64)
    row_offsets, col_ind = _c(row_offsets, np.int32), _c(col_ind, np.int32)
    out = np.zeros(col_ind.size, dtype=np.float64)
    lib().oracle_sddmm_f64(c_int64(m), c_int64(n), c_int64(k), _p(X), _p(Y), _p(row_offsets), _p(col_ind),
                           _p(c_init), c_double(alpha), c_double(beta), int(op_x_t), int(op_y_t), _p(out))
    return out


FRAME_MIXED_TOL = {  # rtol, atol, fixed per-element limit, mantissa bits, emin (test/frame/verify.h:214-226)
    "f16": (0.001953125, 0.001953125, 1e-1, 10, -14),
    "bf16": (0.015625, 0.015625, 1.0, 7, -126),
    "f32": (0.0009765625, 1.52587890625e-5, 1e-2, 23, -126),
}


def verify_mixed_tolerance(out, gold, kind="f32"):
    """The reference test frame's MIXED_TOLERANCE verdict: (passed, {matched, max_abs_err})."""
    rtol, atol, limit, mant, emin = FRAME_MIXED_TOL[kind]
    out, gold = _c(out, np.float32).ravel(), _c(gold, np.float32).ravel()
    stats = np.zeros(2, dtype=np.float64)
    ok = lib().oracle_verify_mixed_tolerance(_p(out), _p(gold), c_int64(out.size), c_double(rtol), c_double(atol),
                                             c_double(limit), int(mant), int(emin), c_double(0.99), _p(stats))
    return ok == 1, {"matched": float(stats[0]), "max_abs_err": float(stats[1])}


# ---- whole-result checks at benchmark size --------------------------------------------------------

def check_spmv_f32(row_ptr, col_ind, val, x, y_old, got, alpha, beta, tol, threads=None):
    """(outputs outside the per-row tolerance, worst err / scale) of a full-size SpMV result against the golden;
    val / x widened to fp32 by the caller (exact for 16-bit storage), threaded over rows."""
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, x, y_old, got = _c(val, np.float32), _c(x, np.float32), _c(y_old, np.float32), _c(got, np.float32)
    worst = c_double(0.0)
    f = lib().oracle_check_spmv_f32
    f.restype = c_int64
    bad = f(_p(row_ptr), _p(col_ind), _p(val), _p(x), _p(y_old), _p(got), c_int64(row_ptr.size - 1), c_float(alpha),
            c_float(beta), c_double(tol), int(threads or hardware_threads()), ctypes.byref(worst))
    return int(bad), float(worst.value)


def check_spmm_f32(row_ptr, col_ind, val, B, C_old, got, alpha, beta, tol, threads=None):
    """The same for SpMM with compact row-major B, C_old and got (all fp32, shapes (k, n), (m, n), (m, n))."""
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, B, C_old, got = _c(val, np.float32), _c(B, np.float32), _c(C_old, np.float32), _c(got, np.float32)
    m, n = got.shape
    worst = c_double(0.0)
    f = lib().oracle_check_spmm_f32
    f.restype = c_int64
    bad = f(_p(row_ptr), _p(col_ind), _p(val), _p(B), _p(C_old), _p(got), c_int64(m), c_int64(n), c_float(alpha),
            c_float(beta), c_double(tol), int(threads or hardware_threads()), ctypes.byref(worst))
    return int(bad), float(worst.value)


# ---- verifiers --------------------------------------------------------------------------------

MIXED_TOL = {  # rtol, atol, max-abs-error limit, required matched ratio (spmv_test.cpp:208-220)
    "f32": (2.0 ** -10, 2.0 ** -16, 1e-2, 0.99),
    "f16": (2.0 ** -9, 2.0 ** -9, 1e-1, 0.99),
    "bf16": (2.0 ** -6, 2.0 ** -6, 1.0, 0.99),
}


def spmv_op(row_offsets, col_ind, val, x, y, alpha, beta, index_base=0) -> np.ndarray:
    """Z = alpha A X + beta Y with the reference's doubly compensated row sums (fp32); row_offsets int32 or int64."""
    ro = np.ascontiguousarray(row_offsets)
    assert ro.dtype in (np.int32, np.int64)
    rows = ro.size - 1
    ci, v = _c(col_ind, np.int32), _c(val, np.float32)
    xx, yy = _c(x, np.float32), _c(y, np.float32)
    z = np.empty(rows, np.float32)
    f = lib().oracle_spmv_op
    f.restype = None
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                  ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_float]
    f(_p(ro), int(ro.dtype == np.int64), _p(ci), _p(v), _p(xx), _p(yy), _p(z), rows, int(index_base), float(alpha),
      float(beta))
    return z


def spmv_exact(row_offsets, col_ind, val, x, y, alpha, beta, index_base=0):
    """(alpha A x + beta y, sum_j |a_ij x_j|) in fp64 from fp32 inputs: the products are exact in fp64, the sums
    are not, but their error is far below fp32 resolution for the sizes the tests use."""
    ro = np.asarray(row_offsets, np.int64) - index_base
    ci = np.asarray(col_ind, np.int64) - index_base
    prod = np.asarray(val, np.float64) * np.asarray(x, np.float64)[ci]
    rows = ro.size - 1
    seg = np.repeat(np.arange(rows), np.diff(ro))
    dot = np.bincount(seg, weights=prod, minlength=rows)[:rows]
    mag = np.bincount(seg, weights=np.abs(prod), minlength=rows)[:rows]
    yy = np.asarray(y, np.float64)
    z = np.float64(np.float32(alpha)) * dot + (np.float64(np.float32(beta)) * yy if beta != 0 else 0.0)
    return z, mag


def verify_mixed(gold, got, kind="f32"):
    rtol, atol, limit, ratio = MIXED_TOL[kind]
    gold, got = _c(gold, np.float32).ravel(), _c(got, np.float32).ravel()
    stats = np.zeros(2, dtype=np.float32)
    rc = lib().oracle_verify_mixed(_p(gold), _p(got), c_int64(gold.size), c_float(rtol), c_float(atol),
                                   c_float(limit), c_float(ratio), _p(stats))
    return rc == 0, {"matched": float(stats[0]), "max_abs_err": float(stats[1])}


def verify_mere_mare(got, gold, m, n, ldc, c_row_major=True, mere_thr=2.0 ** -13, mare_thr=10 * 2.0 ** -13):
    got, gold = _c(got, np.float32).ravel(), _c(gold, np.float32).ravel()
    stats = np.zeros(3, dtype=np.float64)
    rc = lib().oracle_verify_mere_mare(_p(got), _p(gold), c_int64(m), c_int64(n), c_int64(ldc), int(c_row_major),
                                       c_double(mere_thr), c_double(mare_thr), _p(stats))
    return rc == 0, {"mere": stats[0], "mare": stats[1], "mae": stats[2]}


def verify_abs_and_rel(got, gold, rel_tol=1e-3, abs_tol=1e-3) -> int:
    got, gold = _c(got, np.float32).ravel(), _c(gold, np.float32).ravel()
    return int(lib().oracle_verify_abs_and_rel(_p(got), _p(gold), c_int64(got.size), c_float(rel_tol),
                                               c_float(abs_tol)))


# ---- the reference's own golden code (present only where oracle/_ref was built) ---------------

_ref_libs: dict[str, ctypes.CDLL] = {}


def ref_available(name: str) -> bool:
    return (REF_DIR / f"libref_{name}.so").exists()


def ref_lib(name: str) -> ctypes.CDLL:
    if name not in _ref_libs:
        _ref_libs[name] = ctypes.CDLL(str(REF_DIR / f"libref_{name}.so"))
    return _ref_libs[name]


def ref_spmv(row_ptr, col_ind, val, x, y, alpha, beta, comp="f32", val_type="f32", out_type="f32", trans=False,
             cols=None) -> np.ndarray:
    """SpmvCpu / SpmvTransCpu of the reference harness itself (bf16 = its truncating host type)."""
    comp, vt, ot = type_id(comp), type_id(val_type), type_id(out_type)
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, x, y = _c(val, _NP_OF[vt]), _c(x, _NP_OF[vt]), _c(y, _NP_OF[ot])
    rows = row_ptr.size - 1
    ncols = int(cols) if cols is not None else (int(x.size) if not trans else int(y.size))
    out = np.empty_like(y)
    sc = (c_int32 if comp == I32 else c_float)
    a, b = sc(alpha), sc(beta)
    rc = ref_lib("spmv").ref_spmv(_p(row_ptr), _p(col_ind), _p(val), _p(x), _p(y), _p(out), c_int64(rows),
                                  c_int64(ncols), c_int64(col_ind.size), int(trans), comp, vt, ot, ctypes.byref(a),
                                  ctypes.byref(b))
    if rc != 0:
        raise ValueError("the reference harness has no such instantiation")
    return out


def ref_spmm_f32(m, n, row_ptr, col_ind, val, B, ldb, b_row_major, op_b_t, C, ldc, c_row_major, alpha, beta):
    row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np.float32)
    B = _c(B, np.float32).ravel()
    out = _c(C, np.float32).ravel().copy()
    ref_lib("spmm35").ref_spmm_f32(c_int32(m), c_int32(n), c_int64(col_ind.size), _p(row_ptr), _p(col_ind), _p(val),
                                   _p(B), c_int64(B.size), c_int32(ldb), int(b_row_major), int(op_b_t), _p(out),
                                   c_int64(out.size), c_int32(ldc), int(c_row_major), c_float(alpha), c_float(beta))
    return out


def ref_spmm_i8(m, n, row_ptr, col_ind, val, B, ldb, b_row_major, op_b_t, C, ldc, c_row_major, alpha, beta):
    row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np.int8)
    B = _c(B, np.int8).ravel()
    out = _c(C, np.int32).ravel().copy()
    ref_lib("spmm35").ref_spmm_i8(c_int32(m), c_int32(n), c_int64(col_ind.size), _p(row_ptr), _p(col_ind), _p(val),
                                  _p(B), c_int64(B.size), c_int32(ldb), int(b_row_major), int(op_b_t), _p(out),
                                  c_int64(out.size), c_int32(ldc), int(c_row_major), c_int32(alpha), c_int32(beta))
    return out


def ref_f32_to_f16(a):
    a = _c(a, np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    ref_lib("spmm35").ref_f32_to_f16(_p(a), _p(out), c_int64(a.size))
    return out


def ref_f16_to_f32(a):
    a = _c(a, np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    ref_lib("spmm35").ref_f16_to_f32(_p(a), _p(out), c_int64(a.size))
    return out


def ref_generate_random_csr(seed, m, k, nnz):
    rp = np.zeros(m + 1, dtype=np.int32)
    ci = np.zeros(max(nnz, 1), dtype=np.int32)
    v = np.zeros(max(nnz, 1), dtype=np.float32)
    fn = ref_lib("spmm35").ref_generate_random_csr
    fn.restype = c_int32
    got = fn(c_uint32(seed), c_int32(m), c_int32(k), c_int32(nnz), _p(rp), _p(ci), _p(v))
    return rp, ci[:got], v[:got]


def ref_generate_csr22(dist, rows, cols, nnz):
    rp = np.zeros(rows + 1, dtype=np.int32)
    ci = np.zeros(max(nnz, 1), dtype=np.int32)
    v = np.zeros(max(nnz, 1), dtype=np.float32)
    ref_lib("spmm22").ref_generate_csr(int(dist), c_uint64(rows), c_uint64(cols), c_uint64(nnz), _p(rp), _p(ci), _p(v))
    n = int(rp[-1])
    return rp, ci[:n], v[:n]


def ref_spmm_csr_cpu(M, K, N, row_ptr, col_ind, val, B, C, alpha, beta):
    row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np.float32)
    B, C = _c(B, np.float32), _c(C, np.float32)
    Y = np.empty_like(C)
    ref_lib("spmm22").ref_spmm_csr_cpu(c_uint64(M), c_uint64(K), c_uint64(N), _p(row_ptr), _p(col_ind), _p(val), _p(B),
                                       _p(C), _p(Y), c_float(alpha), c_float(beta))
    return Y


# ---- CPU-baseline timing ----------------------------------------------------------------------

def time_spmv_f32(row_ptr, col_ind, val, x, y, alpha, beta, threads: int, reps: int):
    """Times `reps` SpMV passes on the host.  Returns (per-pass seconds array, kind): kind is
    "reference" when the reference harness's own SpmvCpu was timed (oracle/_ref present), else
    "port" (oracle.cpp).  Argument set-up is outside the clock."""
    import time
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    val, x, y = _c(val, np.float32), _c(x, np.float32), _c(y, np.float32)
    rows = row_ptr.size - 1
    per = np.zeros(max(reps, 1), dtype=np.float64)
    if ref_available("spmv"):
        fn = ref_lib("spmv").ref_spmv_bench_f32
        fn.restype = c_double
        fn(_p(row_ptr), _p(col_ind), _p(val), _p(x), _p(y), c_int64(rows), c_int64(x.size), c_int64(col_ind.size),
           c_float(alpha), c_float(beta), int(threads), int(reps), _p(per))
        return per[:reps], "reference"
    for r in range(reps):
        t0 = time.perf_counter()
        spmv_typed(row_ptr, col_ind, val, x, y, alpha, beta, threads=threads)
        per[r] = time.perf_counter() - t0
    return per[:reps], "port"


def time_spmm_f32(row_ptr, col_ind, val, B, C, alpha, beta, threads: int, reps: int):
    """Times `reps` SpMM passes (compact row-major fp32) on the host; see time_spmv_f32."""
    import time
    row_ptr, col_ind, val = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(val, np.float32)
    B, C = _c(B, np.float32), _c(C, np.float32)
    m, n = C.shape
    per = np.zeros(max(reps, 1), dtype=np.float64)
    if ref_available("spmm35"):
        fn = ref_lib("spmm35").ref_spmm_bench_f32
        fn.restype = c_double
        fn(c_int32(m), c_int32(B.shape[0]), c_int32(n), c_int64(col_ind.size), _p(row_ptr), _p(col_ind), _p(val),
           _p(B), _p(C), c_float(alpha), c_float(beta), int(threads), int(reps), _p(per))
        return per[:reps], "reference"
    for r in range(reps):
        t0 = time.perf_counter()
        spmm_f32(row_ptr, col_ind, val, B, C, alpha, beta, threads=threads)
        per[r] = time.perf_counter() - t0
    return per[:reps], "port"


def ref_csrsort(row_ptr, col_ind, perm, index_base=0):
    row_ptr, col_ind, perm = _c(row_ptr, np.int32), _c(col_ind, np.int32), _c(perm, np.int32)
    co, po = np.empty_like(col_ind), np.empty_like(perm)
    ref_lib("convert").ref_csrsort(_p(row_ptr), _p(col_ind), _p(perm), int(row_ptr.size - 1), int(col_ind.size),
                                   int(index_base), _p(co), _p(po))
    return co, po


def ref_coo2csr(coo_row, m, index_base=0):
    coo_row = _c(coo_row, np.int32)
    out = np.empty(m + 1, dtype=np.int32)
    rc = ref_lib("convert").ref_coo2csr(_p(coo_row), int(coo_row.size), int(m), int(index_base), _p(out))
    assert rc == 0
    return out


def ref_csr2csc(m, n, row_ptr, col_ind, values, index_base=0):
    row_ptr, col_ind = _c(row_ptr, np.int32), _c(col_ind, np.int32)
    values = np.ascontiguousarray(values)
    cp, ri, vo = np.empty(n + 1, dtype=np.int32), np.empty(col_ind.size, dtype=np.int32), np.empty_like(values)
    rc = ref_lib("convert").ref_csr2csc(int(m), int(n), int(col_ind.size), _p(row_ptr), _p(col_ind), _p(values),
                                        int(values.dtype.itemsize), int(index_base), _p(cp), _p(ri), _p(vo))
    assert rc == 0
    return cp, ri, vo


def ref_sddmm_f64(m, n, k, X, Y, row_offsets, col_ind, c_init, alpha, beta, op_x_t=False, op_y_t=False):
    X, Y, c_init = _c(X, np.float64).ravel(), _c(Y, np.float64).ravel(), _c(c_init, np.float64)
    row_offsets, col_ind = _c(row_offsets, np.int32), _c(col_ind, np.int32)
    out = np.zeros(col_ind.size, dtype=np.float64)
    ref_lib("sddmm").ref_sddmm_f64(c_int64(m), c_int64(n), c_int64(k), _p(X), c_int64(X.size), _p(Y), c_int64(Y.size),
                                   _p(row_offsets), _p(col_ind), _p(c_init), c_int64(col_ind.size), c_double(alpha),
                                   c_double(beta), int(op_x_t), int(op_y_t), _p(out))
    return out


def ref_sddmm_sparsity(m, n, ratio, lo, hi, seed):
    """(row_offsets, col_ind, fp64 values) of the reference's deterministic SDDMM pattern generator."""
    f = ref_lib("sddmm").ref_sddmm_sparsity
    f.restype = c_int64
    nnz = f(c_int64(m), c_int64(n), c_double(ratio), c_double(lo), c_double(hi), c_uint32(seed), None, None, None)
    ro, ci, v = np.zeros(m + 1, np.int32), np.zeros(nnz, np.int32), np.zeros(nnz, np.float64)
    f(c_int64(m), c_int64(n), c_double(ratio), c_double(lo), c_double(hi), c_uint32(seed), _p(ro), _p(ci), _p(v))
    return ro, ci, v


def ref_sddmm_f32_to_f16(a):
    a = _c(a, np.float32).ravel()
    out = np.empty(a.size, dtype=np.uint16)
    ref_lib("sddmm").ref_sddmm_f32_to_f16(_p(a), _p(out), c_int64(a.size))
    return out


def ref_sddmm_f16_to_f32(a):
    a = _c(a, np.uint16).ravel()
    out = np.empty(a.size, dtype=np.float32)
    ref_lib("sddmm").ref_sddmm_f16_to_f32(_p(a), _p(out), c_int64(a.size))
    return out


def ref_verify_mixed_tolerance(out, gold, kind="f32") -> bool:
    out, gold = _c(out, np.float32).ravel(), _c(gold, np.float32).ravel()
    dtype = {"f32": 0, "f16": 1, "bf16": 27}[kind]
    return ref_lib("sddmm").ref_verify_mixed_tolerance(_p(out), _p(gold), c_int64(out.size), dtype) == 1


def ref_sddmm_uniform(seed, lo, hi, n):
    out = np.empty(n, dtype=np.float64)
    ref_lib("sddmm").ref_sddmm_uniform(c_uint32(seed), c_double(lo), c_double(hi), c_int64(n), _p(out))
    return out
