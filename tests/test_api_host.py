"""CPU: host-side logic of the C API that needs no device -- descriptor life cycle, argument
checks and status codes (reference: sparse/common/aclsparse_descr.cpp, aclsparse_auxiliary.cpp),
and that the shared library exports every symbol the headers declare."""
from __future__ import annotations

import re
import subprocess
from ctypes import byref, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
FAKE = c_void_p(0x1000)  # descriptors only store pointers; nothing here dereferences them


def declared_functions():
    names = []
    for header in ("cann_ops_sparse.h", "b200sp_kernels.h", "b200sp_mg.h"):
        text = (ROOT / "include" / header).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b((?:aclsparse|b200sp)\w+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported(pkg):
    out = subprocess.run(["nm", "-D", "--defined-only", str(pkg.LIB_PATH)], capture_output=True, text=True, check=True)
    exported = {line.split()[-1] for line in out.stdout.splitlines() if " T " in line}
    declared = declared_functions()
    assert len(declared) >= 50
    missing = [n for n in declared if n not in exported]
    assert not missing, missing
    L = pkg.lib()
    for n in declared:
        assert getattr(L, n) is not None


def test_status_enum_values(pkg):
    assert pkg.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR == 10 and pkg.ACL_SPARSE_STATUS_NOT_SUPPORTED == 8
    assert pkg.ACL_BF16 == 27 and pkg.ACL_INT32 == 3


def test_dnvec_lifecycle(pkg):
    L, S = pkg.lib(), pkg
    d = c_void_p()
    assert L.aclsparseCreateDnVec(None, 4, FAKE, S.ACL_FLOAT) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCreateDnVec(byref(d), -1, FAKE, S.ACL_FLOAT) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCreateDnVec(byref(d), 4, None, S.ACL_FLOAT) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCreateDnVec(byref(d), 4, FAKE, 12345) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCreateDnVec(byref(d), 0, None, S.ACL_FLOAT) == 0  # empty vector may have no storage
    assert L.aclsparseDestroyDnVec(d) == 0
    assert L.aclsparseCreateDnVec(byref(d), 7, FAKE, S.ACL_FLOAT16) == 0
    size, vals, t = c_int64(), c_void_p(), c_int()
    assert L.aclsparseDnVecGet(d, byref(size), byref(vals), byref(t)) == 0
    assert (size.value, vals.value, t.value) == (7, 0x1000, S.ACL_FLOAT16)
    assert L.aclsparseDnVecGet(d, None, None, None) == 0  # every out-pointer is optional
    assert L.aclsparseDnVecGetValues(d, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseDnVecSetValues(d, c_void_p(0x2000)) == 0
    assert L.aclsparseConstDnVecGetValues(d, byref(vals)) == 0 and vals.value == 0x2000
    assert L.aclsparseDnVecGet(None, byref(size), None, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseDestroyDnVec(d) == 0
    assert L.aclsparseDestroyDnVec(None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    c = c_void_p()
    assert L.aclsparseCreateConstDnVec(byref(c), 3, FAKE, S.ACL_BF16) == 0
    assert L.aclsparseConstDnVecGet(c, byref(size), byref(vals), byref(t)) == 0 and t.value == S.ACL_BF16
    assert L.aclsparseDestroyDnVec(c) == 0


def test_csr_lifecycle(pkg):
    L, S = pkg.lib(), pkg
    d = c_void_p()
    mk = lambda *a: L.aclsparseCreateCsr(byref(d), *a)
    assert L.aclsparseCreateCsr(None, 2, 2, 1, FAKE, FAKE, FAKE, 0, 0, 0, 0) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert mk(-1, 2, 1, FAKE, FAKE, FAKE, 0, 0, 0, 0) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert mk(2, 2, 1, FAKE, FAKE, FAKE, 5, 0, 0, 0) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    assert mk(2, 3, 1, FAKE, FAKE, FAKE, S.ACL_SPARSE_INDEX_64I, S.ACL_SPARSE_INDEX_32I, 0, 0) == 0  # creation allows 64-bit
    assert L.aclsparseDestroySpMat(d) == 0
    assert mk(2, 3, 4, FAKE, FAKE, FAKE, 0, 0, 0, S.ACL_FLOAT) == 0
    fmt, r, c, n, vals = c_int(), c_int64(), c_int64(), c_int64(), c_void_p()
    assert L.aclsparseSpMatGetFormat(d, byref(fmt)) == 0 and fmt.value == S.ACL_SPARSE_FORMAT_CSR
    assert L.aclsparseSpMatGetSize(d, byref(r), byref(c), byref(n)) == 0 and (r.value, c.value, n.value) == (2, 3, 4)
    assert L.aclsparseSpMatGetSize(d, None, None, None) == 0
    assert L.aclsparseSpMatSetValues(d, c_void_p(0x3000)) == 0
    assert L.aclsparseSpMatGetValues(d, byref(vals)) == 0 and vals.value == 0x3000
    assert L.aclsparseConstSpMatGetValues(d, byref(vals)) == 0
    assert L.aclsparseCsrSetPointers(d, None, FAKE, FAKE) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCsrSetPointers(d, FAKE, None, FAKE) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCsrSetPointers(d, FAKE, FAKE, FAKE) == 0
    assert L.aclsparseCsrSetPointers(None, FAKE, FAKE, FAKE) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseSpMatGetFormat(None, byref(fmt)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseDestroySpMat(d) == 0
    assert L.aclsparseDestroySpMat(None) == 0  # unlike the dense descriptors


def test_dnmat_lifecycle(pkg):
    L, S = pkg.lib(), pkg
    d = c_void_p()
    mk = lambda *a: L.aclsparseCreateDnMat(byref(d), *a)
    bad = S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseCreateDnMat(None, 2, 2, 2, FAKE, 0, 0) == bad
    assert mk(0, 2, 2, FAKE, 0, 0) == bad      # zero-sized matrices are rejected
    assert mk(2, 0, 2, FAKE, 0, 0) == bad
    assert mk(2, 2, 0, FAKE, 0, 0) == bad
    assert mk(2, 2, 2, None, 0, 0) == bad
    assert mk(2, 2, 2, FAKE, 999, 0) == bad
    assert mk(2, 2, 2, FAKE, 0, 2) == bad
    assert mk(2, 4, 3, FAKE, 0, S.ACL_SPARSE_ORDER_ROW) == bad   # ld < cols
    assert mk(4, 2, 3, FAKE, 0, S.ACL_SPARSE_ORDER_COL) == bad   # ld < rows
    assert mk(4, 2, 6, FAKE, S.ACL_BF16, S.ACL_SPARSE_ORDER_COL) == 0
    r, c, ld, vals, t, o = c_int64(), c_int64(), c_int64(), c_void_p(), c_int(), c_int()
    assert L.aclsparseDnMatGet(d, byref(r), byref(c), byref(ld), byref(vals), byref(t), byref(o)) == 0
    assert (r.value, c.value, ld.value, t.value, o.value) == (4, 2, 6, S.ACL_BF16, 1)
    assert L.aclsparseConstDnMatGet(d, None, None, None, None, None, None) == 0
    assert L.aclsparseDnMatSetValues(d, c_void_p(0x4000)) == 0
    assert L.aclsparseDnMatGetValues(d, byref(vals)) == 0 and vals.value == 0x4000
    assert L.aclsparseConstDnMatGetValues(d, byref(vals)) == 0
    assert L.aclsparseDnMatGet(None, None, None, None, None, None, None) == bad
    assert L.aclsparseDestroyDnMat(d) == 0
    assert L.aclsparseDestroyDnMat(None) == bad


def test_handle_argument_checks_without_device(pkg):
    L, S = pkg.lib(), pkg
    assert L.aclsparseCreate(None) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    occupied = c_void_p(0x10)
    assert L.aclsparseCreate(byref(occupied)) == S.ACL_SPARSE_STATUS_INVALID_VALUE  # slot must be NULL
    for fn, args in (("aclsparseDestroy", ()), ("aclsparseSetStream", (None,)), ("aclsparseGetStream", (None,)),
                     ("aclsparseSetWorkspace", (None, 0)), ("aclsparseGetWorkspace", (None, None)),
                     ("aclsparseSetPointerMode", (0,)), ("aclsparseGetPointerMode", (None,))):
        assert getattr(L, fn)(None, *args) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR, fn
    v = c_int()
    assert L.aclsparseGetVersion(None, byref(v)) == 0 and v.value == 10000
    assert L.aclsparseGetVersion(None, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE


def test_spmv_spmm_argument_checks_without_device(pkg):
    """Checks that precede any device work: they must answer the same on a machine with no GPU."""
    L, S = pkg.lib(), pkg
    size = c_size_t()
    H = c_void_p(0x10)  # never dereferenced before the checks below return
    assert L.aclsparseSpMVGetBufferSize(H, 0, None, None, None, None, None, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert L.aclsparseSpMVGetBufferSize(None, 0, None, None, None, None, None, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert L.aclsparseSpMV(H, 0, None, None, None, None, None, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    A, x, y = c_void_p(), c_void_p(), c_void_p()
    assert L.aclsparseCreateCsr(byref(A), 4, 4, 3, FAKE, FAKE, FAKE, 0, 0, S.ACL_SPARSE_INDEX_BASE_ONE, S.ACL_FLOAT) == 0
    assert L.aclsparseCreateDnVec(byref(x), 4, FAKE, S.ACL_FLOAT) == 0
    assert L.aclsparseCreateDnVec(byref(y), 4, FAKE, S.ACL_FLOAT) == 0
    assert L.aclsparseSpMV(H, 0, None, A, x, None, y, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED  # one-based
    L.aclsparseDestroySpMat(A)
    assert L.aclsparseCreateCsr(byref(A), 4, 4, 3, FAKE, FAKE, FAKE, 1, 1, 0, S.ACL_FLOAT) == 0
    assert L.aclsparseSpMV(H, 0, None, A, x, None, y, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED  # 64-bit indices
    L.aclsparseDestroySpMat(A)
    assert L.aclsparseCreateCsr(byref(A), 4, 4, 3, FAKE, FAKE, FAKE, 0, 0, 0, S.ACL_DOUBLE) == 0
    xd, yd = c_void_p(), c_void_p()
    L.aclsparseCreateDnVec(byref(xd), 4, FAKE, S.ACL_DOUBLE)
    L.aclsparseCreateDnVec(byref(yd), 4, FAKE, S.ACL_DOUBLE)
    assert L.aclsparseSpMV(H, 0, None, A, xd, None, yd, S.ACL_FLOAT, 0, None) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED  # fp64 values
    # SpMM: shape / type / layout checks
    B, C = c_void_p(), c_void_p()
    L.aclsparseDestroySpMat(A)
    assert L.aclsparseCreateCsr(byref(A), 4, 5, 3, FAKE, FAKE, FAKE, 0, 0, 0, S.ACL_FLOAT) == 0
    assert L.aclsparseCreateDnMat(byref(B), 5, 8, 8, FAKE, S.ACL_FLOAT, 0) == 0
    assert L.aclsparseCreateDnMat(byref(C), 4, 8, 8, FAKE, S.ACL_FLOAT, 0) == 0
    assert L.aclsparseSpMMGetBufferSize(H, 0, 0, None, A, B, None, C, S.ACL_FLOAT, 0, byref(size)) == 0
    assert size.value >= 256
    Ch = c_void_p()
    assert L.aclsparseCreateDnMat(byref(Ch), 4, 8, 8, FAKE, S.ACL_FLOAT16, 0) == 0
    assert L.aclsparseSpMMGetBufferSize(H, 0, 0, None, A, B, None, Ch, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    Cw = c_void_p()
    assert L.aclsparseCreateDnMat(byref(Cw), 4, 9, 9, FAKE, S.ACL_FLOAT, 0) == 0
    assert L.aclsparseSpMMGetBufferSize(H, 0, 0, None, A, B, None, Cw, S.ACL_FLOAT, 0, byref(size)) == S.ACL_SPARSE_STATUS_INVALID_VALUE
    for d, kill in ((x, L.aclsparseDestroyDnVec), (y, L.aclsparseDestroyDnVec), (xd, L.aclsparseDestroyDnVec),
                    (yd, L.aclsparseDestroyDnVec), (B, L.aclsparseDestroyDnMat), (C, L.aclsparseDestroyDnMat),
                    (Ch, L.aclsparseDestroyDnMat), (Cw, L.aclsparseDestroyDnMat)):
        assert kill(d) == 0
    assert L.aclsparseDestroySpMat(A) == 0


def test_buffer_size_formulas(pkg):
    L = pkg.lib()
    L.b200sp_spmv_plan_bytes.restype = c_size_t
    L.b200sp_spmv_plan_bytes.argtypes = [c_int64, c_int64, c_int64]
    L.b200sp_spmv_tile_plan_bytes.restype = c_size_t
    L.b200sp_spmv_tile_plan_bytes.argtypes = [c_int64, c_int64]
    L.b200sp_spmm_plan_bytes.restype = c_size_t
    L.b200sp_spmm_plan_bytes.argtypes = [c_int64, c_int64, c_int64]
    assert L.b200sp_spmv_plan_bytes(0, 0, 0) >= 256
    rows, nnz = 1 << 20, 1 << 25
    tiles = (rows + nnz + 3839) // 3840  # 256 threads x 15 merge items per tile
    tile_plan = L.b200sp_spmv_tile_plan_bytes(rows, nnz)
    assert 16 * tiles <= tile_plan <= 16 * tiles + 4096   # tile table + counters + two partial arrays, 4 B each
    # binned plan: a list entry per row that can be longer than 32 entries, one per possible long row (512+)
    # {row, start, end, -} per entry; the long list twice (as found, then ordered by length)
    long_len, seg_len = 512, 8192
    cap_long = nnz // long_len + 1
    cap_segs = nnz // seg_len + cap_long   # long rows cut into 8192-entry segments: {row, start, end, slot} each
    bins = 256 + 16 * (min(rows, nnz // 33) + 1) + 2 * 16 * cap_long
    segs = 16 * cap_segs + 8 * cap_long + 4 * cap_long + 4 * cap_segs  # + per-row {first, count}, counters, partial sums
    # too wide for the blocked long-row kernel (more than 64 blocks of 32768 columns): the lists only
    assert max(tile_plan, bins + segs) <= L.b200sp_spmv_plan_bytes(rows, 1 << 22, nnz) <= max(tile_plan, bins + segs) + 4096
    # narrow enough: per possible long row, xBlocks + 1 cut points and xBlocks partial sums, 4 B each
    xb = (rows + 32767) // 32768
    blocked = bins + segs + cap_long * (2 * xb + 1) * 4 + 256
    assert blocked <= L.b200sp_spmv_plan_bytes(rows, rows, nnz) <= blocked + 4096
    assert L.b200sp_spmm_plan_bytes(1 << 18, 1 << 24, 64) >= 2 * ((1 << 24) // 4096) * 64 * 4


def test_coo2csr_argument_checks_without_device(pkg):
    """Order and codes of sparse/coo2csr/arch35/coo2csr_host.cpp:38-78; every case returns before any launch."""
    L, S = pkg.lib(), pkg
    H = c_void_p(0x10)
    f = L.aclsparseXcoo2csr
    INV = S.ACL_SPARSE_STATUS_INVALID_VALUE
    assert f(None, FAKE, 4, 4, FAKE, 0) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert f(H, FAKE, -1, 4, FAKE, 0) == INV
    assert f(H, FAKE, 2 ** 31 - 1, 4, FAKE, 1) == INV      # nnz + base would overflow
    assert f(H, FAKE, 4, -1, FAKE, 0) == INV
    assert f(H, FAKE, 4, 0, FAKE, 0) == INV                # entries but no rows
    assert f(H, FAKE, 4, 4, FAKE, 2) == INV                # index base
    assert f(H, None, 4, 4, FAKE, 0) == INV
    assert f(H, FAKE, 4, 4, None, 0) == INV
    assert f(H, None, -1, -1, None, 7) == INV              # nnz is looked at first


def test_matdescr_and_csrsort_argument_checks_without_device(pkg):
    """sparse/common/aclsparse_matdescr.cpp:25-108 and sparse/csrsort/arch35/csrsort_host.cpp:52-74, 146-222."""
    L, S = pkg.lib(), pkg
    INV = S.ACL_SPARSE_STATUS_INVALID_VALUE
    D = c_void_p()
    assert L.aclsparseCreateMatDescr(None) == INV
    assert L.aclsparseCreateMatDescr(byref(D)) == 0 and D.value
    assert (L.aclsparseGetMatType(D), L.aclsparseGetMatIndexBase(D), L.aclsparseGetMatDiagType(D),
            L.aclsparseGetMatFillMode(D)) == (0, 0, 0, 0)
    L.aclsparseSetMatType(D, 3); L.aclsparseSetMatIndexBase(D, 1); L.aclsparseSetMatDiagType(D, 1)
    L.aclsparseSetMatFillMode(D, 1)
    assert (L.aclsparseGetMatType(D), L.aclsparseGetMatIndexBase(D), L.aclsparseGetMatDiagType(D),
            L.aclsparseGetMatFillMode(D)) == (3, 1, 1, 1)
    L.aclsparseSetMatIndexBase(None, 1)  # setters ignore NULL, getters answer the default for it
    assert L.aclsparseGetMatIndexBase(None) == 0 and L.aclsparseGetMatType(None) == 0

    H = c_void_p(0x10)
    size = c_size_t(99)
    q = L.aclsparseXcsrsort_bufferSizeExt
    assert q(None, 4, 4, 4, FAKE, FAKE, byref(size)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert q(H, 4, 4, 4, FAKE, FAKE, None) == INV
    assert q(H, -1, 4, 4, FAKE, FAKE, byref(size)) == INV
    assert q(H, 0, 4, 4, FAKE, FAKE, byref(size)) == INV      # entries but no rows
    assert q(H, 4, 0, 4, FAKE, FAKE, byref(size)) == INV      # entries but no columns
    assert q(H, 4, 4, 4, None, FAKE, byref(size)) == INV
    assert q(H, 4, 4, 4, FAKE, None, byref(size)) == INV
    assert q(H, 4, 4, 0, FAKE, None, byref(size)) == 0 and size.value == 0

    f = L.aclsparseXcsrsort
    assert f(None, 4, 4, 4, D, FAKE, FAKE, FAKE, FAKE) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert f(H, 4, 4, -4, D, FAKE, FAKE, FAKE, FAKE) == INV
    assert f(H, 4, 4, 4, None, FAKE, FAKE, FAKE, FAKE) == INV
    L.aclsparseSetMatIndexBase(D, 5)
    assert f(H, 4, 4, 4, D, FAKE, FAKE, FAKE, FAKE) == INV
    L.aclsparseSetMatIndexBase(D, 0)
    assert f(H, 4, 4, 0, D, FAKE, None, None, None) == 0          # nothing to sort
    assert f(H, 4, 4, 4, D, FAKE, FAKE, None, FAKE) == INV
    assert f(H, 4, 4, 4, D, FAKE, FAKE, FAKE, None) == INV
    assert L.aclsparseDestroyMatDescr(D) == 0 and L.aclsparseDestroyMatDescr(None) == 0


def test_csr2csc_argument_checks_without_device(pkg):
    """Order and codes of sparse/csr2csc_ex2/arch35/csr2csc_ex2_host.cpp:106-232, 539-640."""
    L, S = pkg.lib(), pkg
    H = c_void_p(0x10)
    INV, NS = S.ACL_SPARSE_STATUS_INVALID_VALUE, S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    size = c_size_t(5)
    q, f = L.aclsparseCsr2cscEx2_bufferSize, L.aclsparseCsr2cscEx2
    F = S.ACL_FLOAT
    assert q(None, 3, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 0, byref(size)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert q(H, -1, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 0, byref(size)) == INV
    assert q(H, 3, -1, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 0, byref(size)) == INV
    assert q(H, 3, 2 ** 31 - 1, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 0, byref(size)) == INV
    assert q(H, 3, 3, -1, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 0, byref(size)) == INV
    assert q(H, 3, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, S.ACL_INT32, 1, 0, 0, byref(size)) == NS   # value type
    assert q(H, 3, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 2, 0, 0, byref(size)) == INV            # action
    assert q(H, 3, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 2, 0, byref(size)) == INV            # index base
    assert q(H, 3, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 2, byref(size)) == INV            # algorithm
    assert q(H, 3, 3, 3, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, F, 1, 0, 0, None) == INV
    for m, n, nnz in ((0, 3, 0), (3, 0, 0), (3, 3, 0)):
        assert q(H, m, n, nnz, None, None, None, None, None, None, S.ACL_BF16, 0, 1, 1, byref(size)) == 0
        assert size.value == 0
    args = lambda **kw: [kw.get(k, d) for k, d in (("csrVal", FAKE), ("rp", FAKE), ("ci", FAKE), ("cscVal", FAKE),
                                                    ("cp", FAKE), ("ri", FAKE))]
    call = lambda m=3, n=3, nnz=3, action=1, **kw: f(H, m, n, nnz, *args(**kw), F, action, 0, 0, FAKE)
    assert call(rp=None) == INV and call(ci=None) == INV and call(csrVal=None) == INV
    assert call(cp=None) == INV and call(ri=None) == INV and call(cscVal=None) == INV
    assert call(csrVal=None, cscVal=None, action=0, rp=None) == INV      # SYMBOLIC needs no values, still needs offsets
    assert call(m=0) == INV and call(n=0) == INV                          # entries without rows / columns


def test_sddmm_argument_checks_without_device(pkg):
    """Order and codes of sparse/sddmm/arch35/sddmm_host.cpp:194-320, 478-510, 660-692 (failing cases only: they
    return before the handle is read)."""
    L, S = pkg.lib(), pkg
    H = c_void_p(0x10)
    INV, NS = S.ACL_SPARSE_STATUS_INVALID_VALUE, S.ACL_SPARSE_STATUS_NOT_SUPPORTED
    X, Y, C, C64, C1, Xh = (c_void_p() for _ in range(6))
    assert L.aclsparseCreateDnMat(byref(X), 4, 8, 8, FAKE, S.ACL_FLOAT, 0) == 0
    assert L.aclsparseCreateDnMat(byref(Xh), 4, 8, 8, FAKE, S.ACL_FLOAT16, 0) == 0
    assert L.aclsparseCreateDnMat(byref(Y), 8, 5, 5, FAKE, S.ACL_FLOAT, 0) == 0
    mk = lambda d, off, base: L.aclsparseCreateCsr(byref(d), 4, 5, 6, FAKE, FAKE, FAKE, off, 0, base, S.ACL_FLOAT)
    assert mk(C, 0, 0) == 0 and mk(C64, S.ACL_SPARSE_INDEX_64I, 0) == 0 and mk(C1, 0, 1) == 0
    N, T = S.ACL_SPARSE_OP_NON_TRANSPOSE, S.ACL_SPARSE_OP_TRANSPOSE
    size = c_size_t()
    q, f, pre = L.aclsparseSDDMMBufferSize, L.aclsparseSDDMM, L.aclsparseSDDMMPreprocess
    F = S.ACL_FLOAT
    assert q(None, N, N, FAKE, X, Y, FAKE, C, F, 0, byref(size)) == S.ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR
    assert q(H, N, N, FAKE, X, Y, FAKE, C, F, 0, None) == INV
    assert q(H, N, N, None, X, Y, FAKE, C, F, 0, byref(size)) == INV
    assert q(H, N, N, FAKE, X, Y, FAKE, C, F, 0, byref(size)) == 0 and size.value > 0
    assert q(H, N, N, FAKE, None, Y, FAKE, C, F, 0, byref(size)) == INV
    assert q(H, N, N, FAKE, X, Y, FAKE, C64, F, 0, byref(size)) == NS          # int64 row offsets
    assert q(H, N, N, FAKE, X, Y, FAKE, C1, F, 0, byref(size)) == NS           # one-based
    assert q(H, 2, N, FAKE, X, Y, FAKE, C, F, 0, byref(size)) == NS            # conjugate transpose
    assert q(H, N, N, FAKE, Xh, Y, FAKE, C, F, 0, byref(size)) == NS           # mixed types
    assert q(H, N, N, FAKE, X, Y, FAKE, C, S.ACL_FLOAT16, 0, byref(size)) == NS
    assert q(H, T, N, FAKE, X, Y, FAKE, C, F, 0, byref(size)) == INV           # X^T is 8 x 4: rows do not match C
    assert q(H, N, T, FAKE, X, Y, FAKE, C, F, 0, byref(size)) == INV           # Y^T is 5 x 8
    assert q(H, N, N, FAKE, X, Y, FAKE, C, F, 1, byref(size)) == NS            # algorithm
    # the compute / preprocess calls check the descriptors before the scalars, and the buffer last
    assert f(H, N, N, None, None, Y, FAKE, C, F, 0, FAKE) == INV
    assert f(H, N, N, None, X, Y, FAKE, C, F, 0, FAKE) == INV
    assert f(H, N, N, FAKE, X, Y, FAKE, C, F, 0, None) == INV
    assert pre(H, N, N, FAKE, X, Y, FAKE, C, F, 0, None) == S.ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES
    assert pre(H, N, N, FAKE, X, Y, FAKE, C, F, 0, FAKE) == 0
    for d in (X, Xh, Y):
        assert L.aclsparseDestroyDnMat(d) == 0
    for d in (C, C64, C1):
        assert L.aclsparseDestroySpMat(d) == 0
