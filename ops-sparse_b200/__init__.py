"""ops-sparse_b200: CSR SpMV / SpMM for B200 behind the aclsparse C API.

The product is `lib/libops_sparse.so` (C++ host layer + hand-written sm_100a kernels).  This
Python package is a thin ctypes mirror of that C API for tests, benchmarks and Python
callers: the functions keep the C names (`aclsparseCreate`, `aclsparseSpMV`, ...), take the
same arguments and return the same `aclsparseStatus_t` codes.  Device memory, streams and
`torch.distributed` come from PyTorch; no arithmetic is done in Python and there is no CPU
fallback: importing `lib()` without the built library raises.

The directory name contains a hyphen, so load it through `__graft_entry__.load_package()`
(or importlib with an explicit module name such as `ops_sparse_b200`).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_double, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libops_sparse.so"

# ---- enums, same numeric values as include/cann_ops_sparse.h and include/acl/acl_base_rt.h
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_BF16 = 0, 1, 2, 3, 27
ACL_INT64, ACL_DOUBLE = 9, 11

ACL_SPARSE_OP_NON_TRANSPOSE, ACL_SPARSE_OP_TRANSPOSE, ACL_SPARSE_OP_CONJUGATE_TRANSPOSE = 0, 1, 2
ACL_SPARSE_ORDER_ROW, ACL_SPARSE_ORDER_COL = 0, 1
ACL_SPARSE_SPMM_ALG_DEFAULT, ACL_SPARSE_SPMM_CSR_ALG1, ACL_SPARSE_SPMM_CSR_FP32_HIGH_PRECISION_ALG = 0, 1, 2
ACL_SPARSE_SPMV_ALG_DEFAULT, ACL_SPARSE_SPMV_CSR_ALG1 = 0, 3
ACL_SPARSE_SPMVOP_ALG_DEFAULT, ACL_SPARSE_SPMVOP_ALG1, ACL_SPARSE_SPMVOP_ALG2 = 0, 1, 2
ACL_SPARSE_INDEX_32I, ACL_SPARSE_INDEX_64I = 0, 1
ACL_SPARSE_INDEX_BASE_ZERO, ACL_SPARSE_INDEX_BASE_ONE = 0, 1
ACL_SPARSE_FORMAT_COO, ACL_SPARSE_FORMAT_CSR, ACL_SPARSE_FORMAT_CSC = 0, 1, 2
ACL_SPARSE_POINTER_MODE_HOST, ACL_SPARSE_POINTER_MODE_DEVICE = 0, 1

STATUS_NAMES = [
    "SUCCESS", "NOT_INITIALIZED", "ALLOC_FAILED", "INVALID_VALUE", "ARCH_MISMATCH", "EXECUTION_FAILED",
    "INTERNAL_ERROR", "MATRIX_TYPE_NOT_SUPPORTED", "NOT_SUPPORTED", "INSUFFICIENT_RESOURCES", "HANDLE_IS_NULLPTR",
]
(ACL_SPARSE_STATUS_SUCCESS, ACL_SPARSE_STATUS_NOT_INITIALIZED, ACL_SPARSE_STATUS_ALLOC_FAILED,
 ACL_SPARSE_STATUS_INVALID_VALUE, ACL_SPARSE_STATUS_ARCH_MISMATCH, ACL_SPARSE_STATUS_EXECUTION_FAILED,
 ACL_SPARSE_STATUS_INTERNAL_ERROR, ACL_SPARSE_STATUS_MATRIX_TYPE_NOT_SUPPORTED, ACL_SPARSE_STATUS_NOT_SUPPORTED,
 ACL_SPARSE_STATUS_INSUFFICIENT_RESOURCES, ACL_SPARSE_STATUS_HANDLE_IS_NULLPTR) = range(11)


class AclSparseError(RuntimeError):
    def __init__(self, call: str, status: int):
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{call} returned ACL_SPARSE_STATUS_{name}")
        self.status = status


def check(status: int, call: str = "aclsparse call") -> None:
    if status != ACL_SPARSE_STATUS_SUCCESS:
        raise AclSparseError(call, status)


P = c_void_p
_SIGNATURES = {
    # handle
    "aclsparseCreate": [POINTER(P)],
    "aclsparseDestroy": [P],
    "aclsparseSetStream": [P, P],
    "aclsparseGetStream": [P, POINTER(P)],
    "aclsparseSetWorkspace": [P, P, c_size_t],
    "aclsparseGetWorkspace": [P, POINTER(P), POINTER(c_size_t)],
    "aclsparseGetVersion": [P, POINTER(c_int)],
    "aclsparseSetPointerMode": [P, c_int],
    "aclsparseGetPointerMode": [P, POINTER(c_int)],
    # dense vector
    "aclsparseCreateDnVec": [POINTER(P), c_int64, P, c_int],
    "aclsparseCreateConstDnVec": [POINTER(P), c_int64, P, c_int],
    "aclsparseDestroyDnVec": [P],
    "aclsparseDnVecGet": [P, POINTER(c_int64), POINTER(P), POINTER(c_int)],
    "aclsparseConstDnVecGet": [P, POINTER(c_int64), POINTER(P), POINTER(c_int)],
    "aclsparseDnVecGetValues": [P, POINTER(P)],
    "aclsparseConstDnVecGetValues": [P, POINTER(P)],
    "aclsparseDnVecSetValues": [P, P],
    # CSR
    "aclsparseCreateCsr": [POINTER(P), c_int64, c_int64, c_int64, P, P, P, c_int, c_int, c_int, c_int],
    "aclsparseCreateConstCsr": [POINTER(P), c_int64, c_int64, c_int64, P, P, P, c_int, c_int, c_int, c_int],
    "aclsparseCsrSetPointers": [P, P, P, P],
    "aclsparseDestroySpMat": [P],
    "aclsparseSpMatGetFormat": [P, POINTER(c_int)],
    "aclsparseSpMatGetValues": [P, POINTER(P)],
    "aclsparseConstSpMatGetValues": [P, POINTER(P)],
    "aclsparseSpMatSetValues": [P, P],
    "aclsparseSpMatGetSize": [P, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64)],
    # dense matrix
    "aclsparseCreateDnMat": [POINTER(P), c_int64, c_int64, c_int64, P, c_int, c_int],
    "aclsparseCreateConstDnMat": [POINTER(P), c_int64, c_int64, c_int64, P, c_int, c_int],
    "aclsparseDestroyDnMat": [P],
    "aclsparseDnMatGet": [P, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), POINTER(P), POINTER(c_int),
                          POINTER(c_int)],
    "aclsparseConstDnMatGet": [P, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), POINTER(P), POINTER(c_int),
                               POINTER(c_int)],
    "aclsparseDnMatGetValues": [P, POINTER(P)],
    "aclsparseConstDnMatGetValues": [P, POINTER(P)],
    "aclsparseDnMatSetValues": [P, P],
    # SpMV: handle, opA, alpha, matA, vecX, beta, vecY, computeType, alg, (bufferSize* | buffer)
    "aclsparseSpMVGetBufferSize": [P, c_int, P, P, P, P, P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMVPreprocess": [P, c_int, P, P, P, P, P, c_int, c_int, P],
    "aclsparseSpMV": [P, c_int, P, P, P, P, P, c_int, c_int, P],
    "b200spRepeatSpMV": [P, c_int, P, P, P, P, P, c_int, c_int, P, c_int],
    "b200spRepeatSpMM": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, P, c_int],
    "b200spSpMMPlanInfo": [P, POINTER(c_int32)],
    # exchange, slice, offset, bytes, firstSeq, replicas, waitMask, then the product's arguments with an array of
    # per-replica dense descriptors, reps
    "b200spMgRepeatSpMV": [P, P, c_size_t, c_size_t, c_uint32, c_int, c_uint32, P, c_int, P, P, P, P, P, c_int, c_int,
                           P, c_int],
    "b200spMgRepeatSpMM": [P, P, c_size_t, c_size_t, c_uint32, c_int, c_uint32, P, c_int, c_int, P, P, P, P, P, c_int,
                           c_int, P, c_int],
    # SpMM: handle, opA, opB, alpha, matA, matB, beta, matC, computeType, alg, (size* | buffer)
    "aclsparseSpMMGetBufferSize": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMMPreprocess": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, P],
    "aclsparseSpMM": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, P],
    # SpMVOp plan API
    "aclsparseSpMVOp_bufferSize": [P, c_int, P, P, P, P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSpMVOp_createDescr": [P, POINTER(P), c_int, P, P, P, P, c_int, c_int, P],
    "aclsparseSpMVOp_destroyDescr": [P],
    "aclsparseSpMVOp_createPlan": [P, P, POINTER(P), P, c_size_t],
    "aclsparseSpMVOp_destroyPlan": [P],
    "aclsparseSpMVOp_setGlobalUserData": [P, P, ctypes.c_char_p, P, c_size_t],
    "aclsparseSpMVOp": [P, P, P, P, P, P, P],
    # SDDMM: handle, opX, opY, alpha, matX, matY, beta, matC, computeType, alg, (size* | buffer)
    "aclsparseSDDMMBufferSize": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, POINTER(c_size_t)],
    "aclsparseSDDMMPreprocess": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, P],
    "aclsparseSDDMM": [P, c_int, c_int, P, P, P, P, P, c_int, c_int, P],
    "aclsparseXcoo2csr": [P, P, c_int, c_int, P, c_int],
    "aclsparseCsr2cscEx2_bufferSize": [P, c_int, c_int, c_int, P, P, P, P, P, P, c_int, c_int, c_int, c_int,
                                       POINTER(c_size_t)],
    "aclsparseCsr2cscEx2": [P, c_int, c_int, c_int, P, P, P, P, P, P, c_int, c_int, c_int, c_int, P],
    "aclsparseCreateMatDescr": [POINTER(P)],
    "aclsparseDestroyMatDescr": [P],
    "aclsparseSetMatType": [P, c_int],
    "aclsparseSetMatIndexBase": [P, c_int],
    "aclsparseSetMatDiagType": [P, c_int],
    "aclsparseSetMatFillMode": [P, c_int],
    "aclsparseGetMatType": [P],
    "aclsparseGetMatIndexBase": [P],
    "aclsparseGetMatDiagType": [P],
    "aclsparseGetMatFillMode": [P],
    "aclsparseXcsrsort_bufferSizeExt": [P, c_int, c_int, c_int, P, P, POINTER(c_size_t)],
    "aclsparseXcsrsort": [P, c_int, c_int, c_int, P, P, P, P, P],
    # multi-GPU helpers (include/b200sp_mg.h)
    "b200spMgPartitionRows": [P, c_int64, c_int32, POINTER(c_int64)],
}
_RESTYPE = {"b200spMgImbalance": c_double}
_SIGNATURES["b200spMgImbalance"] = [P, c_int64, c_int32, POINTER(c_int64)]

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded libops_sparse.so with argument types set.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python ops-sparse_b200/build.py` "
                "(there is no fallback implementation)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPE.get(name, c_int)
        _lib = handle
    return _lib


def __getattr__(name: str):
    # `pkg.aclsparseSpMV(...)` resolves to the C function of the same name.
    if name.startswith("aclsparse") or name.startswith("b200sp"):
        return getattr(lib(), name)
    raise AttributeError(name)


from .api import (  # noqa: E402  (needs the names above)
    CsrMatrix, DnMat, DnVec, Handle, acl_type_of, spmm, spmv,
)

__all__ = [
    "lib", "check", "AclSparseError", "Handle", "CsrMatrix", "DnVec", "DnMat", "spmv", "spmm", "acl_type_of",
]
