"""Object wrappers over the aclsparse C API for callers that hold torch CUDA tensors.

Each class owns one C descriptor (created in __init__, destroyed in close()/__del__) and
keeps a reference to the tensors whose device pointers the descriptor borrows.  The call
sequence is the reference's own (test/spmv/arch22/spmv_test.cpp:415-479,
test/spmm/arch35/spmm_test.cpp:460-516): handle -> descriptors -> GetBufferSize ->
Preprocess -> compute.  All arithmetic happens inside libops_sparse.so.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_int, c_int32, c_size_t, c_void_p

import torch

from . import (
    ACL_BF16, ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_SPARSE_INDEX_32I, ACL_SPARSE_INDEX_64I,
    ACL_SPARSE_INDEX_BASE_ZERO, ACL_SPARSE_SPMVOP_ALG_DEFAULT, ACL_SPARSE_SPMVOP_ALG2,
    ACL_SPARSE_OP_NON_TRANSPOSE, ACL_SPARSE_ORDER_COL, ACL_SPARSE_ORDER_ROW, ACL_SPARSE_POINTER_MODE_DEVICE,
    ACL_SPARSE_SPMM_ALG_DEFAULT, ACL_SPARSE_SPMV_ALG_DEFAULT, check, lib,
)

_ACL_OF = {
    torch.float32: ACL_FLOAT, torch.float16: ACL_FLOAT16, torch.bfloat16: ACL_BF16,
    torch.int32: ACL_INT32, torch.int8: ACL_INT8,
}


def acl_type_of(dtype: torch.dtype) -> int:
    try:
        return _ACL_OF[dtype]
    except KeyError:
        raise TypeError(f"no aclDataType for {dtype}") from None


def _ptr(t: torch.Tensor | None) -> c_void_p | None:
    """Device pointer of a tensor as a C void* (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


class Handle:
    """aclsparseHandle_t bound to a CUDA stream (default: torch's current stream)."""

    def __init__(self, stream: torch.cuda.Stream | None = None):
        self._h = c_void_p()
        check(lib().aclsparseCreate(byref(self._h)), "aclsparseCreate")
        s = stream if stream is not None else torch.cuda.current_stream()
        self.stream = s
        check(lib().aclsparseSetStream(self._h, c_void_p(s.cuda_stream)), "aclsparseSetStream")
        self.device_scalars = False

    @property
    def raw(self) -> c_void_p:
        return self._h

    def set_pointer_mode_device(self, on: bool) -> None:
        check(lib().aclsparseSetPointerMode(self._h, ACL_SPARSE_POINTER_MODE_DEVICE if on else 0),
              "aclsparseSetPointerMode")
        self.device_scalars = on

    def close(self) -> None:
        if self._h:
            lib().aclsparseDestroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DnVec:
    def __init__(self, values: torch.Tensor, size: int | None = None):
        self.values = values
        self._d = c_void_p()
        n = values.numel() if size is None else size
        check(lib().aclsparseCreateDnVec(byref(self._d), n, _ptr(values), acl_type_of(values.dtype)),
              "aclsparseCreateDnVec")

    @property
    def raw(self) -> c_void_p:
        return self._d

    def close(self) -> None:
        if self._d:
            lib().aclsparseDestroyDnVec(self._d)
            self._d = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DnMat:
    """Dense matrix descriptor over a 2-D tensor.  order 'row': ld = stride(0); 'col': the
    tensor holds the column-major storage, i.e. it has shape (cols, ld-ish) transposed."""

    def __init__(self, values: torch.Tensor, rows: int, cols: int, ld: int, order: str = "row"):
        self.values = values
        self.rows, self.cols, self.ld, self.order = rows, cols, ld, order
        self._d = c_void_p()
        check(lib().aclsparseCreateDnMat(byref(self._d), rows, cols, ld, _ptr(values), acl_type_of(values.dtype),
                                         ACL_SPARSE_ORDER_ROW if order == "row" else ACL_SPARSE_ORDER_COL),
              "aclsparseCreateDnMat")

    @classmethod
    def row_major(cls, t: torch.Tensor) -> "DnMat":
        assert t.dim() == 2 and t.stride(1) == 1
        return cls(t, t.shape[0], t.shape[1], t.stride(0), "row")

    @property
    def raw(self) -> c_void_p:
        return self._d

    def close(self) -> None:
        if self._d:
            lib().aclsparseDestroyDnMat(self._d)
            self._d = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CsrMatrix:
    def __init__(self, row_ptr: torch.Tensor, col_ind: torch.Tensor, values: torch.Tensor, rows: int, cols: int,
                 nnz: int | None = None, index_base: int = ACL_SPARSE_INDEX_BASE_ZERO):
        """row_ptr is int32, or int64 for the SpMVOp plan API; index_base 1 likewise is SpMVOp only."""
        assert row_ptr.dtype in (torch.int32, torch.int64) and col_ind.dtype == torch.int32
        self.row_ptr, self.col_ind, self.values = row_ptr, col_ind, values
        self.rows, self.cols = rows, cols
        self.nnz = col_ind.numel() if nnz is None else nnz
        self._d = c_void_p()
        off_type = ACL_SPARSE_INDEX_64I if row_ptr.dtype == torch.int64 else ACL_SPARSE_INDEX_32I
        check(lib().aclsparseCreateCsr(byref(self._d), rows, cols, self.nnz, _ptr(row_ptr), _ptr(col_ind),
                                       _ptr(values), off_type, ACL_SPARSE_INDEX_32I, index_base,
                                       acl_type_of(values.dtype)),
              "aclsparseCreateCsr")
        self.buffer: torch.Tensor | None = None  # workspace recorded by preprocess_*()

    @property
    def raw(self) -> c_void_p:
        return self._d

    def close(self) -> None:
        if self._d:
            lib().aclsparseDestroySpMat(self._d)
            self._d = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _scalars(handle: Handle, alpha, beta, compute_type: int):
    """Returns (alpha_arg, beta_arg, keepalive) for the C call."""
    if handle.device_scalars:
        return _ptr(alpha), _ptr(beta), (alpha, beta)
    ctype = c_int32 if compute_type == ACL_INT32 else c_float
    a, b = ctype(alpha), ctype(beta)
    return ctypes.cast(byref(a), c_void_p), ctypes.cast(byref(b), c_void_p), (a, b)


def _compute_type(values: torch.Tensor, out: torch.Tensor) -> int:
    return ACL_INT32 if (values.dtype in (torch.int32, torch.int8) and out.dtype == torch.int32) else ACL_FLOAT


def spmv_buffer_size(handle: Handle, A: CsrMatrix, x: DnVec, y: DnVec, op: int = ACL_SPARSE_OP_NON_TRANSPOSE) -> int:
    size = c_size_t()
    ct = _compute_type(A.values, y.values)
    check(lib().aclsparseSpMVGetBufferSize(handle.raw, op, None, A.raw, x.raw, None, y.raw, ct,
                                           ACL_SPARSE_SPMV_ALG_DEFAULT, byref(size)), "aclsparseSpMVGetBufferSize")
    return size.value


def spmv_preprocess(handle: Handle, A: CsrMatrix, x: DnVec, y: DnVec, op: int = ACL_SPARSE_OP_NON_TRANSPOSE):
    """GetBufferSize + device allocation + Preprocess; the buffer is kept on A.buffer."""
    nbytes = spmv_buffer_size(handle, A, x, y, op)
    A.buffer = torch.empty(nbytes, dtype=torch.uint8, device=A.row_ptr.device)
    ct = _compute_type(A.values, y.values)
    check(lib().aclsparseSpMVPreprocess(handle.raw, op, None, A.raw, x.raw, None, y.raw, ct,
                                        ACL_SPARSE_SPMV_ALG_DEFAULT, _ptr(A.buffer)), "aclsparseSpMVPreprocess")
    return A.buffer


def spmv(handle: Handle, A: CsrMatrix, x: DnVec, y: DnVec, alpha=1.0, beta=0.0,
         op: int = ACL_SPARSE_OP_NON_TRANSPOSE, buffer: torch.Tensor | None = None) -> None:
    """y = alpha * op(A) x + beta * y, enqueued on the handle's stream."""
    ct = _compute_type(A.values, y.values)
    a, b, keep = _scalars(handle, alpha, beta, ct)
    buf = _ptr(buffer) if buffer is not None else None
    check(lib().aclsparseSpMV(handle.raw, op, a, A.raw, x.raw, b, y.raw, ct, ACL_SPARSE_SPMV_ALG_DEFAULT, buf),
          "aclsparseSpMV")
    del keep


def spmm_buffer_size(handle: Handle, A: CsrMatrix, B: DnMat, C: DnMat, op_b: int = ACL_SPARSE_OP_NON_TRANSPOSE,
                     alg: int = ACL_SPARSE_SPMM_ALG_DEFAULT) -> int:
    size = c_size_t()
    ct = _compute_type(A.values, C.values)
    check(lib().aclsparseSpMMGetBufferSize(handle.raw, ACL_SPARSE_OP_NON_TRANSPOSE, op_b, None, A.raw, B.raw, None,
                                           C.raw, ct, alg, byref(size)), "aclsparseSpMMGetBufferSize")
    return size.value


def spmm_preprocess(handle: Handle, A: CsrMatrix, B: DnMat, C: DnMat, op_b: int = ACL_SPARSE_OP_NON_TRANSPOSE,
                    alg: int = ACL_SPARSE_SPMM_ALG_DEFAULT):
    nbytes = spmm_buffer_size(handle, A, B, C, op_b, alg)
    A.buffer = torch.empty(nbytes, dtype=torch.uint8, device=A.row_ptr.device)
    ct = _compute_type(A.values, C.values)
    check(lib().aclsparseSpMMPreprocess(handle.raw, ACL_SPARSE_OP_NON_TRANSPOSE, op_b, None, A.raw, B.raw, None,
                                        C.raw, ct, alg, _ptr(A.buffer)), "aclsparseSpMMPreprocess")
    return A.buffer


def spmm(handle: Handle, A: CsrMatrix, B: DnMat, C: DnMat, alpha=1.0, beta=0.0,
         op_b: int = ACL_SPARSE_OP_NON_TRANSPOSE, alg: int = ACL_SPARSE_SPMM_ALG_DEFAULT,
         buffer: torch.Tensor | None = None) -> None:
    """C = alpha * A op(B) + beta * C, enqueued on the handle's stream."""
    ct = _compute_type(A.values, C.values)
    a, b, keep = _scalars(handle, alpha, beta, ct)
    buf = buffer if buffer is not None else A.buffer
    if buf is None:
        buf = spmm_preprocess(handle, A, B, C, op_b, alg)
    check(lib().aclsparseSpMM(handle.raw, ACL_SPARSE_OP_NON_TRANSPOSE, op_b, a, A.raw, B.raw, b, C.raw, ct, alg,
                              _ptr(buf)), "aclsparseSpMM")
    del keep


class SpMVOpPlan:
    """aclsparseSpMVOp_bufferSize -> createDescr -> createPlan for one matrix; `run` is aclsparseSpMVOp.

    Z = alpha * A * X + beta * Y in fp32 with compensated row sums; Z may be Y.  The workspace of ALG2
    is owned by this object and lives as long as it does.
    """

    def __init__(self, handle: Handle, A: CsrMatrix, x: DnVec, y: DnVec, z: DnVec,
                 alg: int = ACL_SPARSE_SPMVOP_ALG_DEFAULT):
        self.handle, self.A = handle, A
        size = c_size_t()
        check(lib().aclsparseSpMVOp_bufferSize(handle.raw, ACL_SPARSE_OP_NON_TRANSPOSE, A.raw, x.raw, y.raw, z.raw,
                                               ACL_FLOAT, alg, byref(size)), "aclsparseSpMVOp_bufferSize")
        self.buffer_bytes = size.value
        self.buffer = (torch.empty(max(size.value, 1), dtype=torch.uint8, device=A.col_ind.device)
                       if alg == ACL_SPARSE_SPMVOP_ALG2 else None)
        self._descr, self._plan = c_void_p(), c_void_p()
        check(lib().aclsparseSpMVOp_createDescr(handle.raw, byref(self._descr), ACL_SPARSE_OP_NON_TRANSPOSE, A.raw,
                                                x.raw, y.raw, z.raw, ACL_FLOAT, alg,
                                                _ptr(self.buffer) if self.buffer is not None else None),
              "aclsparseSpMVOp_createDescr")
        check(lib().aclsparseSpMVOp_createPlan(handle.raw, self._descr, byref(self._plan), None, 0),
              "aclsparseSpMVOp_createPlan")

    def run(self, x: DnVec, y: DnVec, z: DnVec, alpha=1.0, beta=0.0) -> None:
        a, b, keep = _scalars(self.handle, alpha, beta, ACL_FLOAT)
        check(lib().aclsparseSpMVOp(self.handle.raw, self._plan, a, b, x.raw, y.raw, z.raw), "aclsparseSpMVOp")
        del keep

    def close(self) -> None:
        if self._plan:
            lib().aclsparseSpMVOp_destroyPlan(self._plan)
            self._plan = c_void_p()
        if self._descr:
            lib().aclsparseSpMVOp_destroyDescr(self._descr)
            self._descr = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
