"""Shared helpers for the parity tests: device upload, tolerance checks."""
from __future__ import annotations

import numpy as np
import torch

TORCH_OF = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i32": torch.int32, "i8": torch.int8}

# Per-row tolerance of the benchmark spec: |err_i| <= tol * sum_j |a_ij * x_j|, tol = 1e-5 for
# fp32 data and 2e-3 for 16-bit values with fp32 accumulation.  With beta != 0 the scale also
# carries |beta * y_i| (the unavoidable final rounding is relative to the whole result) and is
# multiplied by |alpha|.
TOL = {"f32": 1e-5, "f16": 2e-3, "bf16": 2e-3}


def to_device(storage: np.ndarray, kind: str, device) -> torch.Tensor:
    """Uploads oracle storage (uint16 bits for 16-bit floats) as a tensor of the matching dtype."""
    t = torch.from_numpy(np.ascontiguousarray(storage))
    if kind in ("f16", "bf16"):
        t = t.view(torch.int16).view(TORCH_OF[kind])
    return t.to(device)


def to_host(t: torch.Tensor, kind: str) -> np.ndarray:
    """Downloads a tensor back into oracle storage."""
    t = t.detach().cpu().contiguous()
    if kind in ("f16", "bf16"):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def upload_csr(A, kind: str, device, oracle):
    from ops_sparse_b200 import api

    val = oracle.to_storage(A.values, kind)
    return api.CsrMatrix(torch.from_numpy(A.row_ptr).to(device), torch.from_numpy(A.col_ind).to(device),
                         to_device(val, kind, device), A.rows, A.cols), val


def assert_rowwise(got64: np.ndarray, gold64: np.ndarray, scale: np.ndarray, tol: float, what: str) -> None:
    err = np.abs(got64 - gold64)
    bad = ~(err <= tol * scale + 1e-37)
    if bad.any():
        i = int(np.argmax(np.where(bad, err / (scale + 1e-37), 0)))
        raise AssertionError(f"{what}: {int(bad.sum())} of {err.size} outputs outside tol {tol:g}; "
                             f"worst at flat index {i}: got {got64.ravel()[i]!r} gold {gold64.ravel()[i]!r} "
                             f"scale {scale.ravel()[i]!r}")


def make_csr(device, rp, ci, val, vt, rows, cols):
    """CSR descriptor over storage arrays.  Empty index / value arrays are given one padding
    element, because the API (like the reference) rejects null CSR pointers."""
    from ops_sparse_b200 import api

    nnz = int(ci.size)
    d_ci = torch.from_numpy(np.ascontiguousarray(ci)).to(device) if nnz else torch.zeros(1, dtype=torch.int32, device=device)
    d_val = to_device(val, vt, device) if nnz else torch.zeros(1, dtype=TORCH_OF[vt], device=device)
    return api.CsrMatrix(torch.from_numpy(np.ascontiguousarray(rp)).to(device), d_ci, d_val, rows, cols, nnz=nnz)
