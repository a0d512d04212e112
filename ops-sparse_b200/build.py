"""Builds libops_sparse.so (the aclsparse C API + sm_100a kernels) in-tree with nvcc.

Run as a script (`python ops-sparse_b200/build.py [--force] [--verbose]`) or call
`build()`.  The library lands in ops-sparse_b200/lib/libops_sparse.so; nothing is
installed outside the source tree.  Compilation needs no GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libops_sparse.so"

SOURCES = [
    "common/context.cpp",
    "common/descr.cpp",
    "common/repeat.cpp",
    "common/host_product.cpp",
    "spmv/spmv_host.cpp",
    "spmv/spmv_kernels.cu",
    "spmv_op/spmv_op_host.cpp",
    "spmv_op/spmv_op_kernels.cu",
    "convert/coo2csr.cu",
    "convert/csrsort.cu",
    "convert/csr2csc.cu",
    "sddmm/sddmm.cu",
    "spmm/spmm_host.cpp",
    "spmm/spmm_kernels.cu",
    "mg/partition.cpp",
    "mg/exchange.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++20",
    "-Xcompiler", "-fPIC,-Wall,-Wextra",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libops_sparse.so")
    return exe


def _stamp(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.relative_to(ROOT)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source for sm_100a and link the shared library.  Returns its path."""
    srcs = [CSRC / s for s in SOURCES]
    headers = sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")) + sorted((ROOT / "include").rglob("*.h"))
    stamp = _stamp(srcs + headers, " ".join(NVCC_FLAGS))
    stamp_file = LIB_DIR / "build.stamp"
    if not force and LIB_PATH.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB_PATH

    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    inc = ["-I", str(ROOT / "include"), "-I", str(CSRC)]
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.relative_to(CSRC).as_posix().replace("/", "_") + ".o")
        cmd = [nvcc, *flags, *inc, "-DB200SP_BUILDING", "-c", str(src), "-o", str(obj)]
        if src.suffix == ".cpp":
            cmd[1:1] = ["-x", "cu"]  # host files include cuda_runtime_api.h only; one compiler for all
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{r.stdout}{r.stderr}")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, srcs))

    # nvcc links the CUDA runtime statically by default: the library then does not depend on
    # which libcudart.so a host process (for instance one that imported torch) loaded first.
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs),
           "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link of libops_sparse.so failed")
    stamp_file.write_text(stamp)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
