"""Builds the test-side CPU code under oracle/.

  oracle/_build/liboracle.so      the CPU restatement (oracle.cpp), always built
  oracle/_ref/libref_*.so         the reference's own golden functions, compiled from the
                                  reference checkout where it lies (only when it is present)
  oracle/_ref/libref_{convert,sddmm}.so
                                  the reference's golden headers for the CSR producers and SDDMM, likewise
  oracle/_ref/{spmv,spmm35,spmm22}_test
                                  the reference's own harness programs, unmodified, linked
                                  against libops_sparse.so through the acl->CUDA shim headers
The reference checkout is looked for at $B200SP_REFERENCE_DIR, else in a `reference` directory beside this
repository.

Nothing built here is part of the shipped library.  `python oracle/build_oracle.py [--force]`.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
BUILD = HERE / "_build"
REFOUT = HERE / "_ref"
ORACLE_LIB = BUILD / "liboracle.so"
# Where the reference checkout lies: B200SP_REFERENCE_DIR, or a `reference` directory beside this repository.
REFERENCE = Path(os.environ.get("B200SP_REFERENCE_DIR", str(ROOT.parent / "reference")))
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

REF_UNITS = {
    "spmv": ("test/spmv/arch22/spmv_test.cpp", "ref_wrap_spmv.cpp"),
    "spmm35": ("test/spmm/arch35/spmm_test.cpp", "ref_wrap_spmm35.cpp"),
    "spmm22": ("test/spmm/arch22/spmm_test.cpp", "ref_wrap_spmm22.cpp"),
}


# Golden headers of the operators next to the hot path (CSR producers, SDDMM): header-only, wrapped as libraries.
REF_HEADER_UNITS = {
    "convert": ("ref_wrap_convert.cpp", {
        "REF_CSRSORT_GOLDEN": "test/csrsort/arch35/csrsort_golden.h",
        "REF_COO2CSR_GOLDEN": "test/coo2csr/coo2csr_golden.h",
        "REF_CSR2CSC_GOLDEN": "test/csr2csc_ex2/csr2csc_ex2_golden.h",
    }),
    "sddmm": ("ref_wrap_sddmm.cpp", {"REF_SDDMM_GOLDEN": "test/sddmm/sddmm/sddmm_golden.h"}),
}


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(f"$ {' '.join(cmd)}\n{r.stdout}{r.stderr}")
        raise RuntimeError(f"command failed: {cmd[0]} ... {cmd[-1]}")


def _newer(target: Path, *sources: Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources if s.exists())


def build_oracle(force: bool = False) -> Path:
    src = HERE / "oracle.cpp"
    if force or not _newer(ORACLE_LIB, src):
        BUILD.mkdir(exist_ok=True)
        # -ffp-contract=off: keep a*b+c as two roundings, like the golden's plain expression.
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-ffp-contract=off", "-Wall", "-Wextra",
              str(src), "-o", str(ORACLE_LIB)])
    return ORACLE_LIB


def reference_present() -> bool:
    return all((REFERENCE / rel).exists() for rel, _ in REF_UNITS.values())


def build_reference(force: bool = False, ops_lib: Path | None = None) -> dict[str, Path]:
    """Compile the reference's harness sources in place.  Returns the built artefacts."""
    if not reference_present():
        return {}
    REFOUT.mkdir(exist_ok=True)
    ops_lib = ops_lib or ROOT / "ops-sparse_b200" / "lib" / "libops_sparse.so"
    inc = ["-I", str(HERE / "ref_shim"), "-I", str(ROOT / "include"), "-I", str(CUDA_HOME / "include")]
    link = ["-L", str(ops_lib.parent), "-lops_sparse", "-L", str(CUDA_HOME / "lib64"), "-lcudart",
            f"-Wl,-rpath,$ORIGIN/../../ops-sparse_b200/lib", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]
    common = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-w", *inc]
    out: dict[str, Path] = {}
    for name, (rel, wrap) in REF_UNITS.items():
        ref_src = REFERENCE / rel
        lib = REFOUT / f"libref_{name}.so"
        exe = REFOUT / f"{name}_test"
        if force or not _newer(lib, ref_src, HERE / wrap, ops_lib):
            _run([*common, "-fPIC", "-shared", f'-DREF_SOURCE="{ref_src}"', str(HERE / wrap), "-o", str(lib), *link])
        if force or not _newer(exe, ref_src, ops_lib):
            _run([*common, str(ref_src), "-o", str(exe), *link])
        out[f"lib_{name}"] = lib
        out[f"exe_{name}"] = exe
    frame = ["-I", str(REFERENCE / "test" / "frame")]
    for name, (wrap, headers) in REF_HEADER_UNITS.items():
        srcs = [REFERENCE / rel for rel in headers.values()]
        if not all(p.exists() for p in srcs):
            continue
        lib = REFOUT / f"libref_{name}.so"
        if force or not _newer(lib, HERE / wrap, *srcs):
            defs = [f'-D{macro}="{REFERENCE / rel}"' for macro, rel in headers.items()]
            _run([*common, *frame, "-fPIC", "-shared", *defs, str(HERE / wrap), "-o", str(lib)])
        out[f"lib_{name}"] = lib
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    for k, v in build_reference(force).items():
        print(k, v)
