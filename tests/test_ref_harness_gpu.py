"""GPU: the reference's own harness programs, compiled unmodified from its sources against
include/ and linked with libops_sparse.so (oracle/build_oracle.py), must pass on a B200.

They only exist where the reference checkout was present at build time; the built
executables travel with the tree.  Each program generates its inputs, runs its CPU golden,
calls the aclsparse API and applies its own verifier; exit status 0 means every case passed.
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

REF = Path(__file__).resolve().parents[1] / "oracle" / "_ref"


def run(name: str, timeout: int):
    exe = REF / name
    if not exe.exists():
        pytest.skip(f"{exe} was not built (reference sources absent at build time)")
    env = dict(os.environ, B200SP_LOG_LEVEL="1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=timeout, env=env)
    tail = "\n".join((r.stdout + r.stderr).splitlines()[-40:])
    assert r.returncode == 0, f"{name} exited {r.returncode}\n{tail}"
    return r.stdout


def test_reference_spmv_harness(built, device):
    out = run("spmv_test", 900)
    assert "case fail" not in out


def test_reference_spmm_arch35_harness(built, device):
    out = run("spmm35_test", 300)
    assert "Overall: PASS" in out


@pytest.mark.skipif(os.environ.get("B200SP_RUN_SLOW_HARNESS") != "1",
                    reason="the arch22 harness spends about 8 minutes in its own CPU golden loops (200 cases x 10 "
                           "timed repetitions); set B200SP_RUN_SLOW_HARNESS=1 to run it")
def test_reference_spmm_arch22_harness(built, device):
    out = run("spmm22_test", 1500)
    assert "Total: 0 failed" in out
