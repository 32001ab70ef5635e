"""include/shflbw_compat.hpp: reference-style C++ caller code builds against the library
(CPU: compile + link) and, on a GPU, runs and passes its own check."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "cpp" / "compat_spmm_example.cu"
EXE = ROOT / "tests" / "cpp" / "compat_spmm_example.bin"
LIBDIR = ROOT / "shflbw_sparse_nn_b200"


def _build():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if EXE.exists() and EXE.stat().st_mtime > max(SRC.stat().st_mtime, (ROOT / "include" / "shflbw_compat.hpp").stat().st_mtime):
        return
    cmd = [nvcc, "-ccbin", "g++", "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", str(ROOT / "include"), "-o", str(EXE), str(SRC), "-L", str(LIBDIR), "-lshflbw_b200",
           "-Xlinker", f"-rpath={LIBDIR}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_compat_example_compiles_and_links():
    _build()
    assert EXE.exists()


@pytest.mark.gpu
def test_compat_example_runs_and_passes():
    _build()
    res = subprocess.run([str(EXE)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "Passed" in res.stdout, res.stdout + res.stderr
