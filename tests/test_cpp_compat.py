"""include/shflbw_compat.hpp: reference-style C++ caller code builds against the library
(CPU: compile + link) and, on a GPU, runs and passes its own check.  One caller per example of
the reference project: example/spmm.blockwise.cu, example/spconv.blockwise.cu and
example/load_bsr.spmm.blockwise.cu (which reads a matrix dump from stdin)."""
import ctypes
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CPP = ROOT / "tests" / "cpp"
LIBDIR = ROOT / "shflbw_sparse_nn_b200"
EXAMPLES = ["compat_spmm_example", "compat_spconv_example", "compat_load_bsr_spmm_example"]


def _build(name: str) -> Path:
    src, exe = CPP / f"{name}.cu", CPP / f"{name}.bin"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    newest = max(src.stat().st_mtime, (ROOT / "include" / "shflbw_compat.hpp").stat().st_mtime,
                 (ROOT / "include" / "shflbw.h").stat().st_mtime)
    if exe.exists() and exe.stat().st_mtime > newest:
        return exe
    cmd = [nvcc, "-ccbin", "g++", "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", str(ROOT / "include"), "-o", str(exe), str(src), "-L", str(LIBDIR), "-lshflbw_b200",
           "-Xlinker", f"-rpath={LIBDIR}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


@pytest.mark.parametrize("name", EXAMPLES)
def test_compat_example_compiles_and_links(name):
    assert _build(name).exists()


@pytest.mark.gpu
@pytest.mark.parametrize("name", EXAMPLES[:2])
def test_compat_example_runs_and_passes(name):
    res = subprocess.run([str(_build(name))], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.rstrip().endswith("Passed"), res.stdout + res.stderr


@pytest.mark.gpu
def test_load_from_stdin_example_runs_on_the_reference_dump():
    """The dump fed to the example is the reference's own example/mtx_dump.txt, regenerated here:
    1024 x 1024, V = 32, density 0.2, seed 2021, no permutation, libc values (the builder test
    pins that text byte for byte)."""
    import shflbw_sparse_nn_b200 as sb
    ctypes.CDLL(None).srand(1)
    m = sb.BlockwiseSpMatrix().init_random(1024, 1024, 32, 1, 0.2, False, 2021, values="int9")
    res = subprocess.run([str(_build(EXAMPLES[2]))], input=m.dump().decode(), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.rstrip().endswith("Passed"), res.stdout + res.stderr
    assert "Finish matrix loading" in res.stdout
