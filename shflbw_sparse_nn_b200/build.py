"""In-tree build of the native library (nvcc, sm_100a only).

`python -m shflbw_sparse_nn_b200.build` or `build_library()` compiles
`csrc/shflbw_capi.cu` + `csrc/shflbw_format.cc` into `libshflbw_b200.so` next to this file.
nvcc cross-compiles without a GPU.  The shared object is git-ignored; it is a build product.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent
LIB_PATH = PKG_DIR / "libshflbw_b200.so"
SOURCES = [PKG_DIR / "csrc" / "shflbw_capi.cu", PKG_DIR / "csrc" / "shflbw_format.cc"]
HEADERS = [
    PKG_DIR / "csrc" / "panel_umma.cuh",
    PKG_DIR / "csrc" / "aux_kernels.cuh",
    PKG_DIR / "csrc" / "sm100_ptx.cuh",
    PKG_DIR / "csrc" / "shflbw_internal.hpp",
    REPO_ROOT / "include" / "shflbw.h",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")
    return cand


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if sources are newer than the binary. Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [
        _nvcc(), "-ccbin", "g++", "-O3", "-std=c++17",
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-Xcompiler", "-fPIC", "-shared",
        "-I", str(REPO_ROOT / "include"),
        "-o", str(LIB_PATH),
    ] + os.environ.get("SHFLBW_NVCC_FLAGS", "").split() + [str(s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr, file=sys.stderr)
    return LIB_PATH


FAULT_LIB_PATH = PKG_DIR / "libshflbw_b200_faultinject.so"


def build_fault_inject_library(force: bool = False) -> Path:
    """The same library compiled with -DSHFLBW_FAULT_INJECT: it adds one entry point that makes a
    producer warp withhold its barrier arrivals, so a test can watch a bounded in-kernel wait run
    out (and the library recover) without faulting or hanging the GPU.  Test infrastructure: the
    product library has no such switch."""
    if not force and FAULT_LIB_PATH.exists():
        built = FAULT_LIB_PATH.stat().st_mtime
        if all(p.stat().st_mtime <= built for p in SOURCES + HEADERS):
            return FAULT_LIB_PATH
    cmd = [
        _nvcc(), "-ccbin", "g++", "-O3", "-std=c++17",
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-Xcompiler", "-fPIC", "-shared", "-DSHFLBW_FAULT_INJECT",
        "-I", str(REPO_ROOT / "include"),
        "-o", str(FAULT_LIB_PATH),
    ] + [str(s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    return FAULT_LIB_PATH


TOOLS_DIR = PKG_DIR / "bin"
TOOL_SOURCE = PKG_DIR / "csrc" / "benchmark_cli.cu"


def build_tools(force: bool = False) -> dict:
    """Compile the command-line benchmarks (`bin/benchmark.spmm.out`, `bin/benchmark.spconv.out`):
    same flags and output line as the reference's tools of those names.  They link the library
    through an rpath relative to their own location."""
    build_library()
    TOOLS_DIR.mkdir(exist_ok=True)
    out = {}
    for name, defs in (("benchmark.spmm.out", []), ("benchmark.spconv.out", ["-DSHFLBW_BENCH_SPCONV"])):
        exe = TOOLS_DIR / name
        out[name] = exe
        deps = [TOOL_SOURCE, REPO_ROOT / "include" / "shflbw.h", REPO_ROOT / "include" / "shflbw_compat.hpp"]
        if not force and exe.exists() and all(d.stat().st_mtime <= exe.stat().st_mtime for d in deps):
            continue
        cmd = [_nvcc(), "-ccbin", "g++", "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-I", str(REPO_ROOT / "include"), *defs, str(TOOL_SOURCE), "-L", str(PKG_DIR), "-lshflbw_b200",
               "-Xlinker", "-rpath=$ORIGIN/..", "-o", str(exe)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--tools" in sys.argv:
        for exe in build_tools(force="--force" in sys.argv).values():
            print(exe)
