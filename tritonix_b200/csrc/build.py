"""Builds libtritonix_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python tritonix_b200/csrc/build.py [--force] [--verbose]
(run as a script: importing the tritonix_b200 package itself requires the built library)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libtritonix_b200.so"
SOURCES = ["tnx_api.cu", "tnx_umma_gemm.cu", "tnx_strided_gemm.cu", "tnx_conv2d.cu",
           "tnx_swiglu_mlp.cu"]
HEADERS = ["tnx_ptx.cuh", "tnx_internal.h", "../../include/tritonix_b200.h"]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA kernels of tritonix_b200 cannot be built")
    return nvcc


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library.  Returns its path."""
    nvcc = find_nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = CSRC / "build"
    obj_dir.mkdir(exist_ok=True)
    headers = [(CSRC / h).resolve() for h in HEADERS]
    jobs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        if force or _stale(obj, [CSRC / src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stdout + r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out)
    objs = [obj_dir / (s + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB_PATH, objs):
        run([nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"])
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
