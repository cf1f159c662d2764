"""Builds libcugl.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m computelibrary_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library lands in computelibrary_b200/lib/libcugl.so so that it
travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libcugl.so")
SOURCES = ["context.cu", "bandwidth_kernels.cu", "gemmlowp_simt.cu", "gemmlowp_tcgen05.cu", "plans.cu", "noalloc.cu",
           "layer_kernels.cu", "gemmlowp_tcgen05_epi8.cu", "gemmlowp_tcgen05_epi16.cu",
           "gemmlowp_dispatch.cu"]
HEADERS = ["common.cuh", "kernels.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-shared", "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the cugl library cannot be built")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(ROOT, "include", "cugl.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source into one shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB_PATH]
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a toolchain without libgomp; nvcc must use the system g++
    cmd += ["-ccbin", shutil.which("g++") or "g++"]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libcugl.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
