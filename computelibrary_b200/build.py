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

OBJ_DIR = os.path.join(LIB_DIR, "obj")
NVCC_COMPILE_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
]
NVCC_LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the cugl library cannot be built")


def _includes() -> list[str]:
    return ["-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _compile_one(src: str, verbose: bool) -> str:
    """One translation unit -> lib/obj/<name>.o, skipped when the object is newer than the source and headers."""
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    deps = [os.path.join(CSRC, src)] + [os.path.join(CSRC, h) for h in HEADERS] + [os.path.join(ROOT, "include", "cugl.h")]
    if src.startswith("gemmlowp_tcgen05_epi"):
        deps.append(os.path.join(CSRC, "gemmlowp_tcgen05.cu"))  # these units re-include it with another warp count
    if os.path.exists(obj) and all(os.path.getmtime(d) <= os.path.getmtime(obj) for d in deps):
        return obj
    cmd = [_nvcc(), *NVCC_COMPILE_FLAGS, *_includes(), "-ccbin", shutil.which("g++") or "g++"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source (in parallel, one object each) and link one shared library; returns its path."""
    from concurrent.futures import ThreadPoolExecutor
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, verbose), SOURCES))
    if not force and os.path.exists(LIB_PATH) and all(os.path.getmtime(o) <= os.path.getmtime(LIB_PATH) for o in objs):
        return LIB_PATH
    # the image exports CC/CXX pointing at a toolchain without libgomp; nvcc must use the system g++
    cmd = [_nvcc(), *NVCC_LINK_FLAGS, "-ccbin", shutil.which("g++") or "g++", *objs, "-o", LIB_PATH]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libcugl.so")
    return LIB_PATH


PROBE_PATH = os.path.join(LIB_DIR, "probe_tcgen05_rates")


def build_probe(force: bool = False) -> str:
    """The stand-alone program that measures tcgen05 issue rates (bench.py --workload tcgen05_rates runs it)."""
    src = os.path.join(CSRC, "probe_tcgen05_rates.cu")
    os.makedirs(LIB_DIR, exist_ok=True)
    if not force and os.path.exists(PROBE_PATH) and os.path.getmtime(src) <= os.path.getmtime(PROBE_PATH):
        return PROBE_PATH
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-cudart", "static",
           "-ccbin", shutil.which("g++") or "g++", src, "-o", PROBE_PATH]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed on probe_tcgen05_rates.cu")
    return PROBE_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
