"""Builds libarm_compute_cuda.so: the C++ function family (CUGEMMLowpMatrixMultiplyCore, CUGEMMLowpOutputStage,
CUGEMMConvolutionLayer, CUTensor, CUScheduler) on top of libcugl.so.  Plain g++; no CUDA headers are needed on
this side of the C ABI."""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libarm_compute_cuda.so")
INCLUDES = [os.path.join(HERE, "include"), os.path.join(ROOT, "include")]


def compile_flags() -> list[str]:
    return ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra"] + [f"-I{i}" for i in INCLUDES]


def link_flags() -> list[str]:
    return [f"-L{LIB_DIR}", "-lcugl", f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,$ORIGIN"]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = glob.glob(os.path.join(HERE, "src", "*.cpp")) + glob.glob(os.path.join(HERE, "include", "**", "*.h"),
                                                                     recursive=True)
    deps.append(os.path.join(ROOT, "include", "cugl.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False) -> str:
    from computelibrary_b200 import build as cuda_build
    cuda_build.build()
    if not force and not _stale():
        return LIB_PATH
    cxx = shutil.which("g++") or "g++"
    srcs = sorted(glob.glob(os.path.join(HERE, "src", "*.cpp")))
    cmd = [cxx, *compile_flags(), "-shared", "-o", LIB_PATH, *srcs, *link_flags()]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("g++ failed building libarm_compute_cuda.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
