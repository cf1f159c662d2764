"""Builds the host-side C++ of the CUDA backend against an UNMODIFIED Compute Library tree.

    python -m computelibrary_b200.host.build [--force] [ACL_ROOT=<tree>]

Three shared libraries land in computelibrary_b200/lib/ (git-ignored; they travel with the source tree):

  libarm_compute_host.so  Compute Library's own host-side core and runtime sources -- TensorInfo, Tensor,
                          TensorAllocator, MemoryGroup / MemoryManagerOnDemand / BlobLifetimeManager / PoolManager,
                          Utils, AsymmHelpers ... -- compiled IN PLACE from $ACL_ROOT (nothing is copied, the
                          reference's SCons / CMake build is not used: those refuse to build the library for x86-64
                          with neon=1, and none of these files needs NEON).
  libarm_compute_cuda.so  the CU* function family of this repository (CUTensor, CUAllocator, CUScheduler,
                          CUGEMMLowpMatrixMultiplyCore, CUGEMMLowpOutputStage, CUGEMMConvolutionLayer, ...),
                          compiled against the reference's own headers (-I$ACL_ROOT -I$ACL_ROOT/include) and linked
                          to libarm_compute_host.so and libcugl.so.
  libarm_compute_graph_cuda.so  Compute Library's graph frontend and IR (src/graph/**, without its NEON and CL
                          backends), compiled in place, together with this repository's graph backend
                          (host/src/graph/: CUDeviceBackend, CUTensorHandle, CUFunctionFactory), which registers itself
                          when the library is loaded.

Inside Compute Library itself the second set of sources would simply be added to the library's source list
(SConscript / filelist.json) next to src/runtime/NEON and src/runtime/CL.
Without a Compute Library tree the prebuilt libraries are used as they are (the GPU box has none).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj_host")
ACL_HOST_LIB = os.path.join(LIB_DIR, "libarm_compute_host.so")
LIB_PATH = os.path.join(LIB_DIR, "libarm_compute_cuda.so")
GRAPH_LIB = os.path.join(LIB_DIR, "libarm_compute_graph_cuda.so")

# The reference's host sources behind the API types of the path (relative to the tree).  Left out on purpose:
# src/core/GPUTarget.cpp (OpenCL), src/core/Version.cpp (needs a generated header), src/core/utils/ScaleUtils.cpp
# (pulls in CPUInfo), the schedulers (the CUDA backend has its own) and everything under src/cpu, src/gpu.
ACL_GLOBS = ["src/core/*.cpp", "src/core/utils/*.cpp", "src/core/utils/*/*.cpp", "src/core/helpers/*.cpp"]
ACL_EXCLUDE = {"src/core/GPUTarget.cpp", "src/core/Version.cpp", "src/core/utils/ScaleUtils.cpp"}
ACL_RUNTIME = ["Allocator", "BlobLifetimeManager", "BlobMemoryPool", "ISimpleLifetimeManager", "ITensorAllocator",
               "IWeightsManager", "Memory", "MemoryManagerOnDemand", "OffsetLifetimeManager", "OffsetMemoryPool",
               "PoolManager", "SubTensor", "Tensor", "TensorAllocator"]
ACL_DEFINES = ["-DARM_COMPUTE_CPU_ENABLED", "-DARM_COMPUTE_ASSERTS_ENABLED"]
# the graph library: everything under src/graph except the two device backends of the reference
ACL_GRAPH_GLOBS = ["src/graph/*.cpp", "src/graph/*/*.cpp", "src/graph/backends/BackendRegistry.cpp"]


def find_acl_root() -> str | None:
    """$ACL_ROOT, else a directory named "reference" beside this repository."""
    for cand in (os.environ.get("ACL_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "arm_compute", "core", "TensorInfo.h")):
            return cand
    return None


def acl_sources(acl_root: str) -> list[str]:
    rel = []
    for g in ACL_GLOBS:
        rel += [os.path.relpath(p, acl_root) for p in glob.glob(os.path.join(acl_root, g))]
    rel = sorted(set(rel) - ACL_EXCLUDE)
    rel += [f"src/runtime/{n}.cpp" for n in ACL_RUNTIME]
    return rel


def acl_graph_sources(acl_root: str) -> list[str]:
    rel = []
    for g in ACL_GRAPH_GLOBS:
        rel += [os.path.relpath(p, acl_root) for p in glob.glob(os.path.join(acl_root, g))]
    return sorted(r for r in set(rel) if "/backends/NEON/" not in r and "/backends/CL/" not in r)


def include_flags(acl_root: str) -> list[str]:
    return [f"-I{acl_root}", f"-I{acl_root}/include", f"-I{acl_root}/src/cpu/kernels/assembly",
            f"-I{os.path.join(HERE, 'include')}", f"-I{os.path.join(HERE, 'src')}", f"-I{os.path.join(ROOT, 'include')}"]


def compile_flags(acl_root: str) -> list[str]:
    return ["-std=c++17", "-O2", "-fPIC", *ACL_DEFINES, *include_flags(acl_root)]


def link_flags(graph: bool = False) -> list[str]:
    return [f"-L{LIB_DIR}", *(["-larm_compute_graph_cuda"] if graph else []), "-larm_compute_cuda", "-larm_compute_host", "-lcugl", f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,$ORIGIN",
            "-lpthread"]


def _cxx() -> str:
    return shutil.which("g++") or "g++"


def _compile(src: str, obj: str, flags: list[str], extra_deps: list[str]) -> str:
    deps = [src] + extra_deps
    if os.path.exists(obj) and all(os.path.getmtime(d) <= os.path.getmtime(obj) for d in deps):
        return obj
    res = subprocess.run([_cxx(), *flags, "-c", src, "-o", obj], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"g++ failed on {src}")
    return obj


def _link(objs: list[str], out: str, extra: list[str]) -> None:
    if os.path.exists(out) and all(os.path.getmtime(o) <= os.path.getmtime(out) for o in objs):
        return
    res = subprocess.run([_cxx(), "-shared", "-o", out, *objs, *extra], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"g++ failed linking {out}")


def build(force: bool = False, acl_root: str | None = None) -> str:
    from computelibrary_b200 import build as cuda_build
    cuda_build.build()
    acl_root = acl_root or find_acl_root()
    if acl_root is None:
        if os.path.exists(LIB_PATH) and os.path.exists(ACL_HOST_LIB) and os.path.exists(GRAPH_LIB):
            return LIB_PATH  # prebuilt libraries travel with the tree
        raise RuntimeError("no Compute Library tree (set ACL_ROOT) and no prebuilt libarm_compute_cuda.so")
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    workers = os.cpu_count() or 1
    # 1. the reference's host sources, where they lie
    warn_off = ["-w"]  # the reference builds with its own warning set; not ours to police
    acl = acl_sources(acl_root)
    with ThreadPoolExecutor(max_workers=workers) as pool:
        acl_objs = list(pool.map(lambda r: _compile(os.path.join(acl_root, r),
                                                    os.path.join(OBJ_DIR, "acl_" + r.replace("/", "_")[:-4] + ".o"),
                                                    compile_flags(acl_root) + warn_off, []), acl))
    _link(acl_objs, ACL_HOST_LIB, ["-Wl,--no-undefined", "-lpthread"])
    # 2. the CUDA function family
    headers = glob.glob(os.path.join(HERE, "include", "**", "*.h"), recursive=True) + glob.glob(os.path.join(HERE, "src", "*.h"))
    headers.append(os.path.join(ROOT, "include", "cugl.h"))
    srcs = sorted(glob.glob(os.path.join(HERE, "src", "*.cpp")))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        cu_objs = list(pool.map(lambda s: _compile(s, os.path.join(OBJ_DIR, "cu_" + os.path.basename(s)[:-4] + ".o"),
                                                   compile_flags(acl_root) + ["-Wall", "-Wextra"], headers), srcs))
    _link(cu_objs, LIB_PATH, [f"-L{LIB_DIR}", "-larm_compute_host", "-lcugl", f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,$ORIGIN",
                              "-Wl,--no-undefined", "-lpthread"])
    # 3. the reference's graph library + the CUDA graph backend
    gsrc = acl_graph_sources(acl_root)
    bsrc = sorted(glob.glob(os.path.join(HERE, "src", "graph", "*.cpp")))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        g_objs = list(pool.map(lambda r: _compile(os.path.join(acl_root, r),
                                                  os.path.join(OBJ_DIR, "aclg_" + r.replace("/", "_")[:-4] + ".o"),
                                                  compile_flags(acl_root) + warn_off, []), gsrc))
        g_objs += list(pool.map(lambda s: _compile(s, os.path.join(OBJ_DIR, "cug_" + os.path.basename(s)[:-4] + ".o"),
                                                   compile_flags(acl_root) + ["-Wall", "-Wextra"], headers), bsrc))
    _link(g_objs, GRAPH_LIB, [f"-L{LIB_DIR}", "-larm_compute_cuda", "-larm_compute_host", "-lcugl", f"-Wl,-rpath,{LIB_DIR}",
                              "-Wl,-rpath,$ORIGIN", "-Wl,--no-undefined", "-lpthread"])
    return LIB_PATH


if __name__ == "__main__":
    root = next((a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("ACL_ROOT=")), None)
    print(build(force="--force" in sys.argv, acl_root=root))
