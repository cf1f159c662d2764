"""The C++ function family (CUGEMMLowpMatrixMultiplyCore, CUGEMMLowpOutputStage, CUGEMMConvolutionLayer,
CUTensor) driven by a C++ program written like the reference's examples; the program compares with the oracle."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "test_cu_functions")


def build_exe():
    """Compiles the program against the Compute Library headers where a tree is present; elsewhere (the GPU
    box) the executable built beforehand is used as it is."""
    from computelibrary_b200.host import build as hb
    import oracle
    acl_root = hb.find_acl_root()
    if acl_root is None:
        assert os.path.exists(EXE), "no Compute Library tree and no prebuilt tests/cpp/test_cu_functions"
        return EXE
    hb.build()
    if not os.path.exists(oracle.PORT_SO):
        oracle.build(want_ref=False)
    src = EXE + ".cpp"
    deps = [src, hb.LIB_PATH, oracle.PORT_SO]
    if os.path.exists(EXE) and all(os.path.getmtime(d) <= os.path.getmtime(EXE) for d in deps):
        return EXE
    odir = os.path.dirname(oracle.PORT_SO)
    cmd = [shutil.which("g++") or "g++", *hb.compile_flags(acl_root), "-Wall", "-Wextra", src, "-o", EXE, *hb.link_flags(),
           f"-L{odir}", "-lgemmlowp_oracle", f"-Wl,-rpath,{odir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return EXE


FIXTURE_EXE = os.path.join(ROOT, "tests", "cpp", "test_reference_fixture")
# What the reference's fixture headers pull in besides the library itself: its validation framework, the asset
# library's seeded fills, the scalar oracles, and the scheduler / CPU-info singletons the framework's timers name.
# Compiled in place from the Compute Library tree; nothing is copied.
FIXTURE_ACL_SOURCES = [
    "tests/AssetsLibrary.cpp", "tests/RawTensor.cpp", "tests/validation/Helpers.cpp",
    "tests/validation/reference/GEMMLowp.cpp", "tests/validation/reference/ArithmeticOperations.cpp",
    "tests/validation/reference/DequantizationLayer.cpp",
    "tests/framework/Framework.cpp", "tests/framework/Exceptions.cpp", "tests/framework/Utils.cpp",
    "tests/framework/TestFilter.cpp", "tests/framework/Profiler.cpp",
    "tests/framework/instruments/WallClockTimer.cpp", "tests/framework/instruments/SchedulerTimer.cpp",
    "tests/framework/instruments/Instruments.cpp",
    "src/core/CPP/CPPTypes.cpp", "src/common/cpuinfo/CpuInfo.cpp", "src/common/cpuinfo/CpuIsaInfo.cpp",
    "src/common/cpuinfo/CpuModel.cpp", "src/runtime/IScheduler.cpp", "src/runtime/Scheduler.cpp",
    "src/runtime/SchedulerUtils.cpp", "src/runtime/CPP/SingleThreadScheduler.cpp",
]


def build_fixture_exe():
    """The reference's own GEMMLowp validation fixtures instantiated with the CUDA FunctionType / TensorType /
    AccessorType triple (tests/cpp/test_reference_fixture.cpp).  Needs a Compute Library tree to build; the
    executable travels prebuilt to machines without one."""
    from concurrent.futures import ThreadPoolExecutor
    from computelibrary_b200.host import build as hb
    acl_root = hb.find_acl_root()
    if acl_root is None:
        assert os.path.exists(FIXTURE_EXE), "no Compute Library tree and no prebuilt tests/cpp/test_reference_fixture"
        return FIXTURE_EXE
    hb.build()
    src = FIXTURE_EXE + ".cpp"
    deps = [src, os.path.join(ROOT, "tests", "cpp", "CUAccessor.h"), hb.LIB_PATH]
    if os.path.exists(FIXTURE_EXE) and all(os.path.getmtime(d) <= os.path.getmtime(FIXTURE_EXE) for d in deps):
        return FIXTURE_EXE
    obj_dir = os.path.join(ROOT, "tests", "cpp", "obj")
    os.makedirs(obj_dir, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    flags = [*hb.compile_flags(acl_root), f"-I{ROOT}", "-w"]

    def compile_one(rel):
        obj = os.path.join(obj_dir, rel.replace("/", "_")[:-4] + ".o")
        if not os.path.exists(obj):
            res = subprocess.run([cxx, *flags, "-c", os.path.join(acl_root, rel), "-o", obj], capture_output=True, text=True)
            assert res.returncode == 0, res.stderr
        return obj

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 1) as pool:
        objs = list(pool.map(compile_one, FIXTURE_ACL_SOURCES))
    res = subprocess.run([cxx, *flags, src, *objs, "-o", FIXTURE_EXE, *hb.link_flags(), "-fopenmp"], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return FIXTURE_EXE


GRAPH_TEST_EXE = os.path.join(ROOT, "tests", "cpp", "test_graph_backend")
GRAPH_EXAMPLE_EXE = os.path.join(ROOT, "tests", "cpp", "graph_resnet50")


def _build_graph_program(exe, sources, acl_sources=()):
    """A program on the graph frontend + the CUDA graph backend.  `acl_sources` are files of the Compute Library tree
    compiled where they lie (the example itself and the utilities it uses)."""
    from computelibrary_b200.host import build as hb
    import oracle
    acl_root = hb.find_acl_root()
    if acl_root is None:
        assert os.path.exists(exe), f"no Compute Library tree and no prebuilt {os.path.relpath(exe, ROOT)}"
        return exe
    hb.build()
    if not os.path.exists(oracle.PORT_SO):
        oracle.build(want_ref=False)
    deps = list(sources) + [hb.GRAPH_LIB, hb.LIB_PATH]
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    odir = os.path.dirname(oracle.PORT_SO)
    cmd = [shutil.which("g++") or "g++", *hb.compile_flags(acl_root), f"-I{ROOT}", "-w", *sources,
           *[os.path.join(acl_root, r) for r in acl_sources], "-o", exe, *hb.link_flags(graph=True), f"-L{odir}",
           "-lgemmlowp_oracle", f"-Wl,-rpath,{odir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def build_graph_exes():
    t = _build_graph_program(GRAPH_TEST_EXE, [GRAPH_TEST_EXE + ".cpp"])
    # the reference's own example, unmodified, on the graph frontend
    e = _build_graph_program(GRAPH_EXAMPLE_EXE, [], ["examples/graph_resnet50.cpp", "utils/GraphUtils.cpp", "utils/Utils.cpp",
                                                     "utils/CommonGraphOptions.cpp"])
    return t, e


def test_cpp_validate_rules_host_only():
    exe = build_exe()
    res = subprocess.run([exe, "--validate"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_functions_on_gpu():
    exe = build_exe()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_reference_fixtures_with_the_cuda_triple():
    """Compute Library's GEMMLowp fixtures (S32 core, run-twice, accumulate, fused fixed-point and integer stages,
    batched, dequantised F32) run with CUGEMMLowpMatrixMultiplyCore / CUTensor / CUAccessor and compared with the
    reference the fixtures compute themselves."""
    exe = build_fixture_exe()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_graph_frontend_on_the_cuda_backend():
    """A reduced ResNet built with the reference's graph frontend runs on the CUDA backend and matches the oracle."""
    exe, _ = build_graph_exes()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_reference_graph_resnet50_example_runs_unmodified():
    """examples/graph_resnet50.cpp of the reference, compiled as it is, in its synthetic QASYMM8 mode (random weights,
    no data files): --target=CL selects the CUDA backend in a build without OpenCL."""
    _, exe = build_graph_exes()
    res = subprocess.run([exe, "--target=CL", "--type=QASYMM8", "--layout=NHWC", "--batches=4"], capture_output=True, text=True,
                         timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "Test passed" in res.stdout or res.returncode == 0
