"""The C++ function family (CUGEMMLowpMatrixMultiplyCore, CUGEMMLowpOutputStage, CUGEMMConvolutionLayer,
CUTensor) driven by a C++ program written like the reference's examples; the program compares with the oracle."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "test_cu_functions")


def build_exe():
    from computelibrary_b200.host import build as hb
    import oracle
    hb.build()
    if not os.path.exists(oracle.PORT_SO):
        oracle.build(want_ref=False)
    src = EXE + ".cpp"
    deps = [src, hb.LIB_PATH, oracle.PORT_SO]
    if os.path.exists(EXE) and all(os.path.getmtime(d) <= os.path.getmtime(EXE) for d in deps):
        return EXE
    odir = os.path.dirname(oracle.PORT_SO)
    cmd = [shutil.which("g++") or "g++", *hb.compile_flags(), src, "-o", EXE, f"-L{hb.LIB_DIR}", "-larm_compute_cuda",
           "-lcugl", f"-Wl,-rpath,{hb.LIB_DIR}", f"-L{odir}", "-lgemmlowp_oracle", f"-Wl,-rpath,{odir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return EXE


def test_cpp_validate_rules_host_only():
    exe = build_exe()
    res = subprocess.run([exe, "--validate"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_functions_on_gpu():
    exe = build_exe()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
