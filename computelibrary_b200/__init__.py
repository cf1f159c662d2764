"""B200 (sm_100a) backend for Compute Library's quantized GEMM path.

The product is ``libcugl.so`` (hand-written CUDA behind the C ABI of ``include/cugl.h``) plus the C++
function family in ``computelibrary_b200/host`` that keeps the arm_compute API.  This Python package
only builds the library and binds the C ABI with ctypes so that tests and the benchmark can drive it;
there is no Python or CPU implementation of any operator behind it.
"""
from . import capi  # noqa: F401
from .capi import (CuglError, Context, GemmDesc, GemmPlan, ConvDesc, ConvPlan, U8, S8, S32, STAGE_NONE,
                   STAGE_FIXEDPOINT, load_library)

__all__ = ["capi", "CuglError", "Context", "GemmDesc", "GemmPlan", "ConvDesc", "ConvPlan", "U8", "S8", "S32",
           "STAGE_NONE", "STAGE_FIXEDPOINT", "load_library"]
