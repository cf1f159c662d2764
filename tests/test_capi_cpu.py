"""Host-only checks of the C-ABI library: it loads, exports every symbol include/cugl.h declares, refuses to
work without a GPU, and its validate() / multiplier helpers follow the reference rules."""
import ctypes as C
import os

import numpy as np
import pytest

import computelibrary_b200 as cl
from computelibrary_b200 import capi


def test_library_exports_every_declared_symbol():
    lib = cl.load_library()
    declared = capi.header_symbols()
    assert len(declared) >= 40
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/cugl.h but not exported"
    assert set(declared) == set(capi._SIGNATURES), "ctypes binding out of sync with the header"


def test_struct_layout_matches_header():
    # natural C layout: 4 x i32, 6 x i64, 9 x i32 (+pad), 2 x ptr, 6 x i32 + 1 x f32 (+pad)
    assert C.sizeof(capi.GemmDesc) == 16 + 48 + 40 + 16 + 32
    assert capi.GemmDesc.dequantize_scale.offset == 16 + 48 + 40 + 16 + 24
    assert capi.GemmDesc.h_gemmlowp_multipliers.offset == 104
    assert capi.ConvDesc.h_gemmlowp_multipliers.offset == 88


def test_no_cpu_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(cl.CuglError) as e:
        cl.Context(0)
    assert e.value.status == 4 and "no CPU fallback" in e.value.message


def test_multiplier_helper_matches_oracle(port):
    rng = np.random.default_rng(9)
    assert capi.calculate_quantized_multiplier(np.float32(0.02) * np.float32(0.005) / np.float32(0.05)) == (1099511552, 8)
    for _ in range(2000):
        m = np.float32(np.exp(rng.uniform(np.log(1e-8), np.log(500.0))))
        assert capi.calculate_quantized_multiplier(m) == port.calculate_quantized_multiplier(m)
    ws = rng.uniform(1e-3, 1e-2, 300).astype(np.float32)
    m1, s1 = capi.calculate_quantized_multipliers(np.float32(0.01), ws, np.float32(0.1))
    m2, s2 = port.calculate_quantized_multipliers(np.float32(0.01), ws, np.float32(0.1))
    assert np.array_equal(m1, m2) and np.array_equal(s1, s2)
    with pytest.raises(cl.CuglError):
        capi.calculate_quantized_multiplier(-0.5)


def _desc(**kw):
    base = dict(M=8, N=8, K=8, a_dtype=cl.U8, b_dtype=cl.U8, dst_dtype=cl.U8, multiplier=2 ** 30, shift=1,
                min_bound=0, max_bound=255)
    base.update(kw)
    d, keep = capi.make_gemm_desc(**base)
    d._keep = keep
    return d


def test_gemm_validate_rules():
    # the rejection table of tests/validation/NEON/GEMMLowp.cpp:168-200 restated for the C descriptor
    assert capi.gemm_validate(_desc())[0] == 0
    assert capi.gemm_validate(_desc(dst_dtype=cl.S32, stage=cl.STAGE_NONE))[0] == 0
    st, why = capi.gemm_validate(_desc(dst_dtype=cl.S32, stage=cl.STAGE_NONE, has_bias=True))
    assert st == 6 and "Bias addition not supported" in why
    assert capi.gemm_validate(_desc(dst_dtype=cl.S32))[0] == 6                      # stage needs 8-bit dst
    assert capi.gemm_validate(_desc(stage=cl.STAGE_NONE))[0] == 6                   # NONE needs S32 dst
    assert capi.gemm_validate(_desc(stage=1))[0] == 0                               # QUANTIZE_DOWN (integer multiply)
    assert capi.gemm_validate(_desc(stage=3))[0] == 8                               # QUANTIZE_DOWN_FLOAT: unsupported
    assert capi.gemm_validate(_desc(min_bound=10, max_bound=5))[0] == 6
    assert capi.gemm_validate(_desc(K=0))[0] == 6
    assert capi.gemm_validate(_desc(a_dtype=cl.S32))[0] == 6
    assert capi.gemm_validate(_desc(lda=4))[0] == 6
    m = np.full(8, 2 ** 30, np.int32)
    s = np.ones(8, np.int32)
    ok = _desc(a_dtype=cl.S8, b_dtype=cl.S8, dst_dtype=cl.S8, multipliers=m, shifts=s, min_bound=-128, max_bound=127)
    assert capi.gemm_validate(ok)[0] == 0
    bad = _desc(a_dtype=cl.S8, b_dtype=cl.S8, dst_dtype=cl.S8, multipliers=m, shifts=s, b_offset=3, min_bound=-128,
                max_bound=127)
    assert capi.gemm_validate(bad)[0] == 6  # CpuGemmLowpOffsetContributionOutputStageKernel.cpp:832-836
    assert capi.gemm_validate(_desc(multipliers=m, shifts=s, b_offset=3))[0] == 0   # allowed for QASYMM8 dst


def test_conv_validate_rules():
    d, _ = capi.make_conv_desc(2, 8, 8, 16, 4, 3, 3, pad=(1, 1, 1, 1), multiplier=2 ** 30, shift=2, min_bound=0,
                               max_bound=255)
    assert capi.conv_validate(d)[0] == 0
    wo, ho = C.c_int32(), C.c_int32()
    cl.load_library().cugl_conv2d_out_dims(C.byref(d), C.byref(wo), C.byref(ho))
    assert (wo.value, ho.value) == (8, 8)
    d2, _ = capi.make_conv_desc(2, 2, 2, 16, 4, 5, 5, multiplier=2 ** 30, shift=2)
    assert capi.conv_validate(d2)[0] == 6                                         # kernel larger than input
    d3, _ = capi.make_conv_desc(2, 8, 8, 16, 4, 3, 3, src_dtype=cl.S8, w_dtype=cl.U8, multiplier=1, shift=0)
    assert capi.conv_validate(d3)[0] == 6


def test_product_does_not_touch_the_oracle():
    # the shipped package must never import, link or execute anything under oracle/
    pkg = os.path.dirname(capi.__file__)
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".hpp")):
                text = open(os.path.join(root, f), errors="ignore").read()
                assert "import oracle" not in text and "gemmlowp_oracle" not in text and "libacl_ref" not in text, f
