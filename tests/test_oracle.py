"""Pins the CPU restatement (oracle/gemmlowp_oracle.c) to Compute Library's own numbers:
committed golden fixtures produced by the reference's scalar oracle, and -- when the in-place build
oracle/_ref/libacl_ref.so is present -- the reference itself on the reference's dataset shapes."""
import json
import os

import numpy as np
import pytest

from helpers import (GOLDEN_CONV_SCALES, config1, golden_conv_cases, golden_gemm_cases, golden_im2col_cases,
                     golden_int_stage, q8_uniform, type_range)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def gemm_golden():
    return np.load(os.path.join(GOLDEN, "gemmlowp_golden.npz"))


@pytest.fixture(scope="module")
def conv_golden():
    return np.load(os.path.join(GOLDEN, "conv_golden.npz"))


def test_known_answers_scalar(port, known):
    # values that separate the reference's floor-SQDMULH / round-half-up shift from gemmlowp's rounding
    assert port.quantize_down(-3, 2 ** 30, 1, 0, -128, 127) == -1
    assert port.quantize_down(12345, 1099511552, 8, 10, 0, 255) == 35
    assert port.quantize_down(-1000000, 1759218688, 13, 0, -128, 127) == -100
    for *args, want in known["quantize_down"]:
        assert port.quantize_down(*args) == want, args
    for a, b, want in known["sqdmulh"]:
        assert port.sqdmulh(a, b) == want, (a, b)
    for x, e, want in known["rounding_divide_by_pow2"]:
        assert port.rounding_divide_by_pow2(x, e) == want, (x, e)


def test_known_answers_multiplier(port, known):
    assert port.calculate_quantized_multiplier(np.float32(0.02) * np.float32(0.005) / np.float32(0.05)) == (1099511552, 8)
    for m, qm, sh in known["multiplier"]:
        assert port.calculate_quantized_multiplier(np.float32(m)) == (qm, sh), m


def test_config1_golden(port, gemm_golden):
    c1 = config1()
    qm, sh = port.calculate_quantized_multiplier(c1["real_multiplier"])
    assert [qm, sh] == gemm_golden["c1_mult_shift"].tolist()
    acc = port.gemmlowp_core(c1["a"], c1["b"], c1["a_off"], c1["b_off"])
    assert np.array_equal(acc, gemm_golden["c1_acc"])
    out = port.output_stage(acc, c1["bias"], [qm], [sh], c1["offset"], c1["lo"], c1["hi"], np.uint8)
    assert np.array_equal(out, gemm_golden["c1_out"])
    fused = port.gemmlowp_fused(c1["a"], c1["b"], c1["bias"], c1["a_off"], c1["b_off"], [qm], [sh], c1["offset"],
                                c1["lo"], c1["hi"], np.uint8)
    assert np.array_equal(fused, gemm_golden["c1_out"])


def test_gemmlowp_golden(port, gemm_golden):
    for g in golden_gemm_cases():
        acc = port.gemmlowp_core(g["a"], g["b"], g["a_off"], g["b_off"])
        assert np.array_equal(acc, gemm_golden[g["key"] + "_acc"]), g["key"]
        # the decomposition the library (and the CUDA epilogue) uses equals the direct definition
        raw = port.gemmlowp_core(g["a"], g["b"], 0, 0)
        dec = port.offset_contribution(raw, g["a"].shape[1], port.reduce_cols(g["b"]), port.reduce_rows(g["a"]),
                                       g["a_off"], g["b_off"])
        assert np.array_equal(dec, acc), g["key"]
        pt = port.gemmlowp_fused(g["a"], g["b"], g["bias"], g["a_off"], g["b_off"], g["mult"][:1], g["shift"][:1],
                                 g["pt_offset"], g["lo"], g["hi"], g["out_dtype"])
        assert np.array_equal(pt, gemm_golden[g["key"] + "_pt"]), g["key"]
        pc = port.gemmlowp_fused(g["a"], g["b"], g["bias"], g["a_off"], 0, g["mult"], g["shift"], g["pc_offset"],
                                 g["lo"], g["hi"], g["out_dtype"])
        assert np.array_equal(pc, gemm_golden[g["key"] + "_pc"]), g["key"]


def test_conv_golden(port, conv_golden):
    i_scale, o_scale = GOLDEN_CONV_SCALES
    for c in golden_conv_cases():
        mult, shift = port.calculate_quantized_multipliers(i_scale, c["w_scales"], o_scale)
        lo, hi = type_range(c["src"].dtype)
        out = port.conv2d_nhwc(c["src"], c["weights"], c["bias"], c["stride"], c["pad"], c["in_zp"], c["w_zp"], mult,
                               shift, c["out_zp"], lo, hi)
        assert np.array_equal(out, conv_golden[c["key"] + "_out"]), c["key"]


def test_im2col_golden(port, conv_golden):
    for c in golden_im2col_cases():
        cols = port.im2col_nhwc(c["src"], c["kw"], c["kh"], *c["stride"], *c["pad"], c["zp"])
        assert np.array_equal(cols, conv_golden[c["key"]]), c["key"]
        padded = port.im2col_nhwc(c["src"], c["kw"], c["kh"], *c["stride"], *c["pad"], c["zp"],
                                  row_stride=cols.shape[2] + 11)
        assert np.array_equal(padded[:, :, :cols.shape[2]], cols) and not padded[:, :, cols.shape[2]:].any()


# ---- direct comparison with the reference's oracle on the reference's dataset shapes ---------------------
# tests/datasets/SmallGEMMLowpDataset.h:43-52 and LargeGEMMLowpDataset.h:43-52 (M, N, K and offsets)
SMALL = [(21, 13, 33, 0, 0), (52, 13, 33, 0, 4), (31, 27, 23, 18, 23), (32, 72, 4, 13, -20), (21, 1, 1, -20, 13)]
LARGE = [(923, 429, 871, 0, 0), (873, 513, 784, 0, 4), (1021, 973, 221, 5, 13), (1021, 1, 73, -3, -2),
         (941, 1011, 1, -9, 1)]


@pytest.mark.parametrize("M,N,K,ao,bo", SMALL + LARGE)
def test_port_vs_reference_core(port, ref, M, N, K, ao, bo):
    for ad, bd in [(np.uint8, np.uint8), (np.int8, np.int8), (np.uint8, np.int8)]:
        rng = np.random.default_rng(M * 31 + N * 7 + K)
        a, b = q8_uniform(rng, (M, K), ad), q8_uniform(rng, (K, N), bd)
        assert np.array_equal(port.gemmlowp_core(a, b, ao, bo), ref.gemmlowp_core(a, b, ao, bo))


def test_port_vs_reference_batched(port, ref):
    rng = np.random.default_rng(5)
    a, b = q8_uniform(rng, (3, 17, 29), np.int8), q8_uniform(rng, (3, 29, 11), np.int8)
    assert np.array_equal(port.gemmlowp_core(a, b, 3, -7), ref.gemmlowp_core(a, b, 3, -7))
    assert np.array_equal(port.gemmlowp_core(a, b[0], 3, -7), ref.gemmlowp_core(a, b[0], 3, -7))


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("out_dtype", [np.uint8, np.int8])
def test_port_vs_reference_output_stage(port, ref, per_channel, out_dtype):
    rng = np.random.default_rng(11)
    M, N = 37, 53
    acc = rng.integers(-6000, 6001, (M, N)).astype(np.int32)  # fixture range, GEMMLowpFixture.h:1010-1015
    acc[0, :8] = [2 ** 31 - 1, -2 ** 31, 0, -1, 1, 2 ** 30, -2 ** 30, 12345]
    bias = rng.integers(-2000, 2001, N).astype(np.int32)
    n = N if per_channel else 1
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, n).astype(np.int32)
    shift = rng.integers(-2, 12, n).astype(np.int32)
    lo, hi = type_range(out_dtype)
    for bounds in [(lo, hi), (lo + 7, hi - 9), (-2 ** 31, 2 ** 31 - 1)]:
        for b in (None, bias):
            got = port.output_stage(acc, b, mult, shift, 5, bounds[0], bounds[1], out_dtype)
            want = ref.output_stage(acc, b, mult, shift, 5, bounds[0], bounds[1], out_dtype)
            assert np.array_equal(got, want)


def test_port_vs_reference_multiplier(port, ref):
    rng = np.random.default_rng(3)
    for _ in range(2000):
        m = np.float32(np.exp(rng.uniform(np.log(1e-8), np.log(500.0))))
        assert port.calculate_quantized_multiplier(m) == ref.calculate_quantized_multiplier(float(m))


def test_integer_stage_golden(port, gemm_golden):
    """QUANTIZE_DOWN (integer multiply) stage of the restatement against fixtures made by the reference's
    gemmlowp_quantize_down_scale: per-tensor, per-channel, and equal bounds (= no bounded ReLU)."""
    n = 0
    for g in golden_gemm_cases():
        im, ish, ioff, ilo, ihi = golden_int_stage(g)
        acc = port.gemmlowp_core(g["a"], g["b"], g["a_off"], g["b_off"])
        acc0 = port.gemmlowp_core(g["a"], g["b"], g["a_off"], 0)
        od = g["out_dtype"]
        assert np.array_equal(port.output_stage_int(acc, g["bias"], im[:1], ish[:1], ioff, ilo, ihi, od), gemm_golden[g["key"] + "_int_pt"])
        assert np.array_equal(port.output_stage_int(acc0, g["bias"], im, ish, ioff, ilo, ihi, od), gemm_golden[g["key"] + "_int_pc"])
        assert np.array_equal(port.output_stage_int(acc0, None, im, ish, ioff, 0, 0, od), gemm_golden[g["key"] + "_int_nb"])
        assert np.array_equal(port.gemmlowp_fused_int(g["a"], g["b"], g["bias"], g["a_off"], 0, im, ish, ioff, ilo, ihi, od),
                              gemm_golden[g["key"] + "_int_pc"])
        n += 1
    assert n == 24


def test_qsymm16_stage_golden_and_reference(port, ref, gemm_golden):
    """Fixed-point output stage with a QSYMM16 destination: the restatement against fixtures made by the int16_t
    instantiation of the reference's gemmlowp_quantize_down_scale_by_fixedpoint, and against that code directly on
    random accumulators (left shifts, INT32 extremes, equal bounds)."""
    for g in golden_gemm_cases():
        acc = port.gemmlowp_core(g["a"], g["b"], g["a_off"], g["b_off"])
        acc0 = port.gemmlowp_core(g["a"], g["b"], g["a_off"], 0)
        assert np.array_equal(port.output_stage(acc, g["bias"], g["mult"][:1], g["shift"][:1] - 6, 0, -20000, 25000, np.int16),
                              gemm_golden[g["key"] + "_s16_pt"])
        assert np.array_equal(port.output_stage(acc0, None, g["mult"], g["shift"] - 6, 0, -32768, 32767, np.int16),
                              gemm_golden[g["key"] + "_s16_pc"])
    if ref is None:
        return
    rng = np.random.default_rng(5)
    acc = rng.integers(-2 ** 24, 2 ** 24, (37, 53)).astype(np.int32)
    acc.flat[:2] = [2 ** 31 - 1, -2 ** 31]
    bias = rng.integers(-10000, 10000, 53).astype(np.int32)
    for nm in (1, 53):
        mult = rng.integers(2 ** 30, 2 ** 31 - 1, nm).astype(np.int32)
        shift = rng.integers(-1, 12, nm).astype(np.int32)
        for lo, hi in ((-32768, 32767), (-1000, 2000), (0, 0)):
            for b in (None, bias):
                assert np.array_equal(port.output_stage(acc, b, mult, shift, 0, lo, hi, np.int16),
                                      ref.output_stage(acc, b, mult, shift, 0, lo, hi, np.int16)), (nm, lo, hi)


@pytest.mark.parametrize("out_dtype", [np.uint8, np.int8])
def test_port_vs_reference_integer_stage(port, ref, out_dtype):
    rng = np.random.default_rng(77)
    for (M, N) in [(1, 1), (9, 31), (40, 64)]:
        acc = rng.integers(-2 ** 22, 2 ** 22, (M, N)).astype(np.int32)
        acc.flat[0] = 2 ** 31 - 1
        bias = rng.integers(-9000, 9000, N).astype(np.int32)
        for nm in (1, N):
            mult = rng.integers(-50, 500, nm).astype(np.int32)
            shift = rng.integers(0, 24, nm).astype(np.int32)
            for lo, hi in [(0, 0), (5, 100), (-2 ** 31, 2 ** 31 - 1)]:
                for b in (None, bias):
                    assert np.array_equal(port.output_stage_int(acc, b, mult, shift, -321, lo, hi, out_dtype),
                                          ref.output_stage_int(acc, b, mult, shift, -321, lo, hi, out_dtype))


def test_port_vs_reference_dequantized_output(port, ref):
    """The dequantised (F32) GEMMLowp output and its accumulating form against reference::dequantization_layer /
    reference::arithmetic_operation compiled in place."""
    rng = np.random.default_rng(77)
    acc = rng.integers(-2 ** 31, 2 ** 31, 50000, dtype=np.int64).astype(np.int32)
    prev = rng.uniform(-2e4, 2e4, acc.size).astype(np.float32)
    for scale in (np.float32(1 / 255) * np.float32(5 / 255), np.float32(0.37), np.float32(3e-7)):
        assert np.array_equal(ref.dequantize_s32(acc, scale), port.dequantize_s32(acc, scale))
        assert np.array_equal(ref.dequantize_s32(acc, scale, prev), port.dequantize_s32(acc, scale, prev))
