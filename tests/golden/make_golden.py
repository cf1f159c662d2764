"""Generates the committed golden fixtures of tests/golden/ from Compute Library's OWN scalar test oracle
(tests/validation/reference/{GEMMLowp,ConvolutionLayer,Im2Col,PoolingLayer,ArithmeticOperations,ActivationLayer,
SoftmaxLayer}.cpp, UtilsQuantizedAsymm.h and AsymmHelpers.cpp), compiled in place into oracle/_ref/libacl_ref.so by `make -C oracle ref`.

    python tests/golden/make_golden.py        # needs the Compute Library tree; rewrites the fixtures

The fixtures let the CPU-side restatement (oracle/gemmlowp_oracle.c, oracle/layers_oracle.c) and the CUDA path be checked against
reference outputs on machines where the reference tree is absent.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from helpers import (GOLDEN_CONV_SCALES, config1, golden_act_cases, golden_add_cases,  # noqa: E402
                     golden_conv_cases, golden_gemm_cases, golden_im2col_cases, golden_int_stage, golden_pool_cases,
                     golden_softmax_cases, pool_with)


def main():
    ref = oracle.ref()
    assert ref is not None, "build oracle/_ref first: make -C oracle ref"
    rng = np.random.default_rng(20240607)

    # --- scalar known answers -------------------------------------------------------------------
    ka = {"quantize_down": [], "sqdmulh": [], "rounding_divide_by_pow2": [], "multiplier": []}
    cases = [(-3, 2 ** 30, 0, 0, -128, 127), (-3, 2 ** 30, 1, 0, -128, 127), (3, 2 ** 30, 1, 0, -128, 127),
             (12345, 1099511552, 8, 10, 0, 255), (-12345, 1099511552, 8, 10, 0, 255),
             (63999, 1099511552, 8, 10, 0, 255), (64000, 1099511552, 8, 10, 0, 255), (-1, 1099511552, 8, 10, 0, 255),
             (1000000, 1759218688, 13, 0, -128, 127), (-1000000, 1759218688, 13, 0, -128, 127),
             (4999, 1759218688, 13, 0, -128, 127), (-4999, 1759218688, 13, 0, -128, 127),
             (7, 2 ** 30, -2, 0, -128, 127), (-7, 2 ** 30, -2, 0, -128, 127),
             (2 ** 31 - 1, 2 ** 31 - 1, 0, 0, -128, 127), (-2 ** 31, 2 ** 31 - 1, 0, 0, -128, 127)]
    for _ in range(200):
        cases.append((int(rng.integers(-2 ** 24, 2 ** 24)), int(rng.integers(2 ** 30, 2 ** 31 - 1)),
                      int(rng.integers(-3, 16)), int(rng.integers(-128, 128)), -128, 127))
    for c in cases:
        ka["quantize_down"].append([*c, ref.quantize_down(*c)])
    pairs = [(-2 ** 31, -2 ** 31), (-2 ** 31, 2 ** 31 - 1), (2 ** 31 - 1, 2 ** 31 - 1), (-1, 1), (1, -1), (0, 5)]
    pairs += [(int(rng.integers(-2 ** 31, 2 ** 31)), int(rng.integers(-2 ** 31, 2 ** 31))) for _ in range(200)]
    for a, b in pairs:
        ka["sqdmulh"].append([a, b, ref.sqdmulh(a, b)])
    for _ in range(200):
        x, e = int(rng.integers(-2 ** 30, 2 ** 30)), int(rng.integers(0, 31))
        ka["rounding_divide_by_pow2"].append([x, e, ref.rounding_divide_by_pow2(x, e)])
    mults = [np.float32(0.02) * np.float32(0.005) / np.float32(0.05), np.float32(0.01) * np.float32(0.001) / np.float32(0.1),
             np.float32(0.01) * np.float32(0.01) / np.float32(0.1), 0.5, 0.25, 0.99999994, 1.0, 1.5, 2.0, 37.25, 1e-6]
    mults += [float(np.float32(np.exp(rng.uniform(np.log(1e-7), np.log(200.0))))) for _ in range(100)]
    for m in mults:
        qm, sh = ref.calculate_quantized_multiplier(float(np.float32(m)))
        ka["multiplier"].append([float(np.float32(m)), qm, sh])
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(ka, f)

    # --- GEMMLowp: config 1 and odd shapes (inputs are regenerated from the seed, outputs stored) --
    out = {}
    c1 = config1()
    acc = ref.gemmlowp_core(c1["a"], c1["b"], c1["a_off"], c1["b_off"])
    qm, sh = ref.calculate_quantized_multiplier(float(c1["real_multiplier"]))
    out["c1_acc"] = acc
    out["c1_mult_shift"] = np.array([qm, sh], np.int32)
    out["c1_out"] = ref.output_stage(acc, c1["bias"], [qm], [sh], c1["offset"], c1["lo"], c1["hi"], np.uint8)
    for g in golden_gemm_cases():
        acc = ref.gemmlowp_core(g["a"], g["b"], g["a_off"], g["b_off"])
        out[g["key"] + "_acc"] = acc
        out[g["key"] + "_pt"] = ref.output_stage(acc, g["bias"], g["mult"][:1], g["shift"][:1], g["pt_offset"],
                                                 g["lo"], g["hi"], g["out_dtype"])
        # per-channel requantisation is only defined for b_offset == 0 on signed outputs: use 0 throughout
        acc0 = ref.gemmlowp_core(g["a"], g["b"], g["a_off"], 0)
        out[g["key"] + "_pc"] = ref.output_stage(acc0, g["bias"], g["mult"], g["shift"], g["pc_offset"], g["lo"],
                                                 g["hi"], g["out_dtype"])
        # QUANTIZE_DOWN (integer multiply) stage: per-tensor on the full accumulators, per-channel on acc0, and
        # the "equal bounds = no bounded ReLU" rule
        im, ish, ioff, ilo, ihi = golden_int_stage(g)
        out[g["key"] + "_int_pt"] = ref.output_stage_int(acc, g["bias"], im[:1], ish[:1], ioff, ilo, ihi, g["out_dtype"])
        out[g["key"] + "_int_pc"] = ref.output_stage_int(acc0, g["bias"], im, ish, ioff, ilo, ihi, g["out_dtype"])
        out[g["key"] + "_int_nb"] = ref.output_stage_int(acc0, None, im, ish, ioff, 0, 0, g["out_dtype"])
        # QSYMM16 destination of the fixed-point stage: per-tensor with bounds, per-channel over the whole int16 range
        out[g["key"] + "_s16_pt"] = ref.output_stage(acc, g["bias"], g["mult"][:1], g["shift"][:1] - 6, 0, -20000, 25000,
                                                     np.int16)
        out[g["key"] + "_s16_pc"] = ref.output_stage(acc0, None, g["mult"], g["shift"] - 6, 0, -32768, 32767, np.int16)
    np.savez_compressed(os.path.join(HERE, "gemmlowp_golden.npz"), **out)

    # --- convolution (NCHW oracle; stored NHWC) and im2col -----------------------------------------
    conv = {}
    i_scale, o_scale = GOLDEN_CONV_SCALES
    for c in golden_conv_cases():
        o = ref.conv_nchw(c["src"].transpose(0, 3, 1, 2), c["weights"].transpose(0, 3, 1, 2), c["bias"], c["stride"],
                          c["pad"], i_scale, c["in_zp"], c["w_scales"], c["w_zp"], o_scale, c["out_zp"])
        conv[c["key"] + "_out"] = np.ascontiguousarray(o.transpose(0, 2, 3, 1))
    for c in golden_im2col_cases():
        conv[c["key"]] = ref.im2col_nhwc(c["src"], c["kw"], c["kh"], *c["stride"], *c["pad"], c["zp"])
    np.savez_compressed(os.path.join(HERE, "conv_golden.npz"), **conv)

    # --- QASYMM8 layers: pooling, addition, activation, softmax ------------------------------------
    layers = {}
    for c in golden_pool_cases():
        layers[c["key"]] = pool_with(ref, c)
    for c in golden_add_cases():
        layers[c["key"]] = ref.add_qasymm8(c["a"], c["b"], *c["q"])
    for c in golden_act_cases():
        layers[c["key"]] = ref.activation_qasymm8(c["src"], c["act"], c["a"], c["b"], c["in_q"], c["out_q"])
    for c in golden_softmax_cases():
        layers[c["key"]] = ref.softmax_qasymm8(c["src"], c["beta"], c["q"])
    np.savez_compressed(os.path.join(HERE, "layers_golden.npz"), **layers)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
