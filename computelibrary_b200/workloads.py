"""Seeded synthetic stand-ins for the benchmark configurations (shapes, value ranges and quantisation
parameters of the five reference workloads).  No dataset or trained weights are involved: every tensor is
drawn from numpy's default_rng(seed)."""
from __future__ import annotations

import numpy as np


def q8_uniform(rng, shape, dtype, lo=None, hi=None):
    info = np.iinfo(dtype)
    lo = info.min if lo is None else lo
    hi = info.max if hi is None else hi
    return rng.integers(lo, hi + 1, size=shape, dtype=np.int64).astype(dtype)


def type_range(dtype):
    info = np.iinfo(dtype)
    return int(info.min), int(info.max)


# ---- the five benchmark configurations (seeded stand-ins; shapes / distributions of the benchmark specification) ----
def config1(seed=1):
    """examples/neon_gemm_qasymm8-style: u8 [64,256] x u8 [256,128], bias, fixed-point stage to u8."""
    rng = np.random.default_rng(seed)
    M, N, K = 64, 128, 256
    a = q8_uniform(rng, (M, K), np.uint8)
    b = q8_uniform(rng, (K, N), np.uint8)
    bias = rng.integers(-2000, 2001, N).astype(np.int32)
    real = np.float32(0.02) * np.float32(0.005) / np.float32(0.05)
    return dict(a=a, b=b, bias=bias, a_off=-128, b_off=-120, real_multiplier=real, offset=10, lo=0, hi=255,
                out_dtype=np.uint8)


def config2(seed=1, M=4096, N=4096, K=4096):
    """Square s8 GEMMLowp with per-channel weights: A zp -5 (passed negated: +5), out scale 0.1 zp 0."""
    rng = np.random.default_rng(seed)
    a = q8_uniform(rng, (M, K), np.int8)
    b = q8_uniform(rng, (K, N), np.int8, -127, 127)
    w_scales = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), N)).astype(np.float32)
    bias = rng.integers(-10000, 10001, N).astype(np.int32)
    return dict(a=a, b=b, bias=bias, a_off=5, b_off=0, i_scale=np.float32(0.01), w_scales=w_scales,
                o_scale=np.float32(0.1), offset=0, lo=-128, hi=127, out_dtype=np.int8)


def config3(seed=1, B=32, H=56, W=56, C=64, OFM=64):
    """3x3 stride-1 pad-1 NHWC conv: u8 input zp 128, per-channel s8 weights, fused ReLU to u8 (zp 0)."""
    rng = np.random.default_rng(seed)
    src = q8_uniform(rng, (B, H, W, C), np.uint8)
    wgt = q8_uniform(rng, (OFM, 3, 3, C), np.int8, -127, 127)
    w_scales = rng.uniform(2e-3, 8e-3, OFM).astype(np.float32)
    bias = rng.integers(-5000, 5001, OFM).astype(np.int32)
    return dict(src=src, weights=wgt, bias=bias, stride=(1, 1), pad=(1, 1, 1, 1), in_zp=128, w_zp=0,
                i_scale=np.float32(0.03), w_scales=w_scales, o_scale=np.float32(0.05), out_zp=0, lo=0, hi=255)


def config5(seed=1, M=8192, K=4096, N=14336):
    """LLM-style linear: clipped-Gaussian s8 activations, per-channel s8 weights, no bias, s8 out."""
    rng = np.random.default_rng(seed)
    a = np.clip(np.rint(rng.normal(0.0, 30.0, (M, K))), -128, 127).astype(np.int8)
    b = q8_uniform(rng, (K, N), np.int8, -127, 127)
    w_scales = rng.uniform(1e-3, 5e-3, N).astype(np.float32)
    return dict(a=a, b=b, bias=None, a_off=0, b_off=0, i_scale=np.float32(0.02), w_scales=w_scales,
                o_scale=np.float32(0.05), offset=0, lo=-128, hi=127, out_dtype=np.int8)
