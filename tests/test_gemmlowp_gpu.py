"""Parity of the CUDA GEMMLowp path (through the C ABI) with the oracle: bit-exact, tolerance 0."""
import os

import numpy as np
import pytest

from computelibrary_b200 import capi
from helpers import (golden_int_stage, config1, config2, config5, f32_mults, golden_gemm_cases, gpu_gemmlowp, q8_uniform, type_range)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def gemm_golden():
    return np.load(os.path.join(GOLDEN, "gemmlowp_golden.npz"))


@pytest.mark.parametrize("force_simt", [False, True])
def test_golden_cases(ctx, gemm_golden, force_simt):
    """Reference-produced outputs on odd shapes (M=1, N=1, K not a multiple of 16): S32 core, per-tensor and
    per-channel fused output stage, for u8xu8, s8xs8 and u8xs8."""
    for g in golden_gemm_cases():
        acc, _ = gpu_gemmlowp(ctx, g["a"], g["b"], None, g["a_off"], g["b_off"], 0, 0, 0, 0, 0, np.int32,
                              force_simt=force_simt)
        assert np.array_equal(acc, gemm_golden[g["key"] + "_acc"]), g["key"]
        pt, _ = gpu_gemmlowp(ctx, g["a"], g["b"], g["bias"], g["a_off"], g["b_off"], int(g["mult"][0]),
                             int(g["shift"][0]), g["pt_offset"], g["lo"], g["hi"], g["out_dtype"],
                             force_simt=force_simt)
        assert np.array_equal(pt, gemm_golden[g["key"] + "_pt"]), g["key"]
        pc, _ = gpu_gemmlowp(ctx, g["a"], g["b"], g["bias"], g["a_off"], 0, g["mult"], g["shift"], g["pc_offset"],
                             g["lo"], g["hi"], g["out_dtype"], force_simt=force_simt)
        assert np.array_equal(pc, gemm_golden[g["key"] + "_pc"]), g["key"]


def test_config1_fused_and_two_stage(ctx, port, gemm_golden):
    """Configuration 1 of the benchmark against the reference-produced fixture, fused and as core(S32) + output stage."""
    import torch
    c1 = config1()
    qm, sh = capi.calculate_quantized_multiplier(c1["real_multiplier"])
    assert (qm, sh) == (1099511552, 8)
    out, kernel = gpu_gemmlowp(ctx, c1["a"], c1["b"], c1["bias"], c1["a_off"], c1["b_off"], qm, sh, c1["offset"],
                               c1["lo"], c1["hi"], np.uint8)
    assert kernel == "tcgen05"  # 64 rows: one CTA per tile
    assert np.array_equal(out, gemm_golden["c1_out"])
    acc, _ = gpu_gemmlowp(ctx, c1["a"], c1["b"], None, c1["a_off"], c1["b_off"], 0, 0, 0, 0, 0, np.int32)
    assert np.array_equal(acc, gemm_golden["c1_acc"])
    # NEGEMMLowpOutputStage on the S32 result (examples/neon_gemm_qasymm8.cpp:224-239)
    d_acc = torch.from_numpy(acc).cuda()
    d_bias = torch.from_numpy(c1["bias"]).cuda()
    d_out = torch.empty((64, 128), dtype=torch.uint8, device="cuda")
    ctx.output_stage(d_acc, 128 * 4, d_bias, d_out, 128, capi.U8, 64, 128, None, None, qm, sh, 1, c1["offset"],
                     c1["lo"], c1["hi"])
    ctx.sync()
    assert np.array_equal(d_out.cpu().numpy(), gemm_golden["c1_out"])
    # as-given (non-negated) offsets are part of the contract too
    out2, _ = gpu_gemmlowp(ctx, c1["a"], c1["b"], c1["bias"], 128, 120, qm, sh, c1["offset"], 0, 255, np.uint8)
    want2 = port.gemmlowp_fused(c1["a"], c1["b"], c1["bias"], 128, 120, [qm], [sh], c1["offset"], 0, 255, np.uint8)
    assert np.array_equal(out2, want2)


SHAPES = [(128, 256, 128), (129, 257, 130), (64, 64, 16), (300, 520, 1000), (1, 1000, 2048), (257, 64, 576),
          (1000, 96, 147), (512, 128, 4608), (37, 1, 5)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("types", ["u8u8", "s8s8", "u8s8"])
def test_fused_vs_oracle(ctx, port, M, N, K, types):
    ad = np.uint8 if types[:2] == "u8" else np.int8
    bd = np.uint8 if types[2:] == "u8" else np.int8
    rng = np.random.default_rng(M * 131 + N * 17 + K)
    a, b = q8_uniform(rng, (M, K), ad), q8_uniform(rng, (K, N), bd)
    bias = rng.integers(-5000, 5001, N).astype(np.int32)
    lo, hi = type_range(ad)
    # per-tensor, both offsets
    ao, bo = int(rng.integers(-200, 200)), int(rng.integers(-200, 200))
    qm, sh = capi.calculate_quantized_multiplier(np.float32(3.0 / (K * 40.0)))
    want = port.gemmlowp_fused(a, b, bias, ao, bo, [qm], [sh], 7, lo, hi, ad)
    for simt, pair in ((False, True), (False, False), (True, True)):  # SM-pair, one-CTA and generic kernels
        got, kern = gpu_gemmlowp(ctx, a, b, bias, ao, bo, qm, sh, 7, lo, hi, ad, force_simt=simt, ldd_pad=16,
                                 pair=pair)
        assert np.array_equal(got, want), (kern, np.argwhere(got != want)[:5])
    # per-channel (b_offset 0), log-uniform scales as in the benchmark configs
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), N)).astype(np.float32)
    mult, shift = f32_mults(port, 0.02, ws, 0.02 * 0.005 * K * 30)
    got, kern = gpu_gemmlowp(ctx, a, b, bias, ao, 0, mult, shift, -3, lo + 2, hi - 3, ad)
    want = port.gemmlowp_fused(a, b, bias, ao, 0, mult, shift, -3, lo + 2, hi - 3, ad)
    assert np.array_equal(got, want), kern
    # S32 core
    got, _ = gpu_gemmlowp(ctx, a, b, None, ao, bo, 0, 0, 0, 0, 0, np.int32, ldd_pad=4)
    assert np.array_equal(got, port.gemmlowp_core(a, b, ao, bo))


def test_kernel_selection(ctx):
    rng = np.random.default_rng(0)
    a, b = q8_uniform(rng, (64, 48), np.uint8), q8_uniform(rng, (48, 32), np.uint8)
    _, k1 = gpu_gemmlowp(ctx, a, b, None, 0, 0, 2 ** 30, 3, 0, 0, 255, np.uint8)
    assert k1 == "tcgen05"          # K = 48: row stride is a multiple of 16 bytes
    a2, b2 = q8_uniform(rng, (64, 50), np.uint8), q8_uniform(rng, (50, 32), np.uint8)
    got, k2 = gpu_gemmlowp(ctx, a2, b2, None, 0, 0, 2 ** 30, 3, 0, 0, 255, np.uint8)
    # K = 50: TMA cannot address these rows of A, so the plan multiplies a copy of A with a 64-byte row pitch
    assert k2 == "tcgen05"
    _, k3 = gpu_gemmlowp(ctx, a2, b2, None, 0, 0, 2 ** 30, 3, 0, 0, 255, np.uint8, force_simt=True)
    assert k3 == "simt" and np.array_equal(got, _)


def test_negative_shift_and_saturating_multiplier(ctx, port):
    """Left shifts (multiplier >= 1) and the INT32_MIN * INT32_MIN corner of SQDMULH."""
    rng = np.random.default_rng(2)
    M, N, K = 130, 70, 64
    a, b = q8_uniform(rng, (M, K), np.int8), q8_uniform(rng, (K, N), np.int8)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
    shift = rng.integers(-3, 4, N).astype(np.int32)
    mult[5] = -2 ** 31
    bias = rng.integers(-100, 100, N).astype(np.int32)
    for simt in (False, True):
        got, _ = gpu_gemmlowp(ctx, a, b, bias, 3, 0, mult, shift, 1, -128, 127, np.int8, force_simt=simt)
        assert np.array_equal(got, port.gemmlowp_fused(a, b, bias, 3, 0, mult, shift, 1, -128, 127, np.int8))
    qm, sh = capi.calculate_quantized_multiplier(np.float32(2.5))
    assert sh < 0
    got, _ = gpu_gemmlowp(ctx, a, b, None, 0, 0, qm, sh, 0, -128, 127, np.int8)
    assert np.array_equal(got, port.gemmlowp_fused(a, b, None, 0, 0, [qm], [sh], 0, -128, 127, np.int8))


def test_batched(ctx, port):
    """BatchedMatMul (tests/validation/NEON/GEMMLowp.cpp:317-359): batched A with shared and batched B."""
    rng = np.random.default_rng(4)
    a = q8_uniform(rng, (3, 70, 96), np.int8)
    b1 = q8_uniform(rng, (96, 40), np.int8)
    b3 = q8_uniform(rng, (3, 96, 40), np.int8)
    qm, sh = capi.calculate_quantized_multiplier(np.float32(0.0007))
    for b in (b1, b3):
        got, _ = gpu_gemmlowp(ctx, a, b, None, 4, -6, qm, sh, 2, -128, 127, np.int8)
        for i in range(3):
            bi = b if b.ndim == 2 else b[i]
            want = port.gemmlowp_fused(a[i], bi, None, 4, -6, [qm], [sh], 2, -128, 127, np.int8)
            assert np.array_equal(got[i], want)
        acc, _ = gpu_gemmlowp(ctx, a, b, None, 4, -6, 0, 0, 0, 0, 0, np.int32)
        assert np.array_equal(acc, port.gemmlowp_core(a, b, 4, -6))


def test_run_twice_and_variable_b(ctx, port):
    """MultipleExecution (GEMMLowp.cpp:211-297): same plan, same output; B re-laid out per run when it is
    not constant (reshape_b_only_on_first_run = false)."""
    rng = np.random.default_rng(6)
    a, b = q8_uniform(rng, (200, 160), np.uint8), q8_uniform(rng, (160, 300), np.uint8)
    qm, sh = capi.calculate_quantized_multiplier(np.float32(0.0004))
    want = port.gemmlowp_fused(a, b, None, -100, -90, [qm], [sh], 5, 0, 255, np.uint8)
    for const in (True, False):
        got, _ = gpu_gemmlowp(ctx, a, b, None, -100, -90, qm, sh, 5, 0, 255, np.uint8, b_constant=const, runs=3)
        assert np.array_equal(got, want)


def test_update_quantization_parameters(ctx, port):
    import torch
    rng = np.random.default_rng(8)
    M, N, K = 96, 80, 64
    a, b = q8_uniform(rng, (M, K), np.int8), q8_uniform(rng, (K, N), np.int8)
    d1, k1 = capi.make_gemm_desc(M, N, K, capi.S8, capi.S8, capi.S8, 2, 0, multiplier=2 ** 30, shift=6, offset=0,
                                 min_bound=-128, max_bound=127)
    plan = capi.GemmPlan(ctx, d1, k1)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dd = torch.empty((M, N), dtype=torch.int8, device="cuda")
    plan.prepare(db)
    plan.run(da, None, None, dd)
    ctx.sync()
    assert np.array_equal(dd.cpu().numpy(), port.gemmlowp_fused(a, b, None, 2, 0, [2 ** 30], [6], 0, -128, 127, np.int8))
    d2, k2 = capi.make_gemm_desc(M, N, K, capi.S8, capi.S8, capi.S8, -9, 4, multiplier=1518500250, shift=5, offset=-4,
                                 min_bound=-100, max_bound=90)
    plan.update_quantization(d2, k2)
    plan.run(da, None, None, dd)
    ctx.sync()
    assert np.array_equal(dd.cpu().numpy(),
                          port.gemmlowp_fused(a, b, None, -9, 4, [1518500250], [5], -4, -100, 90, np.int8))
    plan.close()


@pytest.mark.parametrize("shape,b_dtype,b_off", [((256, 192, 128), np.int8, 0), ((2600, 320, 192), np.int8, 0),
                                                 ((4099, 136, 80), np.uint8, -7)])
def test_run_host_end_to_end(ctx, port, shape, b_dtype, b_off):
    """The host-buffer entry point: pinned buffers in, pinned buffers out; from 2048 rows on the call pipelines
    row blocks (copy in / multiply / copy out) over three streams, with ragged last blocks and row sums."""
    import ctypes as C
    rng = np.random.default_rng(10)
    M, N, K = shape
    a, b = q8_uniform(rng, (M, K), np.uint8), q8_uniform(rng, (K, N), b_dtype)
    bias = rng.integers(-1000, 1000, N).astype(np.int32)
    import torch
    desc, keep = capi.make_gemm_desc(M, N, K, capi.U8, capi.S8 if b_dtype == np.int8 else capi.U8, capi.U8, -128, b_off,
                                     multiplier=2 ** 30, shift=9, offset=3, min_bound=0, max_bound=255, has_bias=True)
    plan = capi.GemmPlan(ctx, desc, keep)
    plan.prepare(torch.from_numpy(b.view(np.uint8)).cuda())
    h_a, h_d, h_b = ctx.host_alloc(M * K), ctx.host_alloc(M * N), ctx.host_alloc(N * 4)
    C.memmove(h_a, a.ctypes.data, M * K)
    C.memmove(h_b, bias.ctypes.data, N * 4)
    want = port.gemmlowp_fused(a, b, bias, -128, b_off, [2 ** 30], [9], 3, 0, 255, np.uint8)
    for _ in range(2):
        C.memset(h_d, 0xEE, M * N)
        plan.run_host(h_a, h_b, h_d)
        got = np.ctypeslib.as_array((C.c_uint8 * (M * N)).from_address(h_d)).reshape(M, N).copy()
        assert np.array_equal(got, want)
    for p in (h_a, h_d, h_b):
        ctx.host_free(p)
    plan.close()


def test_config2_full_size_properties(ctx, port):
    """4096^3 (configuration 2 of the benchmark): exact on a row sample against the oracle, tensor-core and generic kernels
    agree everywhere, and the result is invariant under a row permutation of A (rows are independent)."""
    c = config2()
    mult, shift = f32_mults(port, c["i_scale"], c["w_scales"], c["o_scale"])
    out, kern = gpu_gemmlowp(ctx, c["a"], c["b"], c["bias"], c["a_off"], 0, mult, shift, 0, -128, 127, np.int8)
    assert kern == "tcgen05_2cta"
    rows = np.r_[0:64, 2000:2064, 4032:4096]
    want = port.gemmlowp_fused(c["a"][rows], c["b"], c["bias"], c["a_off"], 0, mult, shift, 0, -128, 127, np.int8)
    assert np.array_equal(out[rows], want)
    ref2, _ = gpu_gemmlowp(ctx, c["a"], c["b"], c["bias"], c["a_off"], 0, mult, shift, 0, -128, 127, np.int8,
                           force_simt=True)
    assert np.array_equal(out, ref2)
    one_cta, kern1 = gpu_gemmlowp(ctx, c["a"], c["b"], c["bias"], c["a_off"], 0, mult, shift, 0, -128, 127, np.int8,
                                  pair=False)
    assert kern1 == "tcgen05" and np.array_equal(out, one_cta)
    perm = np.random.default_rng(0).permutation(4096)
    outp, _ = gpu_gemmlowp(ctx, c["a"][perm], c["b"], c["bias"], c["a_off"], 0, mult, shift, 0, -128, 127, np.int8)
    assert np.array_equal(outp, out[perm])
    assert 0.05 < np.mean(np.abs(out.astype(np.int32)) == 127 + (out < 0)) < 0.999  # not all saturated


def test_config5_column_shard_property(ctx, port):
    """Config 5 at reduced M: a column shard of B gives exactly the same columns as the full GEMM (what the
    N-sharded multi-GPU run relies on), and a row sample matches the oracle."""
    c = config5(M=512)
    mult, shift = f32_mults(port, c["i_scale"], c["w_scales"], c["o_scale"])
    full, _ = gpu_gemmlowp(ctx, c["a"], c["b"], None, 0, 0, mult, shift, 0, -128, 127, np.int8)
    want = port.gemmlowp_fused(c["a"][:48], c["b"], None, 0, 0, mult, shift, 0, -128, 127, np.int8)
    assert np.array_equal(full[:48], want)
    n0, n1 = 1792 * 3, 1792 * 4
    shard, _ = gpu_gemmlowp(ctx, c["a"], np.ascontiguousarray(c["b"][:, n0:n1]), None, 0, 0, mult[n0:n1],
                            shift[n0:n1], 0, -128, 127, np.int8)
    assert np.array_equal(shard, full[:, n0:n1])


def test_run_multi_destinations(ctx, port):
    """The push all-gather epilogue: one launch writes the same column block into several [M, N_total] matrices
    (here three buffers on one GPU; across GPUs the extra pointers are the peers' buffers)."""
    import torch
    rng = np.random.default_rng(21)
    M, K, n_local, n_total, n0 = 300, 256, 512, 1536, 512
    a, b = q8_uniform(rng, (M, K), np.int8), q8_uniform(rng, (K, n_local), np.int8, -127, 127)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, n_local).astype(np.int32)
    shift = rng.integers(5, 10, n_local).astype(np.int32)
    desc, keep = capi.make_gemm_desc(M, n_local, K, capi.S8, capi.S8, capi.S8, 0, 0, multipliers=mult, shifts=shift,
                                     min_bound=-128, max_bound=127, ldd=n_total)
    plan = capi.GemmPlan(ctx, desc, keep)
    plan.prepare(torch.from_numpy(b.view(np.uint8)).cuda())
    d_a = torch.from_numpy(a.view(np.uint8)).cuda()
    bufs = [torch.full((M, n_total), 0x11, dtype=torch.uint8, device="cuda") for _ in range(3)]
    plan.run_multi(d_a, None, [t.data_ptr() + n0 for t in bufs])
    ctx.sync()
    want = port.gemmlowp_fused(a, b, None, 0, 0, mult, shift, 0, -128, 127, np.int8)
    for t in bufs:
        h = t.cpu().numpy()
        assert np.array_equal(h[:, n0:n0 + n_local].view(np.int8), want)
        assert (h[:, :n0] == 0x11).all() and (h[:, n0 + n_local:] == 0x11).all()
    plan.close()


@pytest.mark.parametrize("epi_warps", [4, 8, 16])
@pytest.mark.parametrize("shape", [(300, 256, 64), (257, 96, 128), (130, 40, 2048), (515, 520, 320), (128, 64, 16)])
def test_epilogue_builds_and_stage_encodings(ctx, port, shape, epi_warps):
    """Both builds of the tensor-core kernels (four / eight epilogue warps) on all three encodings of the output
    stage: shifts >= 2 with non-negative multipliers (one wide multiply-add per element), shifts 0 and 1 (two
    half multiplies), and left shifts / INT32_MIN multipliers (the reference expression as written)."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K + epi_warps)
    a, b = q8_uniform(rng, (M, K), np.uint8), q8_uniform(rng, (K, N), np.int8, -127, 127)
    bias = rng.integers(-20000, 20001, N).astype(np.int32)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
    for lo_shift, hi_shift, label in [(2, 14, "wide"), (0, 6, "fast"), (-2, 5, "generic")]:
        shift = rng.integers(lo_shift, hi_shift, N).astype(np.int32)
        shift[0], shift[-1] = lo_shift, hi_shift - 1
        want = port.gemmlowp_fused(a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8)
        # channel-major: 8-byte aligned rows take the shared-memory byte transpose, a pitch of N + 5 the byte stores
        for pair, cm, pad in ((True, -1, 0), (False, -1, 0), (False, 1, 0), (False, 1, 5), (False, 1, 8)):
            got, kern = gpu_gemmlowp(ctx, a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8, pair=pair,
                                     epi_warps=epi_warps, channel_major=cm, ldd_pad=pad)
            assert kern.startswith("tcgen05")
            assert np.array_equal(got, want), (label, pair, cm, pad, np.argwhere(got != want)[:4])
        # these outputs have fewer tiles than the device has SMs, so the library narrows the tiles by itself; the
        # forced widths cover every tile variant of the build (256 is the only one of the sixteen-warp build)
        for cols in (256, 128, 64):
            got, kern = gpu_gemmlowp(ctx, a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8, epi_warps=epi_warps,
                                     channel_major=-1, tile_columns=cols)
            assert kern.startswith("tcgen05")
            assert np.array_equal(got, want), (label, cols, np.argwhere(got != want)[:4])
    # per-tensor wide encoding with a signed output and a lower bound above the type minimum
    a8 = q8_uniform(rng, (M, K), np.int8)
    got, _ = gpu_gemmlowp(ctx, a8, b, bias, 5, 0, 1759218688, 13, -3, -100, 90, np.int8, epi_warps=epi_warps)
    assert np.array_equal(got, port.gemmlowp_fused(a8, b, bias, 5, 0, [1759218688], [13], -3, -100, 90, np.int8))
    # raw int32 accumulators with the offset terms, row-major and channel-major kernels
    for cm in (-1, 1):
        got, _ = gpu_gemmlowp(ctx, a, b, None, -7, 0, 0, 0, 0, 0, 0, np.int32, epi_warps=epi_warps, channel_major=cm)
        assert np.array_equal(got, port.gemmlowp_core(a, b, -7, 0)), cm
    # asymmetric weights (row-sum term present): never the wide encoding
    bu = q8_uniform(rng, (K, N), np.uint8)
    got, _ = gpu_gemmlowp(ctx, a, bu, bias, -7, -9, 1099511552, 8, 10, 0, 255, np.uint8, epi_warps=epi_warps)
    assert np.array_equal(got, port.gemmlowp_fused(a, bu, bias, -7, -9, [1099511552], [8], 10, 0, 255, np.uint8))


def test_run_multi_destinations_eight_epilogue_warps(ctx, port):
    """The staged multi-destination store of the eight-warp build (64-byte row segments), ragged N and M."""
    import torch
    rng = np.random.default_rng(22)
    M, K, n_local, n_total, n0 = 301, 128, 400, 1200, 400
    a, b = q8_uniform(rng, (M, K), np.int8), q8_uniform(rng, (K, n_local), np.int8, -127, 127)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, n_local).astype(np.int32)
    shift = rng.integers(5, 10, n_local).astype(np.int32)
    want = port.gemmlowp_fused(a, b, None, 0, 0, mult, shift, 0, -128, 127, np.int8)
    for warps in (4, 8, 16):
        desc, keep = capi.make_gemm_desc(M, n_local, K, capi.S8, capi.S8, capi.S8, 0, 0, multipliers=mult, shifts=shift,
                                         min_bound=-128, max_bound=127, ldd=n_total)
        plan = capi.GemmPlan(ctx, desc, keep)
        plan.set_epilogue_warps(warps)
        plan.prepare(torch.from_numpy(b.view(np.uint8)).cuda())
        d_a = torch.from_numpy(a.view(np.uint8)).cuda()
        bufs = [torch.full((M, n_total), 0x11, dtype=torch.uint8, device="cuda") for _ in range(2)]
        plan.run_multi(d_a, None, [t.data_ptr() + n0 for t in bufs])
        ctx.sync()
        for t in bufs:
            h = t.cpu().numpy()
            assert np.array_equal(h[:, n0:n0 + n_local].view(np.int8), want), warps
            assert (h[:, :n0] == 0x11).all() and (h[:, n0 + n_local:] == 0x11).all()
        plan.close()


@pytest.mark.parametrize("shape", [(2304, 2304, 1152), (2290, 2200, 1136), (1024, 5000, 1040)])
def test_pair_kernel_tail_split(ctx, port, shape):
    """SM-pair kernel with a short last wave (81, 81 and 80 tiles of 256 x 256 on 74 SM pairs): the tail tiles run
    as two 256 x 128 halves.  Same bytes as the oracle and as the unsplit kernel, ragged edges included."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    a, b = q8_uniform(rng, (M, K), np.int8), q8_uniform(rng, (K, N), np.int8, -127, 127)
    bias = rng.integers(-20000, 20001, N).astype(np.int32)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
    shift = rng.integers(6, 12, N).astype(np.int32)
    want = port.gemmlowp_fused(a, b, bias, 5, 0, mult, shift, -3, -128, 127, np.int8)
    outs = []
    for split in (True, False):
        import torch
        desc, keep = capi.make_gemm_desc(M, N, K, capi.S8, capi.S8, capi.S8, 5, 0, multipliers=mult, shifts=shift,
                                         offset=-3, min_bound=-128, max_bound=127, has_bias=True)
        plan = capi.GemmPlan(ctx, desc, keep)
        plan.set_tail_split(split)
        assert plan.kernel == "tcgen05_2cta"
        plan.prepare(torch.from_numpy(b.view(np.uint8)).cuda())
        d_dst = torch.full((M, N), 0x55, dtype=torch.uint8, device="cuda")
        plan.run(torch.from_numpy(a.view(np.uint8)).cuda(), None, torch.from_numpy(bias).cuda(), d_dst)
        ctx.sync()
        outs.append(d_dst.cpu().numpy().view(np.int8))
        plan.close()
    assert np.array_equal(outs[0], want), np.argwhere(outs[0] != want)[:5]
    assert np.array_equal(outs[1], want)


@pytest.mark.parametrize("force_simt", [False, True])
def test_fused_quantize_down_stage_golden(ctx, port, gemm_golden, force_simt):
    """NEGEMMLowpMatrixMultiplyCore with a fused QUANTIZE_DOWN (integer multiply) stage against the reference
    fixtures: per-channel and per-tensor, tensor-core (where TMA can address the operands) and generic kernels."""
    for g in golden_gemm_cases():
        im, ish, ioff, ilo, ihi = golden_int_stage(g)
        od = g["out_dtype"]
        got, _ = gpu_gemmlowp(ctx, g["a"], g["b"], g["bias"], g["a_off"], 0, im, ish, ioff, ilo, ihi, od,
                              force_simt=force_simt, integer_stage=True)
        assert np.array_equal(got, gemm_golden[g["key"] + "_int_pc"]), g["key"]
        got, _ = gpu_gemmlowp(ctx, g["a"], g["b"], g["bias"], g["a_off"], g["b_off"], int(im[0]), int(ish[0]), ioff, ilo,
                              ihi, od, force_simt=force_simt, integer_stage=True)
        assert np.array_equal(got, gemm_golden[g["key"] + "_int_pt"]), g["key"]


def test_fused_quantize_down_stage_tensor_core_shapes(ctx, port):
    rng = np.random.default_rng(91)
    for (M, N, K) in [(300, 256, 64), (515, 520, 1088), (130, 40, 2048)]:
        a, b = q8_uniform(rng, (M, K), np.uint8), q8_uniform(rng, (K, N), np.int8, -127, 127)
        bias = rng.integers(-20000, 20001, N).astype(np.int32)
        mult = rng.integers(1, 60, N).astype(np.int32)
        shift = rng.integers(8, 16, N).astype(np.int32)
        want = port.gemmlowp_fused_int(a, b, bias, -9, 0, mult, shift, 4000, 3, 250, np.uint8)
        got, kern = gpu_gemmlowp(ctx, a, b, bias, -9, 0, mult, shift, 4000, 3, 250, np.uint8, integer_stage=True)
        assert kern.startswith("tcgen05") and np.array_equal(got, want), (M, N, K)
        want = port.gemmlowp_fused_int(a, b, None, -9, 0, mult, shift, 4000, 0, 0, np.uint8)   # equal bounds: type range
        got, _ = gpu_gemmlowp(ctx, a, b, None, -9, 0, mult, shift, 4000, 0, 0, np.uint8, integer_stage=True)
        assert np.array_equal(got, want), (M, N, K)


@pytest.mark.parametrize("epi_warps", [4, 8, 16])
@pytest.mark.parametrize("shape", [(38477, 256, 64), (20000, 520, 96), (37900, 300, 496)])
def test_paired_drain(ctx, port, shape, epi_warps):
    """More 128 x 256 tiles than SMs, so a CTA owns several: consecutive tiles of one column block are drained from
    the two accumulator buffers together (one term read for two elements), with single tiles left over where the
    column block changes or the count is odd.  Same bytes as the oracle and as the unpaired epilogue."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K + epi_warps)
    a, b = q8_uniform(rng, (M, K), np.uint8), q8_uniform(rng, (K, N), np.int8, -127, 127)
    bias = rng.integers(-20000, 20001, N).astype(np.int32)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
    shift = rng.integers(2, 12, N).astype(np.int32)
    want = port.gemmlowp_fused(a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8)
    for paired in (True, False):
        got, kern = gpu_gemmlowp(ctx, a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8, pair=False,
                                 epi_warps=epi_warps, channel_major=-1, paired_drain=paired)
        assert kern == "tcgen05"
        assert np.array_equal(got, want), (paired, np.argwhere(got != want)[:4])


# Shapes of tests/datasets/SmallGEMMLowpDataset.h:43-52 and LargeGEMMLowpDataset.h:43-52 as (M, N, K, a_offset, b_offset)
REFERENCE_DATASET_SHAPES = [(13, 33, 21, 0, 0), (13, 33, 52, 0, 4), (27, 23, 31, 18, 23), (72, 17, 32, -9, 1),
                            (1, 33, 21, 0, 0), (13, 1, 21, 5, 13), (973, 221, 1021, 10, 2), (1123, 213, 941, -3, -2),
                            (429, 71, 1021, 1, -1), (1023, 171, 1, 1, 3)]


@pytest.mark.parametrize("M,N,K,ao,bo", REFERENCE_DATASET_SHAPES)
def test_reference_dataset_shapes_run_on_the_tensor_cores(ctx, port, M, N, K, ao, bo):
    """Every shape of the reference's Small / Large GEMMLowp datasets -- K and row pitches that are no multiples of 16
    among them -- runs on the tcgen05 kernel (through a 16-byte-pitch copy of A where needed) and is exact."""
    rng = np.random.default_rng(M * 7 + K)
    a, b = q8_uniform(rng, (M, K), np.uint8), q8_uniform(rng, (K, N), np.uint8)
    got, kern = gpu_gemmlowp(ctx, a, b, None, ao, bo, 0, 0, 0, 0, 0, np.int32)
    assert kern.startswith("tcgen05"), kern
    assert np.array_equal(got, port.gemmlowp_core(a, b, ao, bo))
    bias = rng.integers(-3000, 3001, N).astype(np.int32)
    mult, shift = 1518500250, int(np.ceil(np.log2(max(K, 2) * 255 * 255 / 200)))
    got, kern = gpu_gemmlowp(ctx, a, b, bias, ao, bo, mult, shift, 7, 0, 255, np.uint8, temp_workspace=True)
    assert kern.startswith("tcgen05"), kern
    assert np.array_equal(got, port.gemmlowp_fused(a, b, bias, ao, bo, [mult], [shift], 7, 0, 255, np.uint8))


@pytest.mark.parametrize("M,N,K", [(70, 130, 221), (256, 512, 1040), (300, 64, 96)])
@pytest.mark.parametrize("force_simt", [False, True])
def test_accumulate_and_dequantized_output(ctx, port, M, N, K, force_simt):
    """GEMMInfo::accumulate (dst += A * B, S32) and the s8 x s8 -> F32 rows of the type table: float(int32) * scale with
    one rounding each, identical to the reference's dequantization of the S32 result bit for bit."""
    rng = np.random.default_rng(M + N + K)
    a, b = q8_uniform(rng, (M, K), np.int8), q8_uniform(rng, (K, N), np.int8)
    acc = port.gemmlowp_core(a, b, 3, -4)
    start = rng.integers(-2 ** 20, 2 ** 20, (M, N)).astype(np.int32)
    got, _ = gpu_gemmlowp(ctx, a, b, None, 3, -4, 0, 0, 0, 0, 0, np.int32, accumulate=True, dst_init=start, runs=2,
                          force_simt=force_simt, ldd_pad=4)
    assert np.array_equal(got, start + 2 * acc)
    scale = float(np.float32(1 / 255) * np.float32(5 / 255))
    got, _ = gpu_gemmlowp(ctx, a, b, None, 3, -4, 0, 0, 0, 0, 0, np.float32, dequantize_scale=scale, force_simt=force_simt)
    want = port.dequantize_s32(acc, scale)
    assert got.dtype == np.float32 and np.array_equal(got, want)
    prev = rng.uniform(-100, 100, (M, N)).astype(np.float32)
    got, _ = gpu_gemmlowp(ctx, a, b, None, 3, -4, 0, 0, 0, 0, 0, np.float32, dequantize_scale=scale, accumulate=True,
                          dst_init=prev, force_simt=force_simt)
    assert np.array_equal(got, port.dequantize_s32(acc, scale, prev))


def test_validate_rules_of_the_raw_outputs():
    d, keep = capi.make_gemm_desc(8, 8, 8, capi.S8, capi.S8, capi.F32, stage=capi.STAGE_NONE)
    assert capi.gemm_validate(d)[0] == 6            # an F32 output needs a scale
    d, keep = capi.make_gemm_desc(8, 8, 8, capi.S8, capi.S8, capi.F32, stage=capi.STAGE_NONE, dequantize_scale=0.1)
    assert capi.gemm_validate(d)[0] == 0
    d, keep = capi.make_gemm_desc(8, 8, 8, capi.S8, capi.S8, capi.S8, multiplier=2 ** 30, shift=1, accumulate=True)
    assert capi.gemm_validate(d)[0] == 6            # accumulation only without an output stage


@pytest.mark.parametrize("out_dtype,offset", [(np.uint8, 0), (np.uint8, 7), (np.int8, 0), (np.int8, -11)])
@pytest.mark.parametrize("M,N,K,epi", [(300, 256, 64, 0), (257, 512, 192, 0), (520, 320, 2048, 0), (130, 64, 96, 8), (1000, 256, 512, 1)])
def test_saturating_pack_encoding(ctx, port, out_dtype, offset, M, N, K, epi):
    """Whole-type-range clamps run on the saturating-pack encoding of the output stage (offset folded into the column
    constant, cvt.pack.sat as the clamp): identical to the explicit encoding and to the oracle, for results far
    outside the type range on both sides, shifts up to the limit of the encoding and beyond it."""
    rng = np.random.default_rng(M + N + K + offset)
    a_dt = np.uint8 if out_dtype == np.uint8 else np.int8
    a, b = q8_uniform(rng, (M, K), a_dt), q8_uniform(rng, (K, N), np.int8, -127, 127)
    bias = rng.integers(-400000, 400001, N).astype(np.int32)   # drives many results beyond both ends of the range
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
    lo, hi = type_range(out_dtype)
    for max_shift in (12, 22, 24):
        shift = rng.integers(2, max_shift + 1, N).astype(np.int32)
        shift[0] = max_shift
        want = port.gemmlowp_fused(a, b, bias, 3, 0, mult, shift, offset, lo, hi, out_dtype)
        kw = dict(channel_major=1) if epi == 1 else dict(epi_warps=epi)
        got, _ = gpu_gemmlowp(ctx, a, b, bias, 3, 0, mult, shift, offset, lo, hi, out_dtype, **kw)
        ref, _ = gpu_gemmlowp(ctx, a, b, bias, 3, 0, mult, shift, offset, lo, hi, out_dtype, saturating_pack=False, **kw)
        assert np.array_equal(got, want) and np.array_equal(ref, want), max_shift


@pytest.mark.parametrize("shape", [(300, 200, 64), (300, 208, 64), (700, 520, 64), (1000, 96, 256), (2049, 333, 1536), (40000, 256, 64),
                                   (20000, 64, 128)])
def test_bulk_tensor_stores_against_per_lane_stores(ctx, port, shape):
    """The epilogue's two ways of writing the output -- a warp's rows as one bulk tensor store from shared memory, or
    one store per lane -- on ragged M and N, narrow and wide tiles, short and long K: both against the oracle (a row
    sample for the large cases) and against each other, with a canary pitch that makes the destination rows 16-byte
    aligned (bulk stores possible) or not (the plan must fall back to per-lane stores by itself)."""
    M, N, K = shape
    r = np.random.default_rng(M + N + K)
    a, b = q8_uniform(r, (M, K), np.uint8), q8_uniform(r, (K, N), np.int8, -127, 127)
    bias = r.integers(-4000, 4000, N).astype(np.int32)
    ws = np.exp(r.uniform(np.log(1e-3), np.log(1e-2), N)).astype(np.float32)
    mult, shift = f32_mults(port, 0.05, ws, 0.05 * max(1, K // 64))
    rows = np.unique(np.concatenate([np.arange(0, min(M, 300)), np.arange(max(0, M - 300), M)]))
    want = port.gemmlowp_fused(a[rows], b, bias, -3, 0, mult, shift, 5, 0, 255, np.uint8)
    outs = []
    for tma, pad in ((True, 0), (False, 0), (True, 16 - N % 16 if N % 16 else 16), (True, 3)):
        out, _ = gpu_gemmlowp(ctx, a, b, bias, -3, 0, mult, shift, 5, 0, 255, np.uint8, ldd_pad=pad, tma_store=tma)
        assert np.array_equal(out[rows], want), (tma, pad)
        outs.append(out)
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])


@pytest.mark.parametrize("widths", [(256, 256, 256), (64, 320, 128), (1024, 64, 512)])
def test_chained_launches_with_and_without_dependent_launch(ctx, port, widths):
    """A chain of three GEMMs, each reading what the one before it wrote, launched back to back twenty times over the
    same buffers (so that a kernel also overwrites what its predecessor is still reading unless it waits for it): with
    programmatic stream serialization (the default outside graph capture) and with plain stream order the chain ends
    in the same bytes, equal to the oracle's."""
    import torch
    M, K0 = 3000, 128
    r = np.random.default_rng(sum(widths))
    a = q8_uniform(r, (M, K0), np.uint8)
    dims = (K0,) + widths
    layers, want = [], a
    for k, n in zip(dims[:-1], dims[1:]):
        b = q8_uniform(r, (k, n), np.int8, -127, 127)
        bias = r.integers(-3000, 3000, n).astype(np.int32)
        ws = np.exp(r.uniform(np.log(1e-3), np.log(4e-3), n)).astype(np.float32)
        mult, shift = f32_mults(port, 0.05, ws, 0.05 * max(1, k // 128))
        want = port.gemmlowp_fused(want, b, bias, -2, 0, mult, shift, 4, 0, 255, np.uint8)
        layers.append((k, n, b, bias, mult, shift))
    results = {}
    try:
        for dependent in (True, False):
            ctx.set_dependent_launch(dependent)
            plans, bufs = [], [torch.from_numpy(a).cuda()]
            for k, n, b, bias, mult, shift in layers:
                desc, keep = capi.make_gemm_desc(M, n, k, capi.U8, capi.S8, capi.U8, -2, 0, multipliers=mult, shifts=shift,
                                                 offset=4, min_bound=0, max_bound=255, has_bias=True)
                plan = capi.GemmPlan(ctx, desc, keep)
                plan.prepare(torch.from_numpy(b.view(np.uint8)).cuda())
                plans.append((plan, torch.from_numpy(bias).cuda()))
                bufs.append(torch.zeros((M, n), dtype=torch.uint8, device="cuda"))
            for _ in range(20):
                for i, (plan, d_bias) in enumerate(plans):
                    plan.run(bufs[i], None, d_bias, bufs[i + 1])
            ctx.sync()
            results[dependent] = bufs[-1].cpu().numpy()
            for plan, _ in plans:
                plan.close()
    finally:
        ctx.set_dependent_launch(True)
    assert np.array_equal(results[True], want)
    assert np.array_equal(results[False], want)
