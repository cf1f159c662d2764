"""NEGEMMConvolutionLayer on the GPU (im2col + fused GEMMLowp through the C ABI) against the reference-made
golden fixtures and the oracle: tolerance 0, as tests/validation/NEON/ConvolutionLayer.cpp:102-103."""
import os

import numpy as np
import pytest

from computelibrary_b200 import capi
from helpers import GOLDEN_CONV_SCALES, config3, f32_mults, golden_conv_cases, q8_uniform, type_range

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CODE = {np.dtype(np.uint8): capi.U8, np.dtype(np.int8): capi.S8}


def gpu_conv(ctx, src, weights, bias, stride, pad, in_zp, w_zp, mult, shift, out_zp, lo, hi, dilation=(1, 1),
             implicit=True, want_kernel=None, tile_columns=0, paired_drain=True, tma_im2col=True, want_tma=None,
             resident_weights=True, double_tile=True):
    import torch
    B, H, W, Cc = src.shape
    OFM, kh, kw, _ = weights.shape
    pc = np.ndim(mult) > 0 and len(mult) > 1
    desc, keep = capi.make_conv_desc(B, H, W, Cc, OFM, kh, kw, stride, pad, dilation, CODE[src.dtype],
                                     CODE[weights.dtype], in_zp, w_zp,
                                     multiplier=0 if pc else int(np.ravel(mult)[0]),
                                     shift=0 if pc else int(np.ravel(shift)[0]),
                                     multipliers=mult if pc else None, shifts=shift if pc else None, dst_zp=out_zp,
                                     min_bound=lo, max_bound=hi, has_bias=bias is not None)
    plan = capi.ConvPlan(ctx, desc, keep)
    if not implicit:
        plan.allow_implicit(False)
    if tile_columns:
        plan.set_tile_columns(tile_columns)
    if not paired_drain:
        plan.set_paired_drain(False)
    if tma_im2col is not True:
        plan.allow_tma_im2col(int(tma_im2col))  # 0: the gather; 2: TMA loads for 64-channel inputs too
    if not resident_weights:
        plan.set_resident_weights(False)
    if not double_tile:
        plan.set_double_tile(False)
    if want_tma is not None:
        assert plan.uses_tma_im2col == want_tma
    if want_kernel is not None:
        assert plan.kernel == want_kernel, plan.kernel
    wo, ho = plan.out_dims()
    d_src = torch.from_numpy(src.view(np.uint8)).cuda()
    d_w = torch.from_numpy(weights.view(np.uint8)).cuda()
    d_b = torch.from_numpy(bias).cuda() if bias is not None else None
    # guard regions of canary bytes on both sides of the destination: a store outside the tensor shows up
    guard, n_out = 4096, B * ho * wo * OFM
    whole = torch.full((guard + n_out + guard,), 0xA5, dtype=torch.uint8, device="cuda")
    d_dst = whole[guard:guard + n_out].view(B, ho, wo, OFM)
    plan.prepare(d_w)
    del d_w  # weights may be released after prepare()
    plan.run(d_src, d_b, d_dst)
    plan.run(d_src, d_b, d_dst)
    ctx.sync()
    everything = whole.cpu().numpy()
    plan.close()
    assert (everything[:guard] == 0xA5).all() and (everything[-guard:] == 0xA5).all(), \
        "kernel wrote outside the destination tensor"
    return np.ascontiguousarray(everything[guard:-guard]).view(src.dtype).reshape(B, ho, wo, OFM)


def test_conv_golden(ctx, port):
    gold = np.load(os.path.join(GOLDEN, "conv_golden.npz"))
    i_scale, o_scale = GOLDEN_CONV_SCALES
    for c in golden_conv_cases():
        mult, shift = f32_mults(port, i_scale, c["w_scales"], o_scale)
        lo, hi = type_range(c["src"].dtype)
        out = gpu_conv(ctx, c["src"], c["weights"], c["bias"], c["stride"], c["pad"], c["in_zp"], c["w_zp"], mult,
                       shift, c["out_zp"], lo, hi)
        assert np.array_equal(out, gold[c["key"] + "_out"]), c["key"]


@pytest.mark.parametrize("geom", [(3, 1, 1), (1, 1, 0), (3, 2, 1), (7, 2, 3), (1, 2, 0)])
@pytest.mark.parametrize("act", ["none", "relu", "lu_bounded"])
def test_conv_vs_oracle(ctx, port, geom, act):
    """ResNet-like layer shapes with the three activation variants the reference tests."""
    k, s, p = geom
    rng = np.random.default_rng(k * 100 + s * 10 + p)
    Cc = 3 if k == 7 else 64
    src = q8_uniform(rng, (3, 20, 20, Cc), np.uint8)
    wgt = q8_uniform(rng, (96, k, k, Cc), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, 96).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), 96)).astype(np.float32)
    mult, shift = f32_mults(port, 0.03, ws, 0.05)
    out_zp = 10
    lo, hi = {"none": (0, 255), "relu": (out_zp, 255), "lu_bounded": (out_zp + 2, out_zp + 120)}[act]
    want = port.conv2d_nhwc(src, wgt, bias, (s, s), (p, p, p, p), 128, 0, mult, shift, out_zp, lo, hi)
    for implicit in (True, False):  # gather-in-kernel and explicit im2col lowerings
        got = gpu_conv(ctx, src, wgt, bias, (s, s), (p, p, p, p), 128, 0, mult, shift, out_zp, lo, hi,
                       implicit=implicit)
        assert np.array_equal(got, want), implicit


def test_conv_asymmetric_weights_and_signed(ctx, port):
    rng = np.random.default_rng(77)
    src = q8_uniform(rng, (2, 15, 17, 32), np.int8)
    wgt = q8_uniform(rng, (40, 3, 3, 32), np.int8)
    bias = rng.integers(-500, 501, 40).astype(np.int32)
    mult, shift = f32_mults(port, 0.03, [0.004], 0.3)
    got = gpu_conv(ctx, src, wgt, bias, (1, 1), (1, 1, 1, 1), -5, 9, mult, shift, -3, -128, 127)
    want = port.conv2d_nhwc(src, wgt, bias, (1, 1), (1, 1, 1, 1), -5, 9, mult, shift, -3, -128, 127)
    assert np.array_equal(got, want)
    srcu = q8_uniform(rng, (2, 15, 17, 32), np.uint8)
    wgtu = q8_uniform(rng, (40, 3, 3, 32), np.uint8)
    got = gpu_conv(ctx, srcu, wgtu, bias, (2, 2), (0, 1, 0, 1), 130, 120, mult, shift, 4, 0, 255)
    want = port.conv2d_nhwc(srcu, wgtu, bias, (2, 2), (0, 1, 0, 1), 130, 120, mult, shift, 4, 0, 255)
    assert np.array_equal(got, want)


def test_config3_full_size(ctx, port):
    """Configuration 3 of the benchmark at full size: batch 32, 56x56x64 -> 64, 3x3 s1 p1, fused ReLU; exact on a batch sample
    and identical per image whatever the batch it is computed in (batch sharding needs no exchange)."""
    c = config3()
    mult, shift = f32_mults(port, c["i_scale"], c["w_scales"], c["o_scale"])
    out = gpu_conv(ctx, c["src"], c["weights"], c["bias"], c["stride"], c["pad"], c["in_zp"], 0, mult, shift,
                   c["out_zp"], c["lo"], c["hi"], want_kernel="implicit")
    explicit = gpu_conv(ctx, c["src"], c["weights"], c["bias"], c["stride"], c["pad"], c["in_zp"], 0, mult, shift,
                        c["out_zp"], c["lo"], c["hi"], implicit=False, want_kernel="im2col")
    assert np.array_equal(out, explicit)
    want = port.conv2d_nhwc(c["src"][:2], c["weights"], c["bias"], c["stride"], c["pad"], c["in_zp"], 0, mult, shift,
                            c["out_zp"], c["lo"], c["hi"])
    assert np.array_equal(out[:2], want)
    shard = gpu_conv(ctx, c["src"][28:], c["weights"], c["bias"], c["stride"], c["pad"], c["in_zp"], 0, mult, shift,
                     c["out_zp"], c["lo"], c["hi"])
    assert np.array_equal(shard, out[28:])
    assert 0.01 < (out == 0).mean() < 0.99


@pytest.mark.parametrize("geom", [(3, 1, 1, 1, 64, 96), (3, 2, 1, 1, 128, 300), (1, 2, 0, 1, 256, 64), (5, 1, 2, 1, 32, 40),
                                  (3, 1, 2, 2, 48, 130), (7, 2, 3, 1, 16, 64)])
@pytest.mark.parametrize("in_zp", [0, 128, 7])
def test_implicit_conv_vs_oracle(ctx, port, geom, in_zp):
    """The implicit-GEMM lowering on layer shapes of the ResNet family (3x3 s1/s2, strided 1x1, 5x5, dilated, 7x7)
    with zero and non-zero input zero points (the latter exercise the per-tap correction on border pixels)."""
    k, s, p, d, Cc, OFM = geom
    rng = np.random.default_rng(k * 1000 + s * 100 + Cc + in_zp)
    src = q8_uniform(rng, (2, 19, 23, Cc), np.uint8)
    wgt = q8_uniform(rng, (OFM, k, k, Cc), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, OFM).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)).astype(np.float32)
    mult, shift = f32_mults(port, 0.03, ws, 0.05 * k)
    want = port.conv2d_nhwc(src, wgt, bias, (s, s), (p, p, p, p), in_zp, 0, mult, shift, 3, 0, 255, dilation=(d, d))
    # 0: the library's own choice (narrow tiles here, the outputs are small); then every tile width by name
    for cols in (0, 256, 128, 64):
        got = gpu_conv(ctx, src, wgt, bias, (s, s), (p, p, p, p), in_zp, 0, mult, shift, 3, 0, 255, dilation=(d, d),
                       want_kernel="implicit", tile_columns=cols)
        assert np.array_equal(got, want), (cols, np.argwhere(got != want)[:5])


@pytest.mark.parametrize("geom", [(7, 3, 3, 20, 22), (7, 3, 3, 19, 23), (3, 1, 4, 17, 18), (5, 2, 1, 9, 11), (3, 0, 3, 12, 15),
                                  (2, 1, 2, 10, 10), (4, 2, 4, 21, 16), (3, 1, 3, 17, 18), (7, 3, 3, 19, 24)])
@pytest.mark.parametrize("in_zp", [0, 77])
def test_folded_stride2_conv_vs_oracle(ctx, port, geom, in_zp):
    """Stride-2 convolutions over at most four channels (the 7x7 / 2 stem of ResNet-50 on RGB images) run as a
    2x2 space-to-depth 16-channel stride-1 convolution: even and odd image sizes, even and odd paddings, kernel
    sizes 2..7; both the implicit kernel and the explicit im2col lowering of the folded form."""
    k, p, Cc, H, W = geom
    rng = np.random.default_rng(k * 100 + p * 10 + Cc + in_zp)
    src = q8_uniform(rng, (2, H, W, Cc), np.uint8)
    wgt = q8_uniform(rng, (24, k, k, Cc), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, 24).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), 24)).astype(np.float32)
    mult, shift = f32_mults(port, 0.05, ws, 0.05)
    want = port.conv2d_nhwc(src, wgt, bias, (2, 2), (p, p, p, p), in_zp, 0, mult, shift, 0, 0, 255)
    for implicit in (True, False):
        got = gpu_conv(ctx, src, wgt, bias, (2, 2), (p, p, p, p), in_zp, 0, mult, shift, 0, 0, 255, implicit=implicit,
                       want_kernel="implicit" if implicit else "im2col")
        assert np.array_equal(got, want), (implicit, np.argwhere(got != want)[:5])


@pytest.mark.parametrize("geom", [(1, 1, 0, 64, 256), (3, 1, 1, 32, 40), (3, 2, 1, 16, 130), (1, 1, 0, 24, 20)])
def test_fused_residual_addition(ctx, port, geom):
    """cugl_conv2d_run_residual = convolution, QASYMM8 addition and activation in one kernel: against the oracle's
    three separate layers, on the implicit, the plain-GEMM and (C = 24) the explicit im2col / SIMT-free lowerings."""
    import torch
    k, s, p, Cc, OFM = geom
    rng = np.random.default_rng(k * 100 + Cc + OFM)
    src = q8_uniform(rng, (2, 14, 15, Cc), np.uint8)
    wgt = q8_uniform(rng, (OFM, k, k, Cc), np.int8, -127, 127)
    bias = rng.integers(-3000, 3001, OFM).astype(np.int32)
    ws = (np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)) / np.sqrt(k * k * Cc) * 8).astype(np.float32)
    q = (0.05, 0)
    mult, shift = f32_mults(port, q[0], ws, q[0])
    conv = port.conv2d_nhwc(src, wgt, bias, (s, s), (p, p, p, p), q[1], 0, mult, shift, q[1], 0, 255)
    res = q8_uniform(rng, conv.shape, np.uint8)
    for act, a, cm in (("relu", 0.0, -1), ("bounded_relu", 6.0, -1), ("relu", 0.0, 1)):
        want = port.activation_qasymm8(port.add_qasymm8(conv, res, q, q, q), act, a, 0.0, q, q)
        desc, keep = capi.make_conv_desc(2, 14, 15, Cc, OFM, k, k, (s, s), (p, p, p, p), (1, 1), capi.U8, capi.S8, q[1], 0,
                                         multipliers=mult, shifts=shift, dst_zp=q[1], min_bound=0, max_bound=255)
        plan = capi.ConvPlan(ctx, desc, keep)
        plan.set_residual(q[0], q, q, act=capi.ACT_RELU if act == "relu" else capi.ACT_BOUNDED_RELU, act_a=a)
        plan.set_channel_major(cm)
        plan.prepare(torch.from_numpy(wgt.view(np.uint8)).cuda())
        d_res = torch.from_numpy(res).cuda()
        d_dst = torch.empty(conv.shape, dtype=torch.uint8, device="cuda")
        plan.run_residual(torch.from_numpy(src).cuda(), torch.from_numpy(bias).cuda(), d_res, d_dst)
        ctx.sync()
        assert np.array_equal(d_dst.cpu().numpy(), want), act
        # in place: the residual buffer is also the destination
        plan.run_residual(torch.from_numpy(src).cuda(), torch.from_numpy(bias).cuda(), d_res, d_res)
        ctx.sync()
        assert np.array_equal(d_res.cpu().numpy(), want), act
        plan.close()
    # quantizations for which the addition is NOT a saturating byte addition are refused
    plan = capi.ConvPlan(ctx, desc, keep)
    with pytest.raises(capi.CuglError):
        plan.set_residual(0.05, (0.03, 5), (0.07, 9))
    plan.close()


@pytest.mark.parametrize("OFM", [256, 384])
@pytest.mark.parametrize("paired", [True, False])
def test_short_k_many_tiles_with_and_without_residual(ctx, port, paired, OFM):
    """1x1 convolution 64 -> 256 / 384 on 39200 output rows, with and without a fused residual: 307 row blocks for 148
    CTAs, so every CTA drains pairs of tiles and some a single one, the last row block is ragged, and with 384
    channels the second column block is half empty.  paired: two tiles of a column block drained together (one term
    read for two elements) or every tile on its own."""
    import torch
    rng = np.random.default_rng(99 + OFM)
    B, H, W, Cc = 8, 70, 70, 64
    src = q8_uniform(rng, (B, H, W, Cc), np.uint8)
    wgt = q8_uniform(rng, (OFM, 1, 1, Cc), np.int8, -127, 127)
    bias = rng.integers(-3000, 3001, OFM).astype(np.int32)
    ws = (np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)) / np.sqrt(Cc) * 8).astype(np.float32)
    q = (0.05, 0)
    mult, shift = f32_mults(port, q[0], ws, q[0])
    conv = port.conv2d_nhwc(src, wgt, bias, (1, 1), (0, 0, 0, 0), q[1], 0, mult, shift, q[1], 0, 255)
    res = q8_uniform(rng, conv.shape, np.uint8)
    want = port.activation_qasymm8(port.add_qasymm8(conv, res, q, q, q), "relu", 0.0, 0.0, q, q)
    desc, keep = capi.make_conv_desc(B, H, W, Cc, OFM, 1, 1, (1, 1), (0, 0, 0, 0), (1, 1), capi.U8, capi.S8, q[1], 0,
                                     multipliers=mult, shifts=shift, dst_zp=q[1], min_bound=0, max_bound=255)
    d_src, d_bias = torch.from_numpy(src).cuda(), torch.from_numpy(bias).cuda()
    plan = capi.ConvPlan(ctx, desc, keep)
    plan.set_paired_drain(paired)
    plan.set_channel_major(-1)
    plan.prepare(torch.from_numpy(wgt.view(np.uint8)).cuda())
    d_dst = torch.full(conv.shape, 0xA5, dtype=torch.uint8, device="cuda")
    for _ in range(2):
        plan.run(d_src, d_bias, d_dst)
    ctx.sync()
    assert np.array_equal(d_dst.cpu().numpy(), conv)
    plan.set_residual(q[0], q, q, act=capi.ACT_RELU, act_a=0.0)
    d_res = torch.from_numpy(res).cuda()
    d_dst.fill_(0x5A)
    for _ in range(2):
        plan.run_residual(d_src, d_bias, d_res, d_dst)
    ctx.sync()
    assert np.array_equal(d_dst.cpu().numpy(), want)
    plan.run_residual(d_src, d_bias, d_res, d_res)  # in place
    ctx.sync()
    assert np.array_equal(d_res.cpu().numpy(), want)
    plan.close()


def test_conv_update_quantization_and_bound_workspace(ctx, port):
    """cugl_conv2d_update_quantization (NEGEMMConvolutionLayer::update_quantization_parameters): new input zero
    point, multipliers, output zero point and bounds on prepared weights; on the explicit lowering with its im2col
    matrix in a workspace the caller owns."""
    import torch
    rng = np.random.default_rng(5)
    B, H, W, C_, OFM = 2, 9, 10, 16, 24
    src = q8_uniform(rng, (B, H, W, C_), np.uint8)
    wgt = q8_uniform(rng, (OFM, 3, 3, C_), np.int8, -127, 127)
    bias = rng.integers(-3000, 3001, OFM).astype(np.int32)
    ws = rng.uniform(2e-3, 8e-3, OFM).astype(np.float32)
    d_src, d_w, d_b = torch.from_numpy(src).cuda(), torch.from_numpy(wgt.view(np.uint8)).cuda(), torch.from_numpy(bias).cuda()
    for implicit in (True, False):
        def desc_for(i_scale, i_zp, o_scale, o_zp, lo, hi):
            mult, shift = capi.calculate_quantized_multipliers(np.float32(i_scale), ws, np.float32(o_scale))
            return capi.make_conv_desc(B, H, W, C_, OFM, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1), capi.U8, capi.S8, i_zp, 0,
                                       multipliers=mult, shifts=shift, dst_zp=o_zp, min_bound=lo, max_bound=hi), (mult, shift)
        (desc, keep), (mult, shift) = desc_for(0.03, 128, 0.05, 0, 0, 255)
        plan = capi.ConvPlan(ctx, desc, keep)
        plan.allow_implicit(implicit)
        nbytes = plan.temp_bytes
        assert (nbytes > 0) == (not implicit)
        wsbuf = torch.full((nbytes + 64,), 0x77, dtype=torch.uint8, device="cuda")
        plan.bind_temp(wsbuf, nbytes)
        d_dst = torch.empty((B, H, W, OFM), dtype=torch.uint8, device="cuda")
        plan.prepare(d_w)
        plan.run(d_src, d_b, d_dst)
        ctx.sync()
        assert np.array_equal(d_dst.cpu().numpy(), port.conv2d_nhwc(src, wgt, bias, (1, 1), (1, 1, 1, 1), 128, 0, mult, shift, 0, 0, 255))
        (desc2, keep2), (mult2, shift2) = desc_for(0.02, 100, 0.04, 9, 9, 200)
        plan.update_quantization(desc2, keep2)
        plan.run(d_src, d_b, d_dst)
        ctx.sync()
        assert np.array_equal(d_dst.cpu().numpy(), port.conv2d_nhwc(src, wgt, bias, (1, 1), (1, 1, 1, 1), 100, 0, mult2, shift2, 9, 9, 200))
        assert (wsbuf[nbytes:] == 0x77).all()
        plan.close()


def test_transpose_batched_is_the_nchw_nhwc_permute(ctx):
    import torch
    rng = np.random.default_rng(6)
    x = rng.integers(0, 256, (3, 37, 11 * 13), dtype=np.uint8)  # [B][C][H*W]
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.empty((3, 11 * 13, 37), dtype=torch.uint8, device="cuda")
    ctx.transpose_batched(d_x, d_y, 37, 11 * 13, 3)
    ctx.sync()
    assert np.array_equal(d_y.cpu().numpy(), x.transpose(0, 2, 1))


@pytest.mark.parametrize("geom", [(3, 1, 1, 1, 128, 64, 14, 14), (3, 2, 1, 1, 128, 128, 28, 28), (3, 1, 1, 1, 256, 256, 14, 14),
                                  (3, 1, 1, 1, 512, 96, 7, 7), (3, 1, 2, 2, 128, 130, 19, 23), (5, 2, 2, 1, 128, 40, 21, 17),
                                  (1, 2, 0, 1, 256, 64, 19, 23), (3, 2, (0, 1, 0, 1), 1, 128, 64, 16, 18),
                                  (3, 1, 1, 1, 64, 64, 14, 14), (3, 2, 1, 1, 64, 96, 28, 28), (5, 1, 2, 1, 64, 40, 13, 11),
                                  (3, 1, 1, 1, 64, 300, 10, 12), (2, 1, (0, 1, 0, 1), 1, 64, 64, 9, 9)])
@pytest.mark.parametrize("batch", [1, 5])
def test_tma_im2col_conv_vs_oracle(ctx, port, geom, batch):
    """The im2col-mode TMA route of the implicit lowering (input zero point 0, channels a multiple of 128, or 64 channels
    as 64-byte-swizzle tiles of one filter tap each: odd and even tap counts) on the 3x3
    layer shapes of ResNet-50 (stride 1 and 2), dilated, 5x5 / 2, strided 1x1 and asymmetric padding: against the oracle,
    against the gather route, and with every tile width.  batch 5 makes tiles straddle image boundaries and leaves a
    ragged last tile (rows beyond the last image must read as zero and are never stored)."""
    k, s, p, d, Cc, OFM, H, W = geom
    pad = p if isinstance(p, tuple) else (p, p, p, p)
    rng = np.random.default_rng(k * 1000 + s * 100 + Cc + batch)
    src = q8_uniform(rng, (batch, H, W, Cc), np.uint8)
    wgt = q8_uniform(rng, (OFM, k, k, Cc), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, OFM).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)).astype(np.float32)
    mult, shift = f32_mults(port, 0.03, ws, 0.05 * k)
    want = port.conv2d_nhwc(src, wgt, bias, (s, s), pad, 0, 0, mult, shift, 3, 0, 255, dilation=(d, d))
    gather = gpu_conv(ctx, src, wgt, bias, (s, s), pad, 0, 0, mult, shift, 3, 0, 255, dilation=(d, d), want_kernel="implicit",
                      tma_im2col=False, want_tma=False)
    assert np.array_equal(gather, want)
    for cols in (0, 256, 128, 64):
        got = gpu_conv(ctx, src, wgt, bias, (s, s), pad, 0, 0, mult, shift, 3, 0, 255, dilation=(d, d), want_kernel="implicit",
                       tile_columns=cols, tma_im2col=2 if Cc == 64 else True, want_tma=True)
        assert np.array_equal(got, want), (cols, np.argwhere(got != want)[:5])


def test_tma_im2col_is_not_used_where_it_is_inexact(ctx):
    """A non-zero input zero point (out-of-image taps would read 0 instead of it) or a channel count that is not a
    multiple of 128 keep the plan on the gather; 64 channels take the TMA route only on request."""
    for Cc, zp, want in ((128, 0, True), (64, 0, False), (128, 3, False), (32, 0, False), (192, 0, False)):
        desc, keep = capi.make_conv_desc(1, 8, 8, Cc, 16, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1), capi.U8, capi.S8, zp, 0,
                                         multiplier=1 << 30, shift=8, dst_zp=0, min_bound=0, max_bound=255)
        plan = capi.ConvPlan(ctx, desc, keep)
        assert plan.uses_tma_im2col == want
        plan.allow_tma_im2col(2)
        assert plan.uses_tma_im2col == (zp == 0 and Cc in (64, 128))
        plan.close()


@pytest.mark.parametrize("geom", [(26, 28, 128, 256, 1), (27, 30, 128, 320, 1), (50, 39, 256, 256, 2)])
def test_tma_im2col_on_the_sm_pair_kernel(ctx, port, geom):
    """Convolutions with at least one 256 x 256 tile per SM pair run the im2col-mode route on the cta_group::2 kernel
    (each CTA loads the patches of its own 128 output pixels): against the gather route on the whole output, against
    the oracle on the first and last images; ragged M, ragged N (320 channels) and stride 2."""
    B, H, Cc, OFM, s = geom
    rng = np.random.default_rng(B * 10 + s)
    src = q8_uniform(rng, (B, H, H, Cc), np.uint8)
    wgt = q8_uniform(rng, (OFM, 3, 3, Cc), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, OFM).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)).astype(np.float32)
    mult, shift = f32_mults(port, 0.03, ws, 0.15)
    tma = gpu_conv(ctx, src, wgt, bias, (s, s), (1, 1, 1, 1), 0, 0, mult, shift, 3, 0, 255, want_kernel="implicit", want_tma=True)
    gather = gpu_conv(ctx, src, wgt, bias, (s, s), (1, 1, 1, 1), 0, 0, mult, shift, 3, 0, 255, want_kernel="implicit",
                      tma_im2col=False, want_tma=False)
    assert np.array_equal(tma, gather), np.argwhere(tma != gather)[:5]
    for sl in (slice(0, 1), slice(B - 1, B)):
        want = port.conv2d_nhwc(src[sl], wgt, bias, (s, s), (1, 1, 1, 1), 0, 0, mult, shift, 3, 0, 255)
        assert np.array_equal(tma[sl], want)
    assert 0.01 < (tma == 0).mean() < 0.99 and 0.01 < (tma == 255).mean() + (tma < 255).mean()


@pytest.mark.parametrize("geom", [((3, 3), 1, 1, 64, 64, 30, 28, 128), ((3, 3), 2, 1, 64, 40, 29, 31, 7), ((7, 7), 2, 3, 3, 64, 61, 64, 128),
                                  ((2, 5), 1, 0, 64, 64, 17, 19, 0), ((1, 3), 1, 0, 16, 24, 40, 33, 250),
                                  ((3, 3), 1, 1, 80, 64, 20, 20, 128), ((3, 3), 1, 1, 64, 72, 20, 20, 128)])
@pytest.mark.parametrize("batch", [1, 7])
def test_resident_weights_conv_vs_oracle(ctx, port, geom, batch):
    """Gather convolutions with at most 64 output channels and K <= 640 keep the weight operand in shared memory for the
    life of a thread block: the 3x3 x 64 and folded 7x7 x 3 layers of ResNet-50, K exactly 640, a ragged K (48) and N
    (24, 40), many tiles per block (batch 7) -- against the oracle and against the per-tile reload; K = 720 and 72
    output channels lie past the limits and must come out the same through the reloading kernel."""
    (kh, kw), s, p, Cc, OFM, H, W, in_zp = geom
    rng = np.random.default_rng(kh * 1000 + kw * 100 + Cc + OFM + batch)
    src = q8_uniform(rng, (batch, H, W, Cc), np.uint8)
    wgt = q8_uniform(rng, (OFM, kh, kw, Cc), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, OFM).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)).astype(np.float32)
    mult, shift = f32_mults(port, 0.03, ws, 0.05 * max(kh, kw))
    want = port.conv2d_nhwc(src, wgt, bias, (s, s), (p, p, p, p), in_zp, 0, mult, shift, 3, 0, 255)
    for resident in (True, False):
        got = gpu_conv(ctx, src, wgt, bias, (s, s), (p, p, p, p), in_zp, 0, mult, shift, 3, 0, 255, want_kernel="implicit",
                       tma_im2col=False, resident_weights=resident)
        assert np.array_equal(got, want), (resident, np.argwhere(got != want)[:5])


@pytest.mark.parametrize("geom", [(16, 56, 56, 1, 64, 128), (13, 57, 59, 1, 40, 0), (11, 60, 61, 1, 64, 0), (50, 57, 59, 2, 64, 7)])
def test_double_tile_conv_vs_oracle(ctx, port, geom):
    """3x3 x 64 convolutions large enough (more than 256 output pixels per SM) for the gather kernel's 256-pixel units,
    two tiles per barrier hand-over: a whole number of units, a ragged last unit whose second tile is partly or wholly
    beyond M, stride 2 and 40 output channels -- against the oracle and against the 128-pixel units."""
    B, H, W, s, OFM, in_zp = geom
    rng = np.random.default_rng(B * 100 + H + OFM)
    src = q8_uniform(rng, (B, H, W, 64), np.uint8)
    wgt = q8_uniform(rng, (OFM, 3, 3, 64), np.int8, -127, 127)
    bias = rng.integers(-5000, 5001, OFM).astype(np.int32)
    ws = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), OFM)).astype(np.float32)
    mult, shift = f32_mults(port, 0.03, ws, 0.15)
    want = port.conv2d_nhwc(src, wgt, bias, (s, s), (1, 1, 1, 1), in_zp, 0, mult, shift, 3, 0, 255)
    assert want.shape[0] * want.shape[1] * want.shape[2] > 256 * 148
    for double in (True, False):
        got = gpu_conv(ctx, src, wgt, bias, (s, s), (1, 1, 1, 1), in_zp, 0, mult, shift, 3, 0, 255, want_kernel="implicit",
                       tma_im2col=False, double_tile=double)
        assert np.array_equal(got, want), (double, np.argwhere(got != want)[:5])
