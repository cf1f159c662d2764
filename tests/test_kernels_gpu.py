"""Stand-alone kernels of the path against the oracle (bit-exact)."""
import os

import numpy as np
import pytest

from computelibrary_b200 import capi
from helpers import golden_im2col_cases, q8_uniform, type_range

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _t(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("M,K", [(1, 1), (7, 5), (64, 256), (333, 1000), (4096, 4096), (100, 4608), (5000, 147)])
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_reduce_rows(ctx, port, M, K, dtype):
    import torch
    a = q8_uniform(np.random.default_rng(M + K), (M, K), dtype)
    out = torch.empty(M, dtype=torch.int32, device="cuda")
    code = capi.U8 if dtype == np.uint8 else capi.S8
    ctx.reduce_rows(_t(a.view(np.uint8)), code, M, K, K, out)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), port.reduce_rows(a))
    # strided rows with an odd pitch (exercises the unaligned head/tail path) and a scalar
    pitch = K + 3
    buf = np.zeros((M, pitch), dtype)
    buf[:, :K] = a
    ctx.reduce_rows(_t(buf.view(np.uint8)), code, M, K, pitch, out, scalar=-7)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), port.reduce_rows(a) * -7)


@pytest.mark.parametrize("K,N", [(1, 1), (5, 7), (256, 128), (1000, 333), (4096, 4096), (147, 64), (33, 1001)])
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_reduce_cols(ctx, port, K, N, dtype):
    import torch
    b = q8_uniform(np.random.default_rng(K * 3 + N), (K, N), dtype)
    out = torch.empty(N, dtype=torch.int32, device="cuda")
    code = capi.U8 if dtype == np.uint8 else capi.S8
    ctx.reduce_cols(_t(b.view(np.uint8)), code, K, N, N, out)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), port.reduce_cols(b))
    ctx.reduce_cols(_t(b.view(np.uint8)), code, K, N, N, out, scalar=5)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), port.reduce_cols(b) * 5)


def test_offset_contribution(ctx, port):
    rng = np.random.default_rng(1)
    M, N, K = 97, 131, 77
    mm = rng.integers(-2 ** 20, 2 ** 20, (M, N)).astype(np.int32)
    cs = rng.integers(-30000, 30000, N).astype(np.int32)
    rs = rng.integers(-30000, 30000, M).astype(np.int32)
    for ao, bo in [(0, 0), (5, 0), (0, -7), (-128, 120)]:
        d = _t(mm)
        ctx.offset_contribution(d, M, N, K, N * 4, _t(cs), _t(rs), ao, bo)
        ctx.sync()
        assert np.array_equal(d.cpu().numpy(), port.offset_contribution(mm, K, cs, rs, ao, bo)), (ao, bo)


@pytest.mark.parametrize("out_dtype", [np.uint8, np.int8])
@pytest.mark.parametrize("M,N", [(1, 1), (37, 53), (64, 128), (300, 1001)])
def test_output_stage(ctx, port, out_dtype, M, N):
    import torch
    rng = np.random.default_rng(M * N)
    acc = rng.integers(-6000, 6001, (M, N)).astype(np.int32)
    acc.flat[:4] = [2 ** 31 - 1, -2 ** 31, -1, 1][:acc.size]
    bias = rng.integers(-2000, 2001, N).astype(np.int32)
    lo, hi = type_range(out_dtype)
    code = capi.U8 if out_dtype == np.uint8 else capi.S8
    out = torch.empty((M, N), dtype=torch.uint8, device="cuda")
    for (qm, sh) in [(1099511552, 8), (2 ** 30, 0), (2 ** 30, -2), (2147483647, 31)]:
        for b in (None, bias):
            ctx.output_stage(_t(acc), N * 4, _t(b) if b is not None else None, out, N, code, M, N, None, None, qm,
                             sh, 1, 10, lo + 1, hi - 1)
            ctx.sync()
            want = port.output_stage(acc, b, [qm], [sh], 10, lo + 1, hi - 1, out_dtype)
            assert np.array_equal(out.cpu().numpy().view(out_dtype), want), (qm, sh)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
    shift = rng.integers(-2, 12, N).astype(np.int32)
    # n_mult == 1 means per-tensor in the C ABI, so a single column passes its multiplier by value
    ctx.output_stage(_t(acc), N * 4, _t(bias), out, N, code, M, N, _t(mult), _t(shift), int(mult[0]), int(shift[0]),
                     N, -4, lo, hi)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy().view(out_dtype), port.output_stage(acc, bias, mult, shift, -4, lo, hi, out_dtype))


@pytest.mark.parametrize("out_dtype", [np.uint8, np.int8])
@pytest.mark.parametrize("M,N", [(1, 1), (37, 53), (300, 1001)])
def test_output_stage_quantize_down(ctx, port, out_dtype, M, N):
    """The integer-multiply stage (GEMMLowpOutputStageType::QUANTIZE_DOWN) of the stand-alone output stage."""
    import torch
    rng = np.random.default_rng(M * N + 5)
    acc = rng.integers(-2 ** 22, 2 ** 22, (M, N)).astype(np.int32)
    acc.flat[:2] = [2 ** 31 - 1, -2 ** 31][:acc.size]
    bias = rng.integers(-9000, 9001, N).astype(np.int32)
    lo, hi = type_range(out_dtype)
    code = capi.U8 if out_dtype == np.uint8 else capi.S8
    out = torch.empty((M, N), dtype=torch.uint8, device="cuda")
    for (qm, sh, blo, bhi) in [(3, 5, lo + 1, hi - 1), (-7, 0, 0, 0), (251, 23, lo, hi)]:
        for b in (None, bias):
            ctx.output_stage_quantize_down(_t(acc), N * 4, _t(b) if b is not None else None, out, N, code, M, N, None,
                                           None, qm, sh, 1, 77, blo, bhi)
            ctx.sync()
            want = port.output_stage_int(acc, b, [qm], [sh], 77, blo, bhi, out_dtype)
            assert np.array_equal(out.cpu().numpy().view(out_dtype), want), (qm, sh)
    if N > 1:
        mult = rng.integers(1, 400, N).astype(np.int32)
        shift = rng.integers(0, 20, N).astype(np.int32)
        ctx.output_stage_quantize_down(_t(acc), N * 4, _t(bias), out, N, code, M, N, _t(mult), _t(shift), 0, 0, N, -4,
                                       lo + 3, hi - 3)
        ctx.sync()
        assert np.array_equal(out.cpu().numpy().view(out_dtype),
                              port.output_stage_int(acc, bias, mult, shift, -4, lo + 3, hi - 3, out_dtype))


@pytest.mark.parametrize("M,N", [(1, 1), (37, 53), (300, 1000)])
def test_output_stage_qsymm16(ctx, port, M, N):
    """NEGEMMLowpOutputStage with a QSYMM16 destination (cugl_output_stage, out_dtype CUGL_S16): per-tensor and
    per-channel, with and without bias, odd and 8-byte aligned rows, bounded and whole-range."""
    import torch
    rng = np.random.default_rng(M * N + 16)
    acc = rng.integers(-2 ** 24, 2 ** 24, (M, N)).astype(np.int32)
    acc.flat[:2] = [2 ** 31 - 1, -2 ** 31][:acc.size]
    bias = rng.integers(-9000, 9001, N).astype(np.int32)
    out = torch.empty((M, N), dtype=torch.int16, device="cuda")
    for (qm, sh, lo, hi) in [(1759218688, 9, -32768, 32767), (1234567890, -1, -1000, 2000), (2 ** 31 - 1, 3, 0, 0)]:
        for b in (None, bias):
            ctx.output_stage(_t(acc), N * 4, _t(b) if b is not None else None, out, N * 2, capi.S16, M, N, None, None,
                             qm, sh, 1, 0, lo, hi)
            ctx.sync()
            want = port.output_stage(acc, b, [qm], [sh], 0, lo, hi, np.int16)
            assert np.array_equal(out.cpu().numpy(), want), (qm, sh, lo, hi)
    if N > 1:
        mult = rng.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
        shift = rng.integers(-1, 14, N).astype(np.int32)
        ctx.output_stage(_t(acc), N * 4, _t(bias), out, N * 2, capi.S16, M, N, _t(mult), _t(shift), 0, 0, N, 5, -30000,
                         31000)
        ctx.sync()
        assert np.array_equal(out.cpu().numpy(), port.output_stage(acc, bias, mult, shift, 5, -30000, 31000, np.int16))


def test_im2col_golden_and_oracle(ctx, port):
    import torch
    gold = np.load(os.path.join(GOLDEN, "conv_golden.npz"))
    for c in golden_im2col_cases():
        src = c["src"]
        B, H, W, Cc = src.shape
        kw, kh, (sx, sy), (pl, pr, pt, pb) = c["kw"], c["kh"], c["stride"], c["pad"]
        wo, ho = port.conv_out_dims(W, H, kw, kh, sx, sy, pl, pr, pt, pb)
        K = kh * kw * Cc
        for rs in (K, (K + 15) // 16 * 16 + 16):
            dst = torch.full((B * ho * wo, rs), 0xEE, dtype=torch.uint8, device="cuda")
            ctx.im2col_nhwc(_t(src), dst, Cc, W, H, B, kw, kh, sx, sy, pl, pt, 1, 1, wo, ho, c["zp"], rs)
            ctx.sync()
            got = dst.cpu().numpy().reshape(B, ho * wo, rs)
            assert np.array_equal(got[:, :, :K], gold[c["key"]]), c["key"]
            assert not got[:, :, K:].any()
    # a larger, vectorisable case (C = 64) incl. dilation, against the oracle
    src = q8_uniform(np.random.default_rng(3), (4, 28, 28, 64), np.uint8)
    for (k, s, p, d) in [(3, 1, 1, 1), (3, 2, 1, 1), (3, 1, 2, 2), (7, 2, 3, 1)]:
        wo, ho = port.conv_out_dims(28, 28, k, k, s, s, p, p, p, p, d, d)
        K = k * k * 64
        dst = torch.empty((4 * ho * wo, K), dtype=torch.uint8, device="cuda")
        ctx.im2col_nhwc(_t(src), dst, 64, 28, 28, 4, k, k, s, s, p, p, d, d, wo, ho, 128, K)
        ctx.sync()
        want = port.im2col_nhwc(src, k, k, s, s, p, p, p, p, 128, d, d)
        assert np.array_equal(dst.cpu().numpy().reshape(want.shape), want), (k, s, p, d)


def test_weights_reshape(ctx, port):
    import torch
    w = q8_uniform(np.random.default_rng(5), (70, 3, 3, 24), np.int8)
    K = 3 * 3 * 24
    dst = torch.empty((K, 70), dtype=torch.int8, device="cuda")
    ctx.weights_reshape_nhwc(_t(w), dst, K, 70)
    ctx.sync()
    assert np.array_equal(dst.cpu().numpy(), port.weights_reshape_nhwc(w))
