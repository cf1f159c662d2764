"""CUDA QASYMM8 layers (cugl_pool2d_nhwc, cugl_add_qasymm8, cugl_activation_qasymm8, cugl_softmax_qasymm8)
against the CPU oracle and the committed reference fixtures: bit-exact, except softmax (+-1, the reference's
own tolerance for quantized softmax)."""
import os

import numpy as np
import pytest

from helpers import golden_act_cases, golden_add_cases, golden_pool_cases, golden_softmax_cases, pool_with

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
ACT = {"relu": 0, "bounded_relu": 1, "lu_bounded_relu": 2}


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(GOLDEN, "layers_golden.npz"))


def gpu_pool(ctx, c):
    import torch
    from computelibrary_b200 import capi
    pt, size, stride, pad, excl, glob = c["geom"]
    B, H, W, Cc = c["src"].shape
    d = capi.make_pool_desc(B, H, W, Cc, capi.POOL_MAX if pt == "max" else capi.POOL_AVG, size or (1, 1),
                            stride or (1, 1), pad or (0, 0, 0, 0), c["in_q"], c["out_q"], excl, glob)
    wo, ho = capi.pool_out_dims(d)
    src = torch.from_numpy(c["src"]).cuda()
    dst = torch.full((B, ho, wo, Cc), 0xAB, dtype=torch.uint8, device="cuda")
    ctx.pool2d_nhwc(d, src, dst)
    ctx.sync()
    return dst.cpu().numpy()


def test_pool_golden(ctx, port, golden):
    for c in golden_pool_cases():
        got = gpu_pool(ctx, c)
        np.testing.assert_array_equal(got, golden[c["key"]], err_msg=c["key"])
        np.testing.assert_array_equal(got, pool_with(port, c), err_msg=c["key"])


def test_pool_resnet_shapes(ctx, port):
    r = np.random.default_rng(21)
    for shape, geom in [((2, 112, 112, 64), ("max", (3, 3), (2, 2), (0, 1, 0, 1), False, False)),
                        ((2, 56, 56, 256), ("max", (1, 1), (2, 2), (0, 0, 0, 0), True, False)),
                        ((4, 7, 7, 2048), ("avg", None, None, None, False, True)),
                        # enough outputs for the four-channels-per-thread average kernel (a whole batch of 256 at the
                        # end of ResNet-50 has them too), padded and unpadded windows, both area rules
                        ((2, 40, 40, 128), ("avg", (3, 3), (1, 1), (1, 1, 1, 1), False, False)),
                        ((2, 40, 40, 128), ("avg", (3, 3), (1, 1), (1, 1, 1, 1), True, False)),
                        ((160, 7, 7, 2048), ("avg", None, None, None, False, True))]:
        c = dict(src=r.integers(0, 256, shape, dtype=np.uint8), geom=geom, in_q=(0.05, 0), out_q=(0.05, 0))
        np.testing.assert_array_equal(gpu_pool(ctx, c), pool_with(port, c))


def test_pool_validate(ctx):
    from computelibrary_b200 import capi
    with pytest.raises(capi.CuglError):
        capi.pool_validate(capi.make_pool_desc(1, 8, 8, 4, capi.POOL_MAX, (2, 2), (1, 1), (2, 0, 0, 0), (0.1, 0), (0.1, 0)))
    with pytest.raises(capi.CuglError):
        capi.pool_validate(capi.make_pool_desc(1, 8, 8, 4, capi.POOL_AVG, (3, 3), (0, 1), (0, 0, 0, 0), (0.1, 0), (0.1, 0)))
    with pytest.raises(capi.CuglError):
        capi.pool_validate(capi.make_pool_desc(1, 8, 8, 4, 7, (3, 3), (1, 1), (0, 0, 0, 0), (0.1, 0), (0.1, 0)))


def test_add_golden(ctx, golden):
    import torch
    for c in golden_add_cases():
        n = c["a"].size
        a, b = torch.from_numpy(c["a"]).cuda(), torch.from_numpy(c["b"]).cuda()
        dst = torch.empty(n, dtype=torch.uint8, device="cuda")
        ctx.add_qasymm8(a, b, dst, n, *c["q"])
        ctx.sync()
        np.testing.assert_array_equal(dst.cpu().numpy(), golden[c["key"]], err_msg=c["key"])


def test_add_with_activation_and_unaligned(ctx, port):
    import torch
    from computelibrary_b200 import capi
    r = np.random.default_rng(5)
    n = 100003
    a, b = r.integers(0, 256, n + 1, dtype=np.uint8), r.integers(0, 256, n + 1, dtype=np.uint8)
    qs = ((0.05, 3), (0.04, 9), (0.06, 12))
    want = port.activation_qasymm8(port.add_qasymm8(a[1:], b[1:], *qs), "bounded_relu", 6.0, 0.0, qs[2], qs[2])
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dst = torch.empty(n + 1, dtype=torch.uint8, device="cuda")
    ctx.add_qasymm8(da[1:], db[1:], dst[1:], n, *qs, act=capi.ACT_BOUNDED_RELU, act_a=6.0)   # misaligned by one byte
    ctx.sync()
    np.testing.assert_array_equal(dst[1:].cpu().numpy(), want)
    # every tensor at (0.05, 0) + ReLU: the saturating byte addition of the ResNet-50 residual path
    q0 = (0.05, 0)
    ctx.add_qasymm8(da, db, dst, n + 1, q0, q0, q0, act=capi.ACT_RELU)
    ctx.sync()
    np.testing.assert_array_equal(dst.cpu().numpy(), np.minimum(a.astype(np.int32) + b, 255).astype(np.uint8))


def test_activation_golden(ctx, golden):
    import torch
    for c in golden_act_cases():
        n = c["src"].size
        src = torch.from_numpy(c["src"]).cuda()
        dst = torch.empty(n, dtype=torch.uint8, device="cuda")
        ctx.activation_qasymm8(src, dst, n, ACT[c["act"]], c["a"], c["b"], c["in_q"], c["out_q"])
        ctx.sync()
        np.testing.assert_array_equal(dst.cpu().numpy(), golden[c["key"]], err_msg=c["key"])


def test_softmax_golden(ctx, golden):
    import torch
    for c in golden_softmax_cases():
        rows, cols = c["src"].shape
        src = torch.from_numpy(c["src"]).cuda()
        dst = torch.empty((rows, cols), dtype=torch.uint8, device="cuda")
        ctx.softmax_qasymm8(src, dst, rows, cols, c["beta"], c["q"])
        ctx.sync()
        diff = np.abs(dst.cpu().numpy().astype(np.int32) - golden[c["key"]].astype(np.int32))
        assert diff.max() <= 1, (c["key"], int(diff.max()))


@pytest.mark.parametrize("window", [((3, 3), (2, 2), (0, 1, 0, 1)), ((3, 3), (2, 2), (1, 1, 1, 1)), ((3, 3), (1, 1), (1, 1, 1, 1)),
                                    ((3, 3), (2, 3), (2, 0, 1, 2)), ((2, 2), (2, 2), (0, 0, 0, 0)), ((2, 2), (1, 2), (1, 1, 0, 1)),
                                    ((1, 1), (2, 2), (0, 0, 0, 0)), ((1, 1), (1, 1), (0, 0, 0, 0)), ((3, 2), (2, 2), (1, 0, 0, 1)),
                                    ((5, 5), (3, 3), (2, 2, 2, 2))])
@pytest.mark.parametrize("quant", [((0.05, 0), (0.05, 0)), ((0.05, 3), (0.05, 3)), ((0.05, 3), (0.07, 10)), ((0.11, 0), (0.02, 128))])
def test_max_pool_windows(ctx, port, window, quant):
    """MAX pooling over the unrolled window kernels (3x3, 2x2, 1x1; 16 channels per thread) and the general one (3x2, 5x5
    and 24 channels): padded borders on every side, odd image sizes, strides that differ in x and y, and both the
    identity table (equal quantization: bytes stored as they are) and a real requantisation, against the oracle."""
    size, stride, pad = window
    r = np.random.default_rng(size[0] * 100 + size[1] * 10 + stride[0] + pad[0])
    for shape in ((3, 23, 17, 32), (2, 9, 14, 64), (1, 12, 11, 24)):
        c = dict(src=r.integers(0, 256, shape, dtype=np.uint8), geom=("max", size, stride, pad, False, False),
                 in_q=quant[0], out_q=quant[1])
        np.testing.assert_array_equal(gpu_pool(ctx, c), pool_with(port, c), err_msg=str((shape, window, quant)))
