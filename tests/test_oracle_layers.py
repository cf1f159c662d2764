"""Pins the CPU restatement of the QASYMM8 layers (oracle/layers_oracle.c: pooling, addition, activation,
softmax) to Compute Library's own scalar oracle: the committed fixtures of tests/golden/layers_golden.npz
(produced by the reference's PoolingLayer.cpp / ArithmeticOperations.cpp / ActivationLayer.cpp /
SoftmaxLayer.cpp compiled in place) and, when oracle/_ref/libacl_ref.so is present, the reference itself."""
import os

import numpy as np
import pytest

from helpers import golden_act_cases, golden_add_cases, golden_pool_cases, golden_softmax_cases, pool_with

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(GOLDEN, "layers_golden.npz"))


def test_pool_golden(port, golden):
    n = 0
    for c in golden_pool_cases():
        np.testing.assert_array_equal(pool_with(port, c), golden[c["key"]], err_msg=c["key"])
        n += 1
    assert n == 72


def test_add_golden(port, golden):
    for c in golden_add_cases():
        np.testing.assert_array_equal(port.add_qasymm8(c["a"], c["b"], *c["q"]), golden[c["key"]], err_msg=c["key"])


def test_activation_golden(port, golden):
    for c in golden_act_cases():
        got = port.activation_qasymm8(c["src"], c["act"], c["a"], c["b"], c["in_q"], c["out_q"])
        np.testing.assert_array_equal(got, golden[c["key"]], err_msg=c["key"])


def test_softmax_golden(port, golden):
    # exp comes from the C library: the reference's own quantized softmax tests allow one step
    for c in golden_softmax_cases():
        got = port.softmax_qasymm8(c["src"], c["beta"], c["q"]).astype(np.int32)
        assert np.abs(got - golden[c["key"]].astype(np.int32)).max() <= 1, c["key"]


def test_equal_quantization_identities(port):
    """With equal input and output quantization ReLU is max(q, zero point) and max pooling is the byte maximum;
    with every tensor at (0.05, 0) the residual addition is a saturating byte addition."""
    q = np.arange(256, dtype=np.uint8)
    for scale, zp in [(0.05, 0), (0.03, 10), (0.5, 128), (0.0123, 77)]:
        got = port.activation_qasymm8(q, "relu", 0.0, 0.0, (scale, zp), (scale, zp))
        np.testing.assert_array_equal(got, np.maximum(q, zp))
    a, b = np.meshgrid(q, q)
    got = port.add_qasymm8(a.ravel(), b.ravel(), (0.05, 0), (0.05, 0), (0.05, 0))
    np.testing.assert_array_equal(got, np.minimum(a.ravel().astype(np.int32) + b.ravel(), 255).astype(np.uint8))
    r = np.random.default_rng(3)
    x = r.integers(0, 256, (2, 12, 12, 8), dtype=np.uint8)
    got = port.pool_nhwc(x, "max", (2, 2), (2, 2), (0, 0, 0, 0), (0.05, 0), (0.05, 0))
    np.testing.assert_array_equal(got, x.reshape(2, 6, 2, 6, 2, 8).max(axis=(2, 4)))


def test_layers_against_reference(port, ref):
    """Fresh random cases straight against the reference's code (skipped where it is not built)."""
    r = np.random.default_rng(11)
    for _ in range(10):
        B, H, W, Cc = int(r.integers(1, 3)), int(r.integers(5, 14)), int(r.integers(5, 14)), int(r.integers(1, 40))
        x = r.integers(0, 256, (B, H, W, Cc), dtype=np.uint8)
        in_q = (float(np.float32(r.uniform(0.01, 0.2))), int(r.integers(0, 256)))
        out_q = (float(np.float32(r.uniform(0.01, 0.2))), int(r.integers(0, 256)))
        pw, ph = int(r.integers(1, 4)), int(r.integers(1, 4))
        pad = (int(r.integers(0, pw)), int(r.integers(0, pw)), int(r.integers(0, ph)), int(r.integers(0, ph)))
        stride = (int(r.integers(1, 3)), int(r.integers(1, 3)))
        for pt in ("max", "avg"):
            for excl in (False, True):
                np.testing.assert_array_equal(port.pool_nhwc(x, pt, (pw, ph), stride, pad, in_q, out_q, excl),
                                              ref.pool_nhwc(x, pt, (pw, ph), stride, pad, in_q, out_q, excl))
        y = r.integers(0, 256, x.shape, dtype=np.uint8)
        o_q = (float(np.float32(r.uniform(0.01, 0.4))), int(r.integers(0, 256)))
        np.testing.assert_array_equal(port.add_qasymm8(x, y, in_q, out_q, o_q), ref.add_qasymm8(x, y, in_q, out_q, o_q))
        np.testing.assert_array_equal(port.activation_qasymm8(x, "lu_bounded_relu", 3.0, -1.0, in_q, out_q),
                                      ref.activation_qasymm8(x, "lu_bounded_relu", 3.0, -1.0, in_q, out_q))
