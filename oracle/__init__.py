"""CPU checkers for the quantized GEMM path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module: it is loaded by ``tests/``, by
``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py``.

``port``  -- ctypes view of ``libgemmlowp_oracle.so`` (the plain-C restatement, ``gemmlowp_oracle.c`` and
             ``layers_oracle.c``).
``ref``   -- ctypes view of ``_ref/libacl_ref.so`` (Compute Library's own scalar test oracle compiled in
             place by ``make -C oracle ref``), or ``None`` when that library has not been built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "libgemmlowp_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libacl_ref.so")

_i32 = C.c_int32
_p = C.c_void_p


def find_acl_root() -> str | None:
    """An unmodified Compute Library tree: $ACL_ROOT, else a directory named "reference" beside this repository."""
    for cand in (os.environ.get("ACL_ROOT"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "tests", "validation", "reference")):
            return cand
    return None


def build(want_ref: bool = True, acl_root: str | None = None) -> None:
    """Compile the C restatement and, when a Compute Library tree is present, the in-place reference."""
    subprocess.run(["make", "-C", _HERE, "port"], check=True, capture_output=True)
    acl_root = acl_root or find_acl_root()
    if want_ref and acl_root is not None:
        subprocess.run(["make", "-C", _HERE, "ref", f"ACL_ROOT={acl_root}"], check=True, capture_output=True)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


def _signed(a: np.ndarray) -> int:
    assert a.dtype in (np.int8, np.uint8), a.dtype
    return 1 if a.dtype == np.int8 else 0


def _i32arr(x) -> np.ndarray:
    return np.ascontiguousarray(np.atleast_1d(np.asarray(x, dtype=np.int32)))


class _Layers:
    """QASYMM8 layer oracles; `self._pfx` selects the C restatement ("orc_") or the reference ("ref_")."""

    @staticmethod
    def pool_out_dims(W, H, pw, ph, sx, sy, pl, pr, pt, pb):
        """FLOOR rounding (arm_compute::scaled_dimensions, src/core/Utils.cpp)."""
        return (W + pl + pr - pw) // sx + 1, (H + pt + pb - ph) // sy + 1

    def pool_nhwc(self, src, pool_type, size, stride, pad, in_q, out_q, exclude_padding=False, global_pool=False):
        """src [B,H,W,C] uint8; pool_type "max" | "avg"; size (pw, ph); pad (l, r, t, b); q = (scale, zero point)."""
        src = np.ascontiguousarray(src)
        assert src.dtype == np.uint8
        B, H, W, Cc = src.shape
        if global_pool:
            size, stride, pad = (W, H), (1, 1), (0, 0, 0, 0)
        pw, ph = size
        sx, sy = stride
        pl, pr, pt, pb = pad
        wo, ho = self.pool_out_dims(W, H, pw, ph, sx, sy, pl, pr, pt, pb)
        dst = np.empty((B, ho, wo, Cc), np.uint8)
        ptype = 0 if pool_type == "max" else 1
        if self._pfx == "orc_":
            self.lib.orc_pool_nhwc_u8(_ptr(src), _ptr(dst), Cc, W, H, B, ptype, pw, ph, sx, sy, pl, pr, pt, pb,
                                      int(exclude_padding), wo, ho, C.c_float(in_q[0]), C.c_int(in_q[1]),
                                      C.c_float(out_q[0]), C.c_int(out_q[1]))
        else:
            rw, rh = C.c_int(0), C.c_int(0)
            self.lib.ref_pool_nhwc_u8(_ptr(src), None, Cc, W, H, B, ptype, pw, ph, sx, sy, pl, pr, pt, pb,
                                      int(exclude_padding), int(global_pool), C.c_float(in_q[0]), C.c_int(in_q[1]),
                                      C.c_float(out_q[0]), C.c_int(out_q[1]), C.byref(rw), C.byref(rh))
            assert (rw.value, rh.value) == (wo, ho), "output-shape rule differs from the reference"
            self.lib.ref_pool_nhwc_u8(_ptr(src), _ptr(dst), Cc, W, H, B, ptype, pw, ph, sx, sy, pl, pr, pt, pb,
                                      int(exclude_padding), int(global_pool), C.c_float(in_q[0]), C.c_int(in_q[1]),
                                      C.c_float(out_q[0]), C.c_int(out_q[1]), None, None)
        return dst

    def add_qasymm8(self, a, b, a_q, b_q, o_q):
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        assert a.dtype == np.uint8 and b.dtype == np.uint8 and a.shape == b.shape
        dst = np.empty_like(a)
        getattr(self.lib, self._pfx + "add_qasymm8")(
            _ptr(a), _ptr(b), _ptr(dst), C.c_longlong(a.size), C.c_float(a_q[0]), C.c_int(a_q[1]), C.c_float(b_q[0]),
            C.c_int(b_q[1]), C.c_float(o_q[0]), C.c_int(o_q[1]))
        return dst

    def activation_qasymm8(self, src, act, a, b, in_q, out_q):
        """act: "relu" | "bounded_relu" (upper a) | "lu_bounded_relu" (upper a, lower b)."""
        src = np.ascontiguousarray(src)
        assert src.dtype == np.uint8
        dst = np.empty_like(src)
        code = {"relu": 0, "bounded_relu": 1, "lu_bounded_relu": 2}[act]
        getattr(self.lib, self._pfx + "activation_qasymm8")(
            _ptr(src), _ptr(dst), C.c_longlong(src.size), code, C.c_float(a), C.c_float(b), C.c_float(in_q[0]),
            C.c_int(in_q[1]), C.c_float(out_q[0]), C.c_int(out_q[1]))
        return dst

    def softmax_qasymm8(self, src, beta, in_q):
        """src [rows, cols] uint8; softmax along cols; output quantization (1/256, 0)."""
        src = np.ascontiguousarray(src)
        assert src.dtype == np.uint8 and src.ndim == 2
        dst = np.empty_like(src)
        getattr(self.lib, self._pfx + "softmax_qasymm8")(
            _ptr(src), _ptr(dst), src.shape[0], src.shape[1], C.c_float(beta), C.c_float(in_q[0]), C.c_int(in_q[1]))
        return dst


class _Port(_Layers):
    _pfx = "orc_"

    def __init__(self):
        if not os.path.exists(PORT_SO):
            build(want_ref=False)
        self.lib = C.CDLL(PORT_SO)
        L = self.lib
        L.orc_sqdmulh.restype = _i32
        L.orc_sqdmulh.argtypes = [_i32, _i32]
        L.orc_rounding_divide_by_pow2.restype = _i32
        L.orc_rounding_divide_by_pow2.argtypes = [_i32, _i32]
        L.orc_quantize_down_fixedpoint.restype = _i32
        L.orc_quantize_down_fixedpoint.argtypes = [_i32] * 6
        L.orc_calculate_quantized_multiplier.restype = C.c_int
        L.orc_calculate_quantized_multiplier.argtypes = [C.c_float, _p, _p]
        L.orc_num_threads.restype = C.c_int

    # scalar helpers -----------------------------------------------------------------------------
    def sqdmulh(self, a, b):
        return int(self.lib.orc_sqdmulh(a, b))

    def rounding_divide_by_pow2(self, x, e):
        return int(self.lib.orc_rounding_divide_by_pow2(x, e))

    def quantize_down(self, acc, mult, shift, offset, lo, hi):
        return int(self.lib.orc_quantize_down_fixedpoint(acc, mult, shift, offset, lo, hi))

    def calculate_quantized_multiplier(self, multiplier: float):
        m, s = _i32(0), _i32(0)
        rc = self.lib.orc_calculate_quantized_multiplier(C.c_float(multiplier), C.byref(m), C.byref(s))
        if rc != 0:
            raise ValueError(f"multiplier {multiplier} cannot be quantised")
        return int(m.value), int(s.value)

    def calculate_quantized_multipliers(self, i_scale, w_scales, o_scale):
        w = np.ascontiguousarray(np.asarray(w_scales, dtype=np.float32))
        n = w.size
        m = np.zeros(n, np.int32)
        s = np.zeros(n, np.int32)
        rc = self.lib.orc_calculate_quantized_multipliers(
            C.c_float(i_scale), _ptr(w), C.c_int(n), C.c_float(o_scale), _ptr(m), _ptr(s))
        if rc != 0:
            raise ValueError("scale cannot be quantised")
        return m, s

    def num_threads(self) -> int:
        return int(self.lib.orc_num_threads())

    # matrices -----------------------------------------------------------------------------------
    def gemmlowp_core(self, a, b, a_off, b_off):
        """a [M,K] or [batch,M,K]; b [K,N] or [batch,K,N] -> int32 [.., M, N]."""
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        batched = a.ndim == 3
        batch = a.shape[0] if batched else 1
        M, K = a.shape[-2:]
        N = b.shape[-1]
        assert b.shape[-2] == K
        c = np.empty((batch, M, N), np.int32)
        self.lib.orc_gemmlowp_core(_ptr(a), _signed(a), _ptr(b), _signed(b), _ptr(c), M, N, K, batch,
                                   int(b.ndim == 3), _i32(a_off), _i32(b_off))
        return c if batched else c[0]

    def reduce_rows(self, a):
        a = np.ascontiguousarray(a)
        out = np.empty(a.shape[0], np.int32)
        self.lib.orc_reduce_rows(_ptr(a), _signed(a), a.shape[0], a.shape[1], _ptr(out))
        return out

    def reduce_cols(self, b):
        b = np.ascontiguousarray(b)
        out = np.empty(b.shape[1], np.int32)
        self.lib.orc_reduce_cols(_ptr(b), _signed(b), b.shape[0], b.shape[1], _ptr(out))
        return out

    def offset_contribution(self, mm, K, colsum, rowsum, a_off, b_off):
        mm = np.ascontiguousarray(mm, dtype=np.int32).copy()
        M, N = mm.shape
        cs = _i32arr(colsum if colsum is not None else np.zeros(N))
        rs = _i32arr(rowsum if rowsum is not None else np.zeros(M))
        self.lib.orc_offset_contribution(_ptr(mm), M, N, K, _ptr(cs), _ptr(rs), _i32(a_off), _i32(b_off))
        return mm

    def output_stage(self, acc, bias, mult, shift, offset, lo, hi, out_dtype):
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        M, N = acc.shape
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = None if bias is None else _i32arr(bias)
        out = np.empty((M, N), out_dtype)
        if out.dtype == np.int16:  # QSYMM16 destination
            self.lib.orc_output_stage_s16(_ptr(acc), _ptr(bias), _ptr(out), M, N, _ptr(mult), _ptr(shift),
                                          int(mult.size), _i32(offset), _i32(lo), _i32(hi))
            return out
        self.lib.orc_output_stage(_ptr(acc), _ptr(bias), _ptr(out), _signed(out), M, N, _ptr(mult), _ptr(shift),
                                  int(mult.size), _i32(offset), _i32(lo), _i32(hi))
        return out

    def output_stage_int(self, acc, bias, mult, shift, offset, lo, hi, out_dtype):
        """QUANTIZE_DOWN (integer multiply) stage: ((acc + offset + bias) * mult) >> shift, clamp, saturate."""
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        M, N = acc.shape
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = None if bias is None else _i32arr(bias)
        out = np.empty((M, N), out_dtype)
        self.lib.orc_output_stage_int(_ptr(acc), _ptr(bias), _ptr(out), _signed(out), M, N, _ptr(mult), _ptr(shift),
                                      int(mult.size), _i32(offset), _i32(lo), _i32(hi))
        return out

    @staticmethod
    def dequantize_s32(acc, scale, previous=None):
        """Restates dequantize_s32 (arm_compute/core/QuantizationInfo.h:639-642) on an int32 array:
        float32(acc) * float32(scale), one rounding each; plus one float32 addition when accumulating."""
        r = np.asarray(acc, dtype=np.int32).astype(np.float32) * np.float32(scale)
        return r if previous is None else (np.asarray(previous, np.float32) + r).astype(np.float32)

    def gemmlowp_fused_int(self, a, b, bias, a_off, b_off, mult, shift, offset, lo, hi, out_dtype):
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        M, K = a.shape
        N = b.shape[1]
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = None if bias is None else _i32arr(bias)
        out = np.empty((M, N), out_dtype)
        self.lib.orc_gemmlowp_fused_int(_ptr(a), _signed(a), _ptr(b), _signed(b), _ptr(bias), _ptr(out), _signed(out),
                                        M, N, K, _i32(a_off), _i32(b_off), _ptr(mult), _ptr(shift), int(mult.size),
                                        _i32(offset), _i32(lo), _i32(hi))
        return out

    def gemmlowp_fused(self, a, b, bias, a_off, b_off, mult, shift, offset, lo, hi, out_dtype):
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        M, K = a.shape
        N = b.shape[1]
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = None if bias is None else _i32arr(bias)
        out = np.empty((M, N), out_dtype)
        self.lib.orc_gemmlowp_fused(_ptr(a), _signed(a), _ptr(b), _signed(b), _ptr(bias), _ptr(out), _signed(out), M,
                                    N, K, _i32(a_off), _i32(b_off), _ptr(mult), _ptr(shift), int(mult.size),
                                    _i32(offset), _i32(lo), _i32(hi))
        return out

    # convolution --------------------------------------------------------------------------------
    @staticmethod
    def conv_out_dims(W, H, kw, kh, sx, sy, pl, pr, pt, pb, dx=1, dy=1):
        """FLOOR rounding, as arm_compute::scaled_dimensions (src/core/Utils.cpp)."""
        wo = (W + pl + pr - (dx * (kw - 1) + 1)) // sx + 1
        ho = (H + pt + pb - (dy * (kh - 1) + 1)) // sy + 1
        return wo, ho

    def im2col_nhwc(self, src, kw, kh, sx, sy, pl, pr, pt, pb, pad_value, dx=1, dy=1, row_stride=None):
        src = np.ascontiguousarray(src)
        B, H, W, Cc = src.shape
        wo, ho = self.conv_out_dims(W, H, kw, kh, sx, sy, pl, pr, pt, pb, dx, dy)
        K = kh * kw * Cc
        rs = K if row_stride is None else row_stride
        dst = np.empty((B, ho * wo, rs), src.dtype)
        self.lib.orc_im2col_nhwc(_ptr(src), _ptr(dst), Cc, W, H, B, kw, kh, sx, sy, pl, pt, dx, dy, wo, ho,
                                 int(pad_value) & 0xFF, rs)
        return dst

    def weights_reshape_nhwc(self, w):
        w = np.ascontiguousarray(w)
        OFM, kh, kw, Cc = w.shape
        dst = np.empty((kh * kw * Cc, OFM), w.dtype)
        self.lib.orc_weights_reshape_nhwc(_ptr(w), _ptr(dst), Cc, kw, kh, OFM)
        return dst

    def conv2d_nhwc(self, src, weights, bias, stride, pad, in_zp, w_zp, mult, shift, out_offset, lo, hi,
                    dilation=(1, 1)):
        """src [B,H,W,C]; weights [OFM,kh,kw,C]; pad = (left, right, top, bottom); true zero points."""
        src = np.ascontiguousarray(src)
        weights = np.ascontiguousarray(weights)
        B, H, W, Cc = src.shape
        OFM, kh, kw, _ = weights.shape
        sx, sy = stride
        pl, pr, pt, pb = pad
        dx, dy = dilation
        wo, ho = self.conv_out_dims(W, H, kw, kh, sx, sy, pl, pr, pt, pb, dx, dy)
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = _i32arr(bias if bias is not None else np.zeros(OFM))
        dst = np.empty((B, ho, wo, OFM), src.dtype)
        self.lib.orc_conv2d_nhwc(_ptr(src), _signed(src), _ptr(weights), _signed(weights), _ptr(bias), _ptr(dst), Cc,
                                 W, H, B, kw, kh, OFM, sx, sy, pl, pt, dx, dy, wo, ho, _i32(in_zp), _i32(w_zp),
                                 _ptr(mult), _ptr(shift), int(mult.size), _i32(out_offset), _i32(lo), _i32(hi))
        return dst


class _Ref(_Layers):
    """Compute Library's own test oracle (tests/validation/reference), compiled in place."""
    _pfx = "ref_"

    def __init__(self):
        self.lib = C.CDLL(REF_SO)
        L = self.lib
        for name in ("ref_quantize_down_scalar", "ref_sqdmulh", "ref_rounding_divide_by_pow2"):
            getattr(L, name).restype = C.c_int
        L.ref_quantize_down_scalar.argtypes = [C.c_int] * 6
        L.ref_sqdmulh.argtypes = [C.c_int] * 2
        L.ref_rounding_divide_by_pow2.argtypes = [C.c_int] * 2
        L.ref_calculate_quantized_multiplier.restype = C.c_int
        L.ref_calculate_quantized_multiplier.argtypes = [C.c_float, _p, _p]

    def sqdmulh(self, a, b):
        return int(self.lib.ref_sqdmulh(a, b))

    def rounding_divide_by_pow2(self, x, e):
        return int(self.lib.ref_rounding_divide_by_pow2(x, e))

    def quantize_down(self, acc, mult, shift, offset, lo, hi):
        return int(self.lib.ref_quantize_down_scalar(acc, mult, shift, offset, lo, hi))

    def calculate_quantized_multiplier(self, multiplier: float):
        m, s = _i32(0), _i32(0)
        rc = self.lib.ref_calculate_quantized_multiplier(C.c_float(multiplier), C.byref(m), C.byref(s))
        if rc != 0:
            raise ValueError(f"multiplier {multiplier} cannot be quantised")
        return int(m.value), int(s.value)

    def gemmlowp_core(self, a, b, a_off, b_off):
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        batched = a.ndim == 3
        batch = a.shape[0] if batched else 1
        M, K = a.shape[-2:]
        N = b.shape[-1]
        key = ("u8" if a.dtype == np.uint8 else "s8") + ("u8" if b.dtype == np.uint8 else "s8")
        fn = getattr(self.lib, "ref_gemmlowp_core_" + key)  # s8u8 does not exist in the reference either
        c = np.empty((batch, M, N), np.int32)
        fn(_ptr(a), _ptr(b), _ptr(c), M, N, K, batch, int(b.ndim == 3), _i32(a_off), _i32(b_off))
        return c if batched else c[0]

    def output_stage(self, acc, bias, mult, shift, offset, lo, hi, out_dtype):
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        M, N = acc.shape
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = None if bias is None else _i32arr(bias)
        out = np.empty((M, N), out_dtype)
        fn = {np.dtype(np.int8): self.lib.ref_quantize_down_fixedpoint_s8,
              np.dtype(np.int16): self.lib.ref_quantize_down_fixedpoint_s16,
              np.dtype(np.uint8): self.lib.ref_quantize_down_fixedpoint_u8}[out.dtype]
        fn(_ptr(acc), _ptr(bias), _ptr(out), M, N, _ptr(mult), _ptr(shift), int(mult.size), _i32(offset), _i32(lo),
           _i32(hi))
        return out

    def output_stage_int(self, acc, bias, mult, shift, offset, lo, hi, out_dtype):
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        M, N = acc.shape
        mult, shift = _i32arr(mult), _i32arr(shift)
        bias = None if bias is None else _i32arr(bias)
        out = np.empty((M, N), out_dtype)
        fn = self.lib.ref_quantize_down_scale_s8 if out.dtype == np.int8 else self.lib.ref_quantize_down_scale_u8
        fn(_ptr(acc), _ptr(bias), _ptr(out), M, N, _ptr(mult), _ptr(shift), int(mult.size), _i32(offset), _i32(lo),
           _i32(hi))
        return out

    def dequantize_s32(self, acc, scale, previous=None):
        """The dequantised GEMMLowp output: float(acc) * scale, added to `previous` when given."""
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        out = np.zeros(acc.shape, np.float32) if previous is None else np.array(previous, dtype=np.float32, copy=True)
        self.lib.ref_dequantize_s32_f32(_ptr(acc), _ptr(out), C.c_longlong(acc.size), C.c_float(scale),
                                        0 if previous is None else 1)
        return out

    def conv_nchw(self, src, weights, bias, stride, pad, in_scale, in_zp, w_scales, w_zp, out_scale, out_zp):
        """src [B,C,H,W]; weights [OFM,C,kh,kw]; returns [B,OFM,Ho,Wo] (no activation, as the oracle)."""
        src = np.ascontiguousarray(src)
        weights = np.ascontiguousarray(weights)
        B, Cc, H, W = src.shape
        OFM, _, kh, kw = weights.shape
        sx, sy = stride
        pl, pr, pt, pb = pad
        wo, ho = _Port.conv_out_dims(W, H, kw, kh, sx, sy, pl, pr, pt, pb)
        ws = np.ascontiguousarray(np.atleast_1d(np.asarray(w_scales, dtype=np.float32)))
        key = ("u8" if src.dtype == np.uint8 else "s8") + ("u8" if weights.dtype == np.uint8 else "s8")
        fn = getattr(self.lib, "ref_conv_nchw_" + key)
        bias = _i32arr(bias)
        dst = np.empty((B, OFM, ho, wo), src.dtype)
        fn(_ptr(src), _ptr(weights), _ptr(bias), _ptr(dst), W, H, Cc, B, kw, kh, OFM, sx, sy, pl, pr, pt, pb,
           C.c_float(in_scale), C.c_int(in_zp), _ptr(ws), C.c_int(ws.size), C.c_int(w_zp), C.c_float(out_scale),
           C.c_int(out_zp))
        return dst

    def im2col_nhwc(self, src, kw, kh, sx, sy, pl, pr, pt, pb, zp):
        src = np.ascontiguousarray(src)
        assert src.dtype == np.uint8
        B, H, W, Cc = src.shape
        wo, ho = _Port.conv_out_dims(W, H, kw, kh, sx, sy, pl, pr, pt, pb)
        dst = np.empty((B, ho * wo, kh * kw * Cc), np.uint8)
        self.lib.ref_im2col_nhwc_u8(_ptr(src), _ptr(dst), Cc, W, H, B, kw, kh, sx, sy, pl, pr, pt, pb, C.c_int(zp))
        return dst


_port = None
_ref = None


def port() -> _Port:
    global _port
    if _port is None:
        _port = _Port()
    return _port


def ref():
    """The in-place reference oracle, or None when oracle/_ref/libacl_ref.so is absent."""
    global _ref
    if _ref is None and os.path.exists(REF_SO):
        _ref = _Ref()
    return _ref
