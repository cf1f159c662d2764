"""ctypes binding of include/cugl.h.  Every call goes through libcugl.so; a missing library or a missing
GPU raises -- nothing here computes on the CPU."""
from __future__ import annotations

import ctypes as C
import weakref
import os
import re

from . import build as _build

U8, S8, S32, S16, F32 = 0, 1, 2, 3, 4  # S16: QSYMM16 (stand-alone stage only); F32: dequantized GEMM output
STAGE_NONE, STAGE_QUANTIZE_DOWN, STAGE_FIXEDPOINT = 0, 1, 2
# cugl_status values the tests name
SUCCESS, RUNTIME_ERROR, INVALID_ARGUMENT = 0, 1, 6
INT32_MIN, INT32_MAX = -(2 ** 31), 2 ** 31 - 1

_vp = C.c_void_p
_i32 = C.c_int32
_i64 = C.c_int64
_pi32 = C.POINTER(C.c_int32)


class CuglError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"cugl status {status}: {message}")
        self.status = status
        self.message = message


class GemmDesc(C.Structure):
    """cugl_gemm_desc"""
    _fields_ = [
        ("M", _i32), ("N", _i32), ("K", _i32), ("batch", _i32),
        ("lda", _i64), ("ldb", _i64), ("ldd", _i64),
        ("a_batch_stride", _i64), ("b_batch_stride", _i64), ("d_batch_stride", _i64),
        ("a_dtype", _i32), ("b_dtype", _i32), ("dst_dtype", _i32),
        ("a_offset", _i32), ("b_offset", _i32),
        ("stage", _i32), ("is_quantized_per_channel", _i32),
        ("gemmlowp_multiplier", _i32), ("gemmlowp_shift", _i32),
        ("h_gemmlowp_multipliers", _pi32), ("h_gemmlowp_shifts", _pi32),
        ("gemmlowp_offset", _i32), ("gemmlowp_min_bound", _i32), ("gemmlowp_max_bound", _i32),
        ("has_bias", _i32), ("reshape_b_only_on_first_run", _i32),
        ("accumulate", _i32), ("dequantize_scale", C.c_float),
    ]


class ConvDesc(C.Structure):
    """cugl_conv_desc"""
    _fields_ = [
        ("B", _i32), ("H", _i32), ("W", _i32), ("C", _i32),
        ("OFM", _i32), ("kh", _i32), ("kw", _i32),
        ("stride_x", _i32), ("stride_y", _i32),
        ("pad_left", _i32), ("pad_right", _i32), ("pad_top", _i32), ("pad_bottom", _i32),
        ("dil_x", _i32), ("dil_y", _i32),
        ("src_dtype", _i32), ("w_dtype", _i32),
        ("src_zero_point", _i32), ("w_zero_point", _i32),
        ("is_quantized_per_channel", _i32),
        ("gemmlowp_multiplier", _i32), ("gemmlowp_shift", _i32),
        ("h_gemmlowp_multipliers", _pi32), ("h_gemmlowp_shifts", _pi32),
        ("dst_zero_point", _i32), ("min_bound", _i32), ("max_bound", _i32),
        ("has_bias", _i32),
    ]


class PoolDesc(C.Structure):
    """cugl_pool_desc"""
    _fields_ = [
        ("B", _i32), ("H", _i32), ("W", _i32), ("C", _i32),
        ("pool_type", _i32), ("pool_w", _i32), ("pool_h", _i32),
        ("stride_x", _i32), ("stride_y", _i32),
        ("pad_left", _i32), ("pad_right", _i32), ("pad_top", _i32), ("pad_bottom", _i32),
        ("exclude_padding", _i32), ("is_global", _i32),
        ("src_scale", C.c_float), ("src_zero_point", _i32),
        ("dst_scale", C.c_float), ("dst_zero_point", _i32),
    ]


POOL_MAX, POOL_AVG = 0, 1
ACT_NONE, ACT_RELU, ACT_BOUNDED_RELU, ACT_LU_BOUNDED_RELU = -1, 0, 1, 2

_SIGNATURES = {
    "cugl_context_create": (C.c_int, [C.c_int, _vp, C.POINTER(_vp)]),
    "cugl_context_destroy": (None, [_vp]),
    "cugl_last_error_string": (C.c_char_p, [_vp]),
    "cugl_context_stream": (_vp, [_vp]),
    "cugl_context_device": (C.c_int, [_vp]),
    "cugl_context_sm_count": (C.c_int, [_vp]),
    "cugl_context_set_trace_buffer": (C.c_int, [_vp, _vp]),
    "cugl_context_set_wait_limit_us": (C.c_int, [_vp, C.c_uint64]),
    "cugl_context_set_dependent_launch": (C.c_int, [_vp, C.c_int]),
    "cugl_context_withhold_copy_once": (C.c_int, [_vp, C.c_int]),
    "cugl_malloc": (C.c_int, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "cugl_free": (C.c_int, [_vp, _vp]),
    "cugl_host_alloc": (C.c_int, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "cugl_host_free": (C.c_int, [_vp, _vp]),
    "cugl_memcpy_h2d": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "cugl_memcpy_d2h": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "cugl_memcpy2d_h2d": (C.c_int, [_vp, _vp, C.c_size_t, _vp, C.c_size_t, C.c_size_t, C.c_size_t]),
    "cugl_memcpy2d_d2h": (C.c_int, [_vp, _vp, C.c_size_t, _vp, C.c_size_t, C.c_size_t, C.c_size_t]),
    "cugl_memset": (C.c_int, [_vp, _vp, C.c_int, C.c_size_t]),
    "cugl_sync": (C.c_int, [_vp]),
    "cugl_calculate_quantized_multiplier": (C.c_int, [C.c_float, _pi32, _pi32]),
    "cugl_calculate_quantized_multipliers": (C.c_int, [C.c_float, C.POINTER(C.c_float), C.c_int, C.c_float, _pi32,
                                                       _pi32]),
    "cugl_gemmlowp_validate": (C.c_int, [C.POINTER(GemmDesc), C.POINTER(C.c_char_p)]),
    "cugl_gemmlowp_plan_create": (C.c_int, [_vp, C.POINTER(GemmDesc), C.POINTER(_vp)]),
    "cugl_gemmlowp_plan_destroy": (None, [_vp]),
    "cugl_gemmlowp_prepare": (C.c_int, [_vp, _vp]),
    "cugl_gemmlowp_run": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "cugl_gemmlowp_run_host": (C.c_int, [_vp, _vp, _vp, _vp]),
    "cugl_gemmlowp_run_multi": (C.c_int, [_vp, _vp, _vp, C.POINTER(_vp), _i32]),
    "cugl_ipc_get_handle": (C.c_int, [_vp, _vp, _vp]),
    "cugl_ipc_open_handle": (C.c_int, [_vp, _vp, C.POINTER(_vp)]),
    "cugl_ipc_close_handle": (C.c_int, [_vp, _vp]),
    "cugl_gemmlowp_update_quantization": (C.c_int, [_vp, C.POINTER(GemmDesc)]),
    "cugl_gemmlowp_plan_kernel": (C.c_char_p, [_vp]),
    "cugl_gemmlowp_plan_force_simt": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_allow_pair_kernel": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_set_host_pipeline": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_launches": (C.c_int, [_vp]),
    "cugl_gemmlowp_run_noalloc": (C.c_int, [_vp, C.POINTER(GemmDesc), _vp, _vp, _vp, _vp, _vp, _vp]),
    "cugl_gemmlowp_noalloc_status": (C.c_int, [_vp]),
    "cugl_memcpy_d2d": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "cugl_gemmlowp_plan_set_saturating_pack": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_saturating_pack": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_temp_bytes": (C.c_size_t, [_vp]),
    "cugl_gemmlowp_plan_bind_temp": (C.c_int, [_vp, _vp, C.c_size_t]),
    "cugl_conv2d_update_quantization": (C.c_int, [_vp, C.POINTER(ConvDesc)]),
    "cugl_transpose_batched": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32]),
    "cugl_conv2d_plan_temp_bytes": (C.c_size_t, [_vp]),
    "cugl_conv2d_plan_bind_temp": (C.c_int, [_vp, _vp, C.c_size_t]),
    "cugl_reduce_rows": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i64, _i32, _vp]),
    "cugl_reduce_cols": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i64, _i32, _vp]),
    "cugl_offset_contribution": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i64, _vp, _vp, _i32, _i32]),
    "cugl_output_stage": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32,
                                    _i32, _i32, _i32]),
    "cugl_output_stage_quantize_down": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _i32, _i32,
                                                  _i32, _i32, _i32, _i32]),
    "cugl_im2col_nhwc": (C.c_int, [_vp, _vp, _vp] + [_i32] * 15 + [_i64]),
    "cugl_weights_reshape_nhwc": (C.c_int, [_vp, _vp, _vp, _i32, _i32]),
    "cugl_conv2d_validate": (C.c_int, [C.POINTER(ConvDesc), C.POINTER(C.c_char_p)]),
    "cugl_conv2d_plan_create": (C.c_int, [_vp, C.POINTER(ConvDesc), C.POINTER(_vp)]),
    "cugl_conv2d_plan_destroy": (None, [_vp]),
    "cugl_conv2d_prepare": (C.c_int, [_vp, _vp]),
    "cugl_conv2d_run": (C.c_int, [_vp, _vp, _vp, _vp]),
    "cugl_conv2d_run_host": (C.c_int, [_vp, _vp, _vp, _vp]),
    "cugl_conv2d_out_dims": (None, [C.POINTER(ConvDesc), _pi32, _pi32]),
    "cugl_conv2d_plan_launches": (C.c_int, [_vp]),
    "cugl_conv2d_plan_kernel": (C.c_char_p, [_vp]),
    "cugl_conv2d_plan_allow_implicit": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_allow_tma_im2col": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_uses_tma_im2col": (C.c_int, [_vp]),
    "cugl_conv2d_plan_set_epilogue_warps": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_tile_columns": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_paired_drain": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_tma_store": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_resident_weights": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_double_tile": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_set_tma_store": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_set_paired_drain": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_set_tile_columns": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_residual": (C.c_int, [_vp, C.c_float, C.c_float, _i32, C.c_float, _i32, _i32, C.c_float,
                                                C.c_float]),
    "cugl_conv2d_run_residual": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "cugl_gemmlowp_plan_set_epilogue_warps": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_set_channel_major": (C.c_int, [_vp, C.c_int]),
    "cugl_gemmlowp_plan_set_tail_split": (C.c_int, [_vp, C.c_int]),
    "cugl_conv2d_plan_set_channel_major": (C.c_int, [_vp, C.c_int]),
    "cugl_pool2d_out_dims": (None, [C.POINTER(PoolDesc), _pi32, _pi32]),
    "cugl_pool2d_validate": (C.c_int, [C.POINTER(PoolDesc)]),
    "cugl_pool2d_nhwc": (C.c_int, [_vp, C.POINTER(PoolDesc), _vp, _vp]),
    "cugl_add_qasymm8": (C.c_int, [_vp, _vp, _vp, _vp, _i64, C.c_float, _i32, C.c_float, _i32, C.c_float, _i32,
                                   _i32, C.c_float, C.c_float]),
    "cugl_activation_qasymm8": (C.c_int, [_vp, _vp, _vp, _i64, _i32, C.c_float, C.c_float, C.c_float, _i32,
                                          C.c_float, _i32]),
    "cugl_softmax_qasymm8": (C.c_int, [_vp, _vp, _vp, _i32, _i32, C.c_float, C.c_float, _i32]),
}

_lib = None


def header_symbols() -> list[str]:
    """Every function include/cugl.h declares (parsed from the header text)."""
    with open(os.path.join(_build.ROOT, "include", "cugl.h")) as f:
        text = f.read()
    return sorted(set(re.findall(r"CUGL_API[^;(]*?\b(cugl_\w+)\s*\(", text)))


def load_library(build_if_missing: bool = True) -> C.CDLL:
    """dlopen libcugl.so (building it first when the sources are newer) and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if build_if_missing:
        try:
            path = _build.build()
        except Exception:
            if not os.path.exists(path):
                raise
    if not os.path.exists(path):
        raise OSError(f"{path} is missing: run `python -m computelibrary_b200.build`")
    lib = C.CDLL(path)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def _check(status: int, ctx=None):
    if status != 0:
        msg = load_library().cugl_last_error_string(ctx)
        raise CuglError(status, msg.decode() if msg else "")


def calculate_quantized_multiplier(multiplier: float):
    m, s = _i32(0), _i32(0)
    _check(load_library().cugl_calculate_quantized_multiplier(C.c_float(multiplier), C.byref(m), C.byref(s)))
    return int(m.value), int(s.value)


def calculate_quantized_multipliers(i_scale: float, w_scales, o_scale: float):
    import numpy as np
    w = np.ascontiguousarray(np.asarray(w_scales, dtype=np.float32))
    m = np.zeros(w.size, np.int32)
    s = np.zeros(w.size, np.int32)
    _check(load_library().cugl_calculate_quantized_multipliers(
        C.c_float(i_scale), w.ctypes.data_as(C.POINTER(C.c_float)), int(w.size), C.c_float(o_scale),
        m.ctypes.data_as(_pi32), s.ctypes.data_as(_pi32)))
    return m, s


def _dptr(t):
    """Device pointer of a torch tensor / raw int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


class Context:
    """cugl_context on one device.  stream: raw cudaStream_t as an int (0 = the CUDA default stream, e.g.
    torch.cuda.current_stream().cuda_stream), or None to let the context create a stream of its own."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.lib = load_library()
        h = _vp()
        arg = _vp(-1 & (2 ** 64 - 1)) if stream is None else _vp(stream)  # CUGL_STREAM_CREATE
        _check(self.lib.cugl_context_create(device, arg, C.byref(h)))
        self._plans = weakref.WeakSet()  # live GemmPlan / ConvPlan objects of this context, see close()
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            # plans hold a pointer to the context: destroy the ones still alive first, whatever order the garbage
            # collector would have picked
            for plan in list(getattr(self, "_plans", ())):
                plan.close()
            self.lib.cugl_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, status: int):
        _check(status, self.handle)

    def set_trace_buffer(self, buf):
        self.check(self.lib.cugl_context_set_trace_buffer(self.handle, _dptr(buf)))

    def set_dependent_launch(self, on: bool = True):
        """Programmatic stream serialization of the tensor-core kernels (on by default)."""
        self.check(self.lib.cugl_context_set_dependent_launch(self.handle, int(on)))

    def set_wait_limit_us(self, microseconds: int):
        """Bound of every device-side barrier wait of the tensor-core kernels (0: the two-second default)."""
        self.check(self.lib.cugl_context_set_wait_limit_us(self.handle, int(microseconds)))

    def withhold_copy_once(self, k_block: int):
        """Test instrument: the next tensor-core GEMM launch leaves out one operand copy in CTA 0."""
        self.check(self.lib.cugl_context_withhold_copy_once(self.handle, int(k_block)))

    def sync(self):
        self.check(self.lib.cugl_sync(self.handle))

    @property
    def sm_count(self) -> int:
        return self.lib.cugl_context_sm_count(self.handle)

    @property
    def stream(self) -> int:
        return self.lib.cugl_context_stream(self.handle) or 0

    # memory -------------------------------------------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        p = _vp()
        self.check(self.lib.cugl_malloc(self.handle, nbytes, C.byref(p)))
        return p.value or 0

    def free(self, ptr: int):
        self.check(self.lib.cugl_free(self.handle, _vp(ptr)))

    def host_alloc(self, nbytes: int) -> int:
        p = _vp()
        self.check(self.lib.cugl_host_alloc(self.handle, nbytes, C.byref(p)))
        return p.value or 0

    def host_free(self, ptr: int):
        self.check(self.lib.cugl_host_free(self.handle, _vp(ptr)))

    def h2d(self, d_ptr: int, h_ptr: int, nbytes: int):
        self.check(self.lib.cugl_memcpy_h2d(self.handle, _vp(d_ptr), _vp(h_ptr), nbytes))

    def d2h(self, h_ptr: int, d_ptr: int, nbytes: int):
        self.check(self.lib.cugl_memcpy_d2h(self.handle, _vp(h_ptr), _vp(d_ptr), nbytes))

    def ipc_get_handle(self, d_ptr: int) -> bytes:
        buf = C.create_string_buffer(64)
        self.check(self.lib.cugl_ipc_get_handle(self.handle, _vp(d_ptr), buf))
        return buf.raw

    def ipc_open_handle(self, handle: bytes) -> int:
        p = _vp()
        self.check(self.lib.cugl_ipc_open_handle(self.handle, C.create_string_buffer(handle, 64), C.byref(p)))
        return p.value or 0

    def ipc_close_handle(self, d_ptr: int):
        self.check(self.lib.cugl_ipc_close_handle(self.handle, _vp(d_ptr)))

    # stand-alone kernels --------------------------------------------------------------------------
    def reduce_rows(self, a, dtype, M, K, lda, out, scalar=1):
        self.check(self.lib.cugl_reduce_rows(self.handle, _dptr(a), dtype, M, K, lda, scalar, _dptr(out)))

    def reduce_cols(self, b, dtype, K, N, ldb, out, scalar=1):
        self.check(self.lib.cugl_reduce_cols(self.handle, _dptr(b), dtype, K, N, ldb, scalar, _dptr(out)))

    def offset_contribution(self, mm, M, N, K, ld_bytes, colsum, rowsum, a_off, b_off):
        self.check(self.lib.cugl_offset_contribution(self.handle, _dptr(mm), M, N, K, ld_bytes, _dptr(colsum),
                                                     _dptr(rowsum), a_off, b_off))

    def output_stage(self, src, ld_in, bias, out, ld_out, out_dtype, M, N, mults, shifts, mult, shift, n_mult,
                     offset, lo, hi):
        self.check(self.lib.cugl_output_stage(self.handle, _dptr(src), ld_in, _dptr(bias), _dptr(out), ld_out,
                                              out_dtype, M, N, _dptr(mults), _dptr(shifts), mult, shift, n_mult,
                                              offset, lo, hi))

    def output_stage_quantize_down(self, src, ld_in, bias, out, ld_out, out_dtype, M, N, mults, shifts, mult, shift,
                                   n_mult, offset, lo, hi):
        self.check(self.lib.cugl_output_stage_quantize_down(self.handle, _dptr(src), ld_in, _dptr(bias), _dptr(out),
                                                            ld_out, out_dtype, M, N, _dptr(mults), _dptr(shifts), mult,
                                                            shift, n_mult, offset, lo, hi))

    def im2col_nhwc(self, src, dst, C_, W, H, B, kw, kh, sx, sy, pl, pt, dx, dy, Wo, Ho, pad_value, row_stride):
        self.check(self.lib.cugl_im2col_nhwc(self.handle, _dptr(src), _dptr(dst), C_, W, H, B, kw, kh, sx, sy, pl, pt,
                                             dx, dy, Wo, Ho, pad_value, row_stride))

    # QASYMM8 layers: q = (scale, zero point) -------------------------------------------------------------
    def pool2d_nhwc(self, desc: "PoolDesc", src, dst):
        self.check(self.lib.cugl_pool2d_nhwc(self.handle, C.byref(desc), _dptr(src), _dptr(dst)))

    def add_qasymm8(self, a, b, dst, n, a_q, b_q, o_q, act=ACT_NONE, act_a=0.0, act_b=0.0):
        self.check(self.lib.cugl_add_qasymm8(self.handle, _dptr(a), _dptr(b), _dptr(dst), n, a_q[0], a_q[1], b_q[0],
                                             b_q[1], o_q[0], o_q[1], act, act_a, act_b))

    def activation_qasymm8(self, src, dst, n, act, act_a, act_b, in_q, out_q):
        self.check(self.lib.cugl_activation_qasymm8(self.handle, _dptr(src), _dptr(dst), n, act, act_a, act_b,
                                                    in_q[0], in_q[1], out_q[0], out_q[1]))

    def softmax_qasymm8(self, src, dst, rows, cols, beta, in_q):
        self.check(self.lib.cugl_softmax_qasymm8(self.handle, _dptr(src), _dptr(dst), rows, cols, beta, in_q[0],
                                                 in_q[1]))

    def transpose_batched(self, src, dst, rows, cols, batch):
        self.check(self.lib.cugl_transpose_batched(self.handle, _dptr(src), _dptr(dst), rows, cols, batch))

    def weights_reshape_nhwc(self, w, dst, K, OFM):
        self.check(self.lib.cugl_weights_reshape_nhwc(self.handle, _dptr(w), _dptr(dst), K, OFM))


def make_gemm_desc(M, N, K, a_dtype, b_dtype, dst_dtype, a_offset=0, b_offset=0, stage=STAGE_FIXEDPOINT,
                   multiplier=0, shift=0, multipliers=None, shifts=None, offset=0, min_bound=INT32_MIN,
                   max_bound=INT32_MAX, has_bias=False, batch=1, lda=None, ldb=None, ldd=None,
                   a_batch_stride=None, b_batch_stride=0, d_batch_stride=None, b_constant=True, accumulate=False,
                   dequantize_scale=0.0):
    """Fill a cugl_gemm_desc for dense row-major operands unless strides are given.  Returns
    (desc, keepalive) -- keepalive holds the numpy arrays the descriptor points into."""
    import numpy as np
    dsz = 4 if dst_dtype in (S32, F32) else 1
    d = GemmDesc()
    d.M, d.N, d.K, d.batch = M, N, K, batch
    d.lda = K if lda is None else lda
    d.ldb = N if ldb is None else ldb
    d.ldd = N * dsz if ldd is None else ldd
    d.a_batch_stride = d.lda * M if a_batch_stride is None else a_batch_stride
    d.b_batch_stride = b_batch_stride
    d.d_batch_stride = d.ldd * M if d_batch_stride is None else d_batch_stride
    d.a_dtype, d.b_dtype, d.dst_dtype = a_dtype, b_dtype, dst_dtype
    d.a_offset, d.b_offset = a_offset, b_offset
    d.stage = stage
    keep = []
    if multipliers is not None:
        m = np.ascontiguousarray(np.asarray(multipliers, dtype=np.int32))
        s = np.ascontiguousarray(np.asarray(shifts, dtype=np.int32))
        keep += [m, s]
        d.is_quantized_per_channel = 1
        d.h_gemmlowp_multipliers = m.ctypes.data_as(_pi32)
        d.h_gemmlowp_shifts = s.ctypes.data_as(_pi32)
        d.gemmlowp_multiplier, d.gemmlowp_shift = int(m[0]), int(s[0])
    else:
        d.is_quantized_per_channel = 0
        d.gemmlowp_multiplier, d.gemmlowp_shift = multiplier, shift
    d.gemmlowp_offset = offset
    d.gemmlowp_min_bound, d.gemmlowp_max_bound = min_bound, max_bound
    d.has_bias = int(has_bias)
    d.reshape_b_only_on_first_run = int(b_constant)
    d.accumulate = int(accumulate)
    d.dequantize_scale = float(dequantize_scale)
    return d, keep


def gemmlowp_run_noalloc(stream: int, desc: GemmDesc, a, b, bias, multipliers, shifts, dst):
    """cugl_gemmlowp_run_noalloc: one fused GEMMLowp on `stream` using the library's fixed workspace."""
    _check(load_library().cugl_gemmlowp_run_noalloc(_vp(stream) if stream else None, C.byref(desc), _dptr(a), _dptr(b),
                                                   _dptr(bias), _dptr(multipliers), _dptr(shifts), _dptr(dst)))


def gemmlowp_noalloc_status(stream: int):
    """cugl_gemmlowp_noalloc_status: waits for `stream`; raises CuglError if an allocation-free call timed out."""
    _check(load_library().cugl_gemmlowp_noalloc_status(_vp(stream) if stream else None))


def gemm_validate(desc: GemmDesc):
    """Returns (status, reason)."""
    why = C.c_char_p()
    st = load_library().cugl_gemmlowp_validate(C.byref(desc), C.byref(why))
    return st, (why.value or b"").decode()


def make_pool_desc(B, H, W, C_, pool_type, size=(1, 1), stride=(1, 1), pad=(0, 0, 0, 0), in_q=(1.0, 0),
                   out_q=(1.0, 0), exclude_padding=False, global_pool=False) -> PoolDesc:
    """pad = (left, right, top, bottom); size = (width, height); q = (scale, zero point)."""
    d = PoolDesc()
    d.B, d.H, d.W, d.C = B, H, W, C_
    d.pool_type = pool_type
    d.pool_w, d.pool_h = size
    d.stride_x, d.stride_y = stride
    d.pad_left, d.pad_right, d.pad_top, d.pad_bottom = pad
    d.exclude_padding, d.is_global = int(exclude_padding), int(global_pool)
    d.src_scale, d.src_zero_point = in_q
    d.dst_scale, d.dst_zero_point = out_q
    return d


def pool_out_dims(desc: PoolDesc):
    wo, ho = _i32(0), _i32(0)
    load_library().cugl_pool2d_out_dims(C.byref(desc), C.byref(wo), C.byref(ho))
    return int(wo.value), int(ho.value)


def pool_validate(desc: PoolDesc):
    lib = load_library()
    st = lib.cugl_pool2d_validate(C.byref(desc))
    if st != 0:
        raise CuglError(st, (lib.cugl_last_error_string(None) or b"").decode())


def conv_validate(desc: ConvDesc):
    why = C.c_char_p()
    st = load_library().cugl_conv2d_validate(C.byref(desc), C.byref(why))
    return st, (why.value or b"").decode()


class GemmPlan:
    """cugl_gemm_plan: a configured NEGEMMLowpMatrixMultiplyCore."""

    def __init__(self, ctx: Context, desc: GemmDesc, keepalive=None):
        self.ctx = ctx
        self.desc = desc
        self._keep = keepalive
        h = _vp()
        ctx.check(ctx.lib.cugl_gemmlowp_plan_create(ctx.handle, C.byref(desc), C.byref(h)))
        self.handle = h
        ctx._plans.add(self)

    def close(self):
        if getattr(self, "handle", None):
            self.ctx.lib.cugl_gemmlowp_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prepare(self, b):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_prepare(self.handle, _dptr(b)))

    def run(self, a, b, bias, dst):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_run(self.handle, _dptr(a), _dptr(b), _dptr(bias), _dptr(dst)))

    def run_multi(self, a, bias, dsts):
        """dsts: device pointers (ints / tensors) of every destination matrix, this GPU's own first."""
        arr = (_vp * len(dsts))(*[_dptr(d) for d in dsts])
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_run_multi(self.handle, _dptr(a), _dptr(bias), arr, len(dsts)))

    def run_host(self, h_a: int, h_bias, h_dst: int):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_run_host(self.handle, _vp(h_a), _vp(h_bias) if h_bias else None,
                                                           _vp(h_dst)))

    def update_quantization(self, desc: GemmDesc, keepalive=None):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_update_quantization(self.handle, C.byref(desc)))
        self.desc, self._keep = desc, keepalive

    def force_simt(self, on: bool = True):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_force_simt(self.handle, int(on)))

    def set_epilogue_warps(self, warps: int):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_epilogue_warps(self.handle, int(warps)))

    def set_tile_columns(self, columns: int):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_tile_columns(self.handle, int(columns)))

    def set_saturating_pack(self, on: bool = True):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_saturating_pack(self.handle, int(on)))

    def set_paired_drain(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_paired_drain(self.handle, int(on)))

    def set_tma_store(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_tma_store(self.handle, int(on)))

    def set_channel_major(self, mode: int):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_channel_major(self.handle, int(mode)))

    def set_tail_split(self, on: bool = True):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_tail_split(self.handle, int(on)))

    def set_host_pipeline(self, blocks: int):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_set_host_pipeline(self.handle, int(blocks)))

    def allow_pair_kernel(self, on: bool = True):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_allow_pair_kernel(self.handle, int(on)))

    @property
    def temp_bytes(self) -> int:
        return int(self.ctx.lib.cugl_gemmlowp_plan_temp_bytes(self.handle))

    def bind_temp(self, ws, nbytes: int):
        self.ctx.check(self.ctx.lib.cugl_gemmlowp_plan_bind_temp(self.handle, _dptr(ws), nbytes))

    @property
    def kernel(self) -> str:
        return self.ctx.lib.cugl_gemmlowp_plan_kernel(self.handle).decode()

    @property
    def launches(self) -> int:
        return self.ctx.lib.cugl_gemmlowp_plan_launches(self.handle)


def make_conv_desc(B, H, W, C_, OFM, kh, kw, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1), src_dtype=U8,
                   w_dtype=S8, src_zp=0, w_zp=0, multiplier=0, shift=0, multipliers=None, shifts=None, dst_zp=0,
                   min_bound=INT32_MIN, max_bound=INT32_MAX, has_bias=True):
    """pad = (left, right, top, bottom); stride / dilation = (x, y).  Returns (desc, keepalive)."""
    import numpy as np
    d = ConvDesc()
    d.B, d.H, d.W, d.C = B, H, W, C_
    d.OFM, d.kh, d.kw = OFM, kh, kw
    d.stride_x, d.stride_y = stride
    d.pad_left, d.pad_right, d.pad_top, d.pad_bottom = pad
    d.dil_x, d.dil_y = dilation
    d.src_dtype, d.w_dtype = src_dtype, w_dtype
    d.src_zero_point, d.w_zero_point = src_zp, w_zp
    keep = []
    if multipliers is not None:
        m = np.ascontiguousarray(np.asarray(multipliers, dtype=np.int32))
        s = np.ascontiguousarray(np.asarray(shifts, dtype=np.int32))
        keep += [m, s]
        d.is_quantized_per_channel = 1
        d.h_gemmlowp_multipliers = m.ctypes.data_as(_pi32)
        d.h_gemmlowp_shifts = s.ctypes.data_as(_pi32)
        d.gemmlowp_multiplier, d.gemmlowp_shift = int(m[0]), int(s[0])
    else:
        d.gemmlowp_multiplier, d.gemmlowp_shift = multiplier, shift
    d.dst_zero_point = dst_zp
    d.min_bound, d.max_bound = min_bound, max_bound
    d.has_bias = int(has_bias)
    return d, keep


class ConvPlan:
    """cugl_conv_plan: a configured NEGEMMConvolutionLayer (NHWC, 8-bit)."""

    def __init__(self, ctx: Context, desc: ConvDesc, keepalive=None):
        self.ctx = ctx
        self.desc = desc
        self._keep = keepalive
        h = _vp()
        ctx.check(ctx.lib.cugl_conv2d_plan_create(ctx.handle, C.byref(desc), C.byref(h)))
        self.handle = h
        ctx._plans.add(self)

    def close(self):
        if getattr(self, "handle", None):
            self.ctx.lib.cugl_conv2d_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def out_dims(self):
        wo, ho = _i32(0), _i32(0)
        self.ctx.lib.cugl_conv2d_out_dims(C.byref(self.desc), C.byref(wo), C.byref(ho))
        return int(wo.value), int(ho.value)

    def prepare(self, weights):
        self.ctx.check(self.ctx.lib.cugl_conv2d_prepare(self.handle, _dptr(weights)))

    def run(self, src, bias, dst):
        self.ctx.check(self.ctx.lib.cugl_conv2d_run(self.handle, _dptr(src), _dptr(bias), _dptr(dst)))

    def update_quantization(self, desc: "ConvDesc", keepalive=None):
        self.ctx.check(self.ctx.lib.cugl_conv2d_update_quantization(self.handle, C.byref(desc)))
        self.desc, self._keep = desc, keepalive

    def set_residual(self, conv_out_scale, res_q, dst_q, act=ACT_NONE, act_a=0.0, act_b=0.0):
        """Configure the fused residual addition; raises CuglError (UNSUPPORTED_CONFIG) when the addition is not a
        saturating byte addition for these quantizations."""
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_residual(self.handle, conv_out_scale, res_q[0], res_q[1],
                                                                  dst_q[0], dst_q[1], act, act_a, act_b))

    def run_residual(self, src, bias, residual, dst):
        self.ctx.check(self.ctx.lib.cugl_conv2d_run_residual(self.handle, _dptr(src), _dptr(bias), _dptr(residual),
                                                             _dptr(dst)))

    def run_host(self, h_src: int, h_bias, h_dst: int):
        self.ctx.check(self.ctx.lib.cugl_conv2d_run_host(self.handle, _vp(h_src), _vp(h_bias) if h_bias else None,
                                                         _vp(h_dst)))

    def set_epilogue_warps(self, warps: int):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_epilogue_warps(self.handle, int(warps)))

    def set_tile_columns(self, columns: int):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_tile_columns(self.handle, int(columns)))

    def set_saturating_pack(self, on: bool = True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_saturating_pack(self.handle, int(on)))

    def set_paired_drain(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_paired_drain(self.handle, int(on)))

    def set_tma_store(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_tma_store(self.handle, int(on)))

    def set_resident_weights(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_resident_weights(self.handle, int(on)))

    def set_double_tile(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_double_tile(self.handle, int(on)))

    def set_channel_major(self, mode: int):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_set_channel_major(self.handle, int(mode)))

    def allow_implicit(self, on: bool = True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_allow_implicit(self.handle, int(on)))

    def allow_tma_im2col(self, on=True):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_allow_tma_im2col(self.handle, int(on)))

    @property
    def uses_tma_im2col(self) -> bool:
        return bool(self.ctx.lib.cugl_conv2d_plan_uses_tma_im2col(self.handle))

    @property
    def temp_bytes(self) -> int:
        return int(self.ctx.lib.cugl_conv2d_plan_temp_bytes(self.handle))

    def bind_temp(self, ws, nbytes: int):
        self.ctx.check(self.ctx.lib.cugl_conv2d_plan_bind_temp(self.handle, _dptr(ws), nbytes))

    @property
    def kernel(self) -> str:
        return self.ctx.lib.cugl_conv2d_plan_kernel(self.handle).decode()

    @property
    def launches(self) -> int:
        return self.ctx.lib.cugl_conv2d_plan_launches(self.handle)
