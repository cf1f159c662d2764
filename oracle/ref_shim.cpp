// TEST INFRASTRUCTURE ONLY — not part of the shipped library.
//
// C-ABI wrapper around Compute Library's own scalar test oracle, compiled IN PLACE from an
// unmodified Compute Library source tree (see oracle/Makefile, target `ref`).  No reference
// source is copied into this repository: this file only #includes the reference translation
// units so that template instantiations the reference does not export (e.g. the u8 x s8
// GEMMLowp core with non-zero offsets) can be requested here.
//
// Wrapped reference entry points:
//   reference::gemmlowp_matrix_multiply_core           tests/validation/reference/GEMMLowp.cpp:202-255
//   reference::gemmlowp_quantize_down_scale_by_fixedpoint  tests/validation/reference/GEMMLowp.cpp:106-158,309-340
//   reference::gemmlowp_quantize_down_scale            tests/validation/reference/GEMMLowp.cpp:66-104,278-307
//   reference::convolution_layer (NCHW)                tests/validation/reference/ConvolutionLayer.cpp:43-151
//   reference::im2col (NHWC / NCHW)                    tests/validation/reference/Im2Col.cpp:40-197
//   quantization::calculate_quantized_multiplier       src/core/utils/quantization/AsymmHelpers.cpp:43-91
//   validation::quantize_down_scale_by_fixedpoint      tests/validation/reference/UtilsQuantizedAsymm.h:69-89
#include "tests/validation/reference/GEMMLowp.cpp" // NOLINT: in-place inclusion on purpose

// ConvolutionLayer.cpp uses the test framework's ARM_COMPUTE_ASSERT on two loop indices; that macro
// would drag the whole test runner into the link.  Replace only the assertion mechanism.
#include "tests/framework/Asserts.h"
#undef ARM_COMPUTE_ASSERT
#define ARM_COMPUTE_ASSERT(X)                       \
    do                                              \
    {                                               \
        if (!(X))                                   \
        {                                           \
            throw std::runtime_error("assert: " #X); \
        }                                           \
    } while (false)
#include "tests/validation/reference/ConvolutionLayer.cpp" // NOLINT: in-place inclusion on purpose
#include "tests/validation/reference/Im2Col.h"
#include "arm_compute/core/utils/quantization/AsymmHelpers.h"

#include <cstring>
#include <vector>

using namespace arm_compute;
using namespace arm_compute::test;
using namespace arm_compute::test::validation;

namespace
{
template <typename T>
DataType dtype_of()
{
    return std::is_same<T, uint8_t>::value ? DataType::QASYMM8 : DataType::QASYMM8_SIGNED;
}

template <typename TA, typename TB>
void core(const void *a, const void *b, int32_t *c, int M, int N, int K, int batch, int b_batched, int a_off, int b_off)
{
    SimpleTensor<TA> ta(TensorShape(K, M, batch), dtype_of<TA>());
    SimpleTensor<TB> tb(b_batched ? TensorShape(N, K, batch) : TensorShape(N, K), dtype_of<TB>());
    std::memcpy(ta.data(), a, size_t(M) * K * batch);
    std::memcpy(tb.data(), b, size_t(N) * K * (b_batched ? batch : 1));
    SimpleTensor<int32_t> tc =
        reference::gemmlowp_matrix_multiply_core<int32_t, TA, TB>(ta, tb, TensorShape(N, M, batch), a_off, b_off);
    std::memcpy(c, tc.data(), size_t(M) * N * batch * sizeof(int32_t));
}

template <typename TO>
void qdown(const int32_t *in, const int32_t *bias, void *out, int M, int N, const int32_t *mult, const int32_t *shift,
           int n_mult, int offset, int lo, int hi)
{
    SimpleTensor<int32_t> tin(TensorShape(N, M), DataType::S32);
    std::memcpy(tin.data(), in, size_t(M) * N * sizeof(int32_t));
    std::vector<int32_t> vm(mult, mult + n_mult), vs(shift, shift + n_mult);
    SimpleTensor<TO>     dst;
    if (bias != nullptr)
    {
        SimpleTensor<int32_t> tb(TensorShape(N), DataType::S32);
        std::memcpy(tb.data(), bias, size_t(N) * sizeof(int32_t));
        dst = reference::gemmlowp_quantize_down_scale_by_fixedpoint<int32_t, TO>(tin, tb, vm, vs, offset, lo, hi);
    }
    else
    {
        dst = reference::gemmlowp_quantize_down_scale_by_fixedpoint<int32_t, TO>(tin, vm, vs, offset, lo, hi);
    }
    std::memcpy(out, dst.data(), size_t(M) * N * sizeof(TO));
}

template <typename TO>
void qdown_int(const int32_t *in, const int32_t *bias, void *out, int M, int N, const int32_t *mult, const int32_t *shift,
               int n_mult, int offset, int lo, int hi)
{
    SimpleTensor<int32_t> tin(TensorShape(N, M), DataType::S32);
    std::memcpy(tin.data(), in, size_t(M) * N * sizeof(int32_t));
    std::vector<int32_t> vm(mult, mult + n_mult), vs(shift, shift + n_mult);
    SimpleTensor<TO>     dst;
    if (bias != nullptr)
    {
        SimpleTensor<int32_t> tb(TensorShape(N), DataType::S32);
        std::memcpy(tb.data(), bias, size_t(N) * sizeof(int32_t));
        dst = reference::gemmlowp_quantize_down_scale<int32_t, TO>(tin, tb, offset, vm, vs, lo, hi);
    }
    else
    {
        dst = reference::gemmlowp_quantize_down_scale<int32_t, TO>(tin, offset, vm, vs, lo, hi);
    }
    std::memcpy(out, dst.data(), size_t(M) * N);
}

// NCHW convolution exactly as the conv fixture drives it: src [W,H,C,B], weights [kw,kh,C,OFM].
template <typename TI, typename TW>
void conv(const void *src, const void *wgt, const int32_t *bias, void *dst, int W, int H, int C, int B, int kw, int kh,
          int OFM, int sx, int sy, int pl, int pr, int pt, int pb, float in_scale, int in_zp, const float *w_scales,
          int n_w_scales, int w_zp, float out_scale, int out_zp)
{
    SimpleTensor<TI> ts(TensorShape(W, H, C, B), dtype_of<TI>(), 1, QuantizationInfo(in_scale, in_zp));
    QuantizationInfo wq;
    DataType         wdt = dtype_of<TW>();
    if (n_w_scales > 1)
    {
        wq  = QuantizationInfo(std::vector<float>(w_scales, w_scales + n_w_scales));
        wdt = DataType::QSYMM8_PER_CHANNEL;
    }
    else
    {
        wq = QuantizationInfo(w_scales[0], w_zp);
    }
    SimpleTensor<TW>      tw(TensorShape(kw, kh, C, OFM), wdt, 1, wq);
    SimpleTensor<int32_t> tb(TensorShape(OFM), DataType::S32);
    std::memcpy(ts.data(), src, size_t(W) * H * C * B);
    std::memcpy(tw.data(), wgt, size_t(kw) * kh * C * OFM);
    std::memcpy(tb.data(), bias, size_t(OFM) * sizeof(int32_t));
    PadStrideInfo info(sx, sy, pl, pr, pt, pb, DimensionRoundingType::FLOOR);
    auto          wh = scaled_dimensions(W, H, kw, kh, info, Size2D(1, 1));
    TensorShape   out_shape(wh.first, wh.second, OFM, B);
    SimpleTensor<TI> out = reference::convolution_layer<TI, TW, int32_t, TI>(ts, tw, tb, out_shape, info, Size2D(1, 1),
                                                                             1, QuantizationInfo(out_scale, out_zp));
    std::memcpy(dst, out.data(), out.size());
}
} // namespace

extern "C"
{
    // a: [batch][M][K], b: [K][N] (or [batch][K][N]), c: [batch][M][N]
    void ref_gemmlowp_core_u8u8(const uint8_t *a, const uint8_t *b, int32_t *c, int M, int N, int K, int batch,
                                int b_batched, int a_off, int b_off)
    {
        core<uint8_t, uint8_t>(a, b, c, M, N, K, batch, b_batched, a_off, b_off);
    }
    void ref_gemmlowp_core_s8s8(const int8_t *a, const int8_t *b, int32_t *c, int M, int N, int K, int batch,
                                int b_batched, int a_off, int b_off)
    {
        core<int8_t, int8_t>(a, b, c, M, N, K, batch, b_batched, a_off, b_off);
    }
    void ref_gemmlowp_core_u8s8(const uint8_t *a, const int8_t *b, int32_t *c, int M, int N, int K, int batch,
                                int b_batched, int a_off, int b_off)
    {
        core<uint8_t, int8_t>(a, b, c, M, N, K, batch, b_batched, a_off, b_off);
    }

    void ref_quantize_down_fixedpoint_u8(const int32_t *in, const int32_t *bias, uint8_t *out, int M, int N,
                                         const int32_t *mult, const int32_t *shift, int n_mult, int offset, int lo,
                                         int hi)
    {
        qdown<uint8_t>(in, bias, out, M, N, mult, shift, n_mult, offset, lo, hi);
    }
    void ref_quantize_down_fixedpoint_s8(const int32_t *in, const int32_t *bias, int8_t *out, int M, int N,
                                         const int32_t *mult, const int32_t *shift, int n_mult, int offset, int lo,
                                         int hi)
    {
        qdown<int8_t>(in, bias, out, M, N, mult, shift, n_mult, offset, lo, hi);
    }

    // QSYMM16 destination: the int16_t instantiation of the same reference template (GEMMLowp.cpp:423-436)
    void ref_quantize_down_fixedpoint_s16(const int32_t *in, const int32_t *bias, int16_t *out, int M, int N,
                                          const int32_t *mult, const int32_t *shift, int n_mult, int offset, int lo,
                                          int hi)
    {
        qdown<int16_t>(in, bias, out, M, N, mult, shift, n_mult, offset, lo, hi);
    }

    // reference::gemmlowp_quantize_down_scale (the QUANTIZE_DOWN integer stage), GEMMLowp.cpp:66-104, 278-307
    void ref_quantize_down_scale_u8(const int32_t *in, const int32_t *bias, uint8_t *out, int M, int N,
                                    const int32_t *mult, const int32_t *shift, int n_mult, int offset, int lo, int hi)
    {
        qdown_int<uint8_t>(in, bias, out, M, N, mult, shift, n_mult, offset, lo, hi);
    }
    void ref_quantize_down_scale_s8(const int32_t *in, const int32_t *bias, int8_t *out, int M, int N,
                                    const int32_t *mult, const int32_t *shift, int n_mult, int offset, int lo, int hi)
    {
        qdown_int<int8_t>(in, bias, out, M, N, mult, shift, n_mult, offset, lo, hi);
    }

    int ref_quantize_down_scalar(int val, int mult, int shift, int offset, int lo, int hi)
    {
        return quantize_down_scale_by_fixedpoint(val, mult, shift, offset, lo, hi);
    }
    int ref_sqdmulh(int a, int b)
    {
        return asymm_int_mult(a, b);
    }
    int ref_rounding_divide_by_pow2(int x, int e)
    {
        return asymm_rounding_divide_by_pow2(x, e);
    }

    int ref_calculate_quantized_multiplier(float multiplier, int32_t *qm, int32_t *shift)
    {
        Status s = quantization::calculate_quantized_multiplier(multiplier, qm, shift);
        return s.error_code() == ErrorCode::OK ? 0 : 1;
    }

    void ref_conv_nchw_u8u8(const uint8_t *src, const uint8_t *wgt, const int32_t *bias, uint8_t *dst, int W, int H,
                            int C, int B, int kw, int kh, int OFM, int sx, int sy, int pl, int pr, int pt, int pb,
                            float in_scale, int in_zp, const float *w_scales, int n_w_scales, int w_zp,
                            float out_scale, int out_zp)
    {
        conv<uint8_t, uint8_t>(src, wgt, bias, dst, W, H, C, B, kw, kh, OFM, sx, sy, pl, pr, pt, pb, in_scale, in_zp,
                               w_scales, n_w_scales, w_zp, out_scale, out_zp);
    }
    void ref_conv_nchw_u8s8(const uint8_t *src, const int8_t *wgt, const int32_t *bias, uint8_t *dst, int W, int H,
                            int C, int B, int kw, int kh, int OFM, int sx, int sy, int pl, int pr, int pt, int pb,
                            float in_scale, int in_zp, const float *w_scales, int n_w_scales, int w_zp,
                            float out_scale, int out_zp)
    {
        conv<uint8_t, int8_t>(src, wgt, bias, dst, W, H, C, B, kw, kh, OFM, sx, sy, pl, pr, pt, pb, in_scale, in_zp,
                              w_scales, n_w_scales, w_zp, out_scale, out_zp);
    }
    void ref_conv_nchw_s8s8(const int8_t *src, const int8_t *wgt, const int32_t *bias, int8_t *dst, int W, int H, int C,
                            int B, int kw, int kh, int OFM, int sx, int sy, int pl, int pr, int pt, int pb,
                            float in_scale, int in_zp, const float *w_scales, int n_w_scales, int w_zp,
                            float out_scale, int out_zp)
    {
        conv<int8_t, int8_t>(src, wgt, bias, dst, W, H, C, B, kw, kh, OFM, sx, sy, pl, pr, pt, pb, in_scale, in_zp,
                             w_scales, n_w_scales, w_zp, out_scale, out_zp);
    }

    // NHWC im2col of a QASYMM8 tensor: src [C,W,H,B] -> dst [kh*kw*C, Wo*Ho, B]; pad value = zero point.
    void ref_im2col_nhwc_u8(const uint8_t *src, uint8_t *dst, int C, int W, int H, int B, int kw, int kh, int sx,
                            int sy, int pl, int pr, int pt, int pb, int zp)
    {
        PadStrideInfo info(sx, sy, pl, pr, pt, pb, DimensionRoundingType::FLOOR);
        auto          wh = scaled_dimensions(W, H, kw, kh, info);
        SimpleTensor<uint8_t> ts(TensorShape(C, W, H, B), DataType::QASYMM8, 1, QuantizationInfo(1.f, zp),
                                 DataLayout::NHWC);
        SimpleTensor<uint8_t> td(TensorShape(kw * kh * C, wh.first * wh.second, B), DataType::QASYMM8, 1,
                                 QuantizationInfo(1.f, zp), DataLayout::NHWC);
        std::memcpy(ts.data(), src, ts.size());
        reference::im2col<uint8_t>(ts, td, Size2D(kw, kh), info, false, 1, 0);
        std::memcpy(dst, td.data(), td.size());
    }
}
