/*
 * TEST INFRASTRUCTURE ONLY -- not part of the shipped library, never linked into libcugl.so.
 *
 * Plain-C restatement of the QASYMM8 layers that sit between the convolutions of a quantized network
 * (pooling, element-wise addition, ReLU-family activation, softmax), as Compute Library's scalar test
 * oracle states them: dequantize to float, apply the float operator, quantize.  Every function cites the
 * reference file it follows (paths relative to the Compute Library tree).  The float operations are
 * written in the reference's own evaluation order and this file is compiled with -ffp-contract=off, so the
 * results are bit-identical to the reference oracle; tests/test_oracle_layers.py pins that against
 * oracle/_ref/libacl_ref.so (the reference's own code compiled in place) and against the committed
 * fixtures of tests/golden/layers_golden.npz.  Softmax depends on the C library's expf and is pinned
 * within +-1 (the tolerance the reference's own quantized softmax tests use).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_EXPORT __attribute__((visibility("default")))

/* arm_compute/core/QuantizationInfo.h:342-345 (dequantize): (int(value) - offset) * scale, in float */
static inline float deq_u8(uint8_t v, float scale, int zp)
{
    return (float)((int)v - zp) * scale;
}

/* arm_compute/core/QuantizationInfo.h:268-273 (quantize, TO_NEAREST_UP): lround(value / scale) + offset,
 * clamped to the type range; lround rounds halves away from zero. */
static inline uint8_t quant_u8(float v, float scale, int zp)
{
    long q = lroundf(v / scale) + zp;
    if (q < 0) q = 0;
    if (q > 255) q = 255;
    return (uint8_t)q;
}

/* reference::pooling_layer<uint8_t>: tests/validation/reference/PoolingLayer.cpp:218-230 (dequantize, float
 * pooling, quantize with the output quantization) around pooling_layer_internal<float>, :40-196.
 * MAX (:78-134): window clipped to the image, strict '>' against lowest(); AVG (:137-172): sum in window
 * order (y outer, x inner), divided by the window area including or excluding the padding.
 * Layout here: src [B][H][W][C], dst [B][Ho][Wo][C]; the caller supplies Wo, Ho.  pool_type 0 = MAX, 1 = AVG. */
ORC_EXPORT void orc_pool_nhwc_u8(const uint8_t *src, uint8_t *dst, int C, int W, int H, int B, int pool_type, int pw,
                                 int ph, int sx, int sy, int pl, int pr, int pt, int pb, int exclude_padding, int Wo,
                                 int Ho, float in_scale, int in_zp, float out_scale, int out_zp)
{
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
    {
        for (int h = 0; h < Ho; ++h)
        {
            for (int w = 0; w < Wo; ++w)
            {
                for (int c = 0; c < C; ++c)
                {
                    int   wstart = w * sx - pl;
                    int   hstart = h * sy - pt;
                    float res;
                    if (pool_type == 0)
                    {
                        int wend = wstart + pw < W ? wstart + pw : W;
                        int hend = hstart + ph < H ? hstart + ph : H;
                        if (wstart < 0) wstart = 0;
                        if (hstart < 0) hstart = 0;
                        float max_val = -3.402823466e+38f; /* numeric_limits<float>::lowest() */
                        for (int y = hstart; y < hend; ++y)
                        {
                            for (int x = wstart; x < wend; ++x)
                            {
                                const float v = deq_u8(src[(((size_t)b * H + y) * W + x) * C + c], in_scale, in_zp);
                                if (v > max_val) max_val = v;
                            }
                        }
                        res = max_val;
                    }
                    else
                    {
                        int wend = wstart + pw < W + pr ? wstart + pw : W + pr;
                        int hend = hstart + ph < H + pb ? hstart + ph : H + pb;
                        int pool = (hend - hstart) * (wend - wstart);
                        if (wstart < 0) wstart = 0;
                        if (hstart < 0) hstart = 0;
                        if (wend > W) wend = W;
                        if (hend > H) hend = H;
                        if (exclude_padding) pool = (hend - hstart) * (wend - wstart);
                        float avg = 0.f;
                        for (int y = hstart; y < hend; ++y)
                        {
                            for (int x = wstart; x < wend; ++x)
                            {
                                avg += deq_u8(src[(((size_t)b * H + y) * W + x) * C + c], in_scale, in_zp);
                            }
                        }
                        res = avg / (float)pool;
                    }
                    dst[(((size_t)b * Ho + h) * Wo + w) * C + c] = quant_u8(res, out_scale, out_zp);
                }
            }
        }
    }
}

/* reference::arithmetic_operation<uint8_t>(ADD): tests/validation/reference/ArithmeticOperations.cpp:124-151
 * with arithm_op<float> (:40-53): the two dequantized values are added in double and cast to float (one
 * rounding, the same value as a float addition), then quantized with the output quantization. */
ORC_EXPORT void orc_add_qasymm8(const uint8_t *a, const uint8_t *b, uint8_t *dst, long long n, float a_scale,
                                int a_zp, float b_scale, int b_zp, float o_scale, int o_zp)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i)
    {
        const double s = (double)deq_u8(a[i], a_scale, a_zp) + (double)deq_u8(b[i], b_scale, b_zp);
        dst[i]         = quant_u8((float)s, o_scale, o_zp);
    }
}

/* reference::activation_layer<uint8_t>: tests/validation/reference/ActivationLayer.cpp:61-71 with
 * activate_float (ActivationLayer.h:54-62).  act: 0 RELU max(0,x); 1 BOUNDED_RELU min(a, max(0,x));
 * 2 LU_BOUNDED_RELU min(a, max(b,x)). */
ORC_EXPORT void orc_activation_qasymm8(const uint8_t *src, uint8_t *dst, long long n, int act, float a, float b,
                                       float in_scale, int in_zp, float out_scale, int out_zp)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i)
    {
        const float x = deq_u8(src[i], in_scale, in_zp);
        float       r;
        if (act == 0)
        {
            r = x > 0.f ? x : 0.f;
        }
        else if (act == 1)
        {
            const float t = x > 0.f ? x : 0.f;
            r             = t < a ? t : a;
        }
        else
        {
            const float t = x > b ? x : b;
            r             = t < a ? t : a;
        }
        dst[i] = quant_u8(r, out_scale, out_zp);
    }
}

/* reference::softmax_layer<uint8_t>: tests/validation/reference/SoftmaxLayer.cpp:201-213 around
 * softmax_layer_generic<float> (:39-107): row maximum, exp((x - max) * beta) summed in index order,
 * division by the sum; output quantization fixed at (1/256, 0) (src/core/Utils.cpp:421-439). */
ORC_EXPORT void orc_softmax_qasymm8(const uint8_t *src, uint8_t *dst, int rows, int cols, float beta, float in_scale,
                                    int in_zp)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
    {
        const uint8_t *s = src + (size_t)r * cols;
        uint8_t       *d = dst + (size_t)r * cols;
        float         *e = (float *)malloc(sizeof(float) * (size_t)cols);
        float          m = deq_u8(s[0], in_scale, in_zp);
        for (int i = 1; i < cols; ++i)
        {
            const float v = deq_u8(s[i], in_scale, in_zp);
            if (v > m) m = v;
        }
        float sum = 0.f;
        for (int i = 0; i < cols; ++i)
        {
            e[i] = expf((deq_u8(s[i], in_scale, in_zp) - m) * beta);
            sum += e[i];
        }
        for (int i = 0; i < cols; ++i)
        {
            d[i] = quant_u8(e[i] / sum, 1.f / 256.f, 0);
        }
        free(e);
    }
}
