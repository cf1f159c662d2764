/*
 * TEST INFRASTRUCTURE ONLY -- not part of the shipped library, never linked into libcugl.so.
 *
 * Plain-C restatement of Compute Library's quantized GEMM hot path, written from the algorithm the
 * reference states in the files cited on each function (paths relative to the Compute Library tree).
 * It is pinned two ways by the CPU test-suite:
 *   - against the known-answer values of tests/golden/known_answers.json, produced by the
 *     reference's own UtilsQuantizedAsymm.h / AsymmHelpers.cpp;
 *   - against the reference's own scalar test oracle compiled in place (oracle/_ref/libacl_ref.so,
 *     built by `make -C oracle ref`) on the reference's small / large GEMMLowp dataset shapes and on
 *     small convolution shapes, plus golden fixtures generated from that library.
 *
 * All arithmetic is two's-complement int32 with wrap-around (computed through uint32_t so that the C
 * code has no undefined behaviour where the reference would overflow).
 */
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

static inline int32_t wrap_add(int32_t a, int32_t b)
{
    return (int32_t)((uint32_t)a + (uint32_t)b);
}
static inline int32_t wrap_mul(int32_t a, int32_t b)
{
    return (int32_t)((uint32_t)a * (uint32_t)b);
}

/* SQDMULH: doubling multiply, high half, NOT rounded; saturates only for INT32_MIN * INT32_MIN.
 * tests/validation/reference/UtilsQuantizedAsymm.h:60-67 (asymm_int_mult);
 * src/core/utils/quantization/AsymmHelpers.cpp:247-254. */
ORC_EXPORT int32_t orc_sqdmulh(int32_t a, int32_t b)
{
    if (a == INT32_MIN && b == INT32_MIN)
    {
        return INT32_MAX;
    }
    const int64_t ab = (int64_t)a * (int64_t)b; /* |ab| < 2^62: no overflow */
    /* (ab * 2) >> 32 with an arithmetic shift == floor(ab / 2^31), truncated to 32 bits */
    return (int32_t)(uint32_t)(uint64_t)(ab >> 31);
}

/* SRSHL with a negative shift: round-half-up arithmetic right shift.
 * tests/validation/reference/UtilsQuantizedAsymm.h:53-56; AsymmHelpers.cpp:256-259. */
ORC_EXPORT int32_t orc_rounding_divide_by_pow2(int32_t x, int32_t exponent)
{
    if (exponent == 0)
    {
        return x;
    }
    const int32_t biased = wrap_add(x, (int32_t)(1u << (exponent - 1)));
    return biased >> exponent; /* gcc: arithmetic shift on signed */
}

/* tests/validation/reference/UtilsQuantizedAsymm.h:69-89 and GEMMLowp.cpp:122-157: requantise one
 * accumulator; min/max are applied as given and the result is then saturated to the 8-bit range. */
ORC_EXPORT int32_t orc_quantize_down_fixedpoint(int32_t acc, int32_t mult, int32_t shift, int32_t offset_after_shift,
                                                int32_t lo, int32_t hi)
{
    int32_t r;
    if (shift < 0)
    {
        r = orc_sqdmulh(wrap_mul(acc, (int32_t)(1u << (-shift))), mult);
    }
    else
    {
        r = orc_rounding_divide_by_pow2(orc_sqdmulh(acc, mult), shift);
    }
    r = wrap_add(r, offset_after_shift);
    if (r < lo)
    {
        r = lo;
    }
    if (r > hi)
    {
        r = hi;
    }
    return r;
}

/* float multiplier -> (int32 Q0.31 multiplier, shift); shift > 0 is a right shift, < 0 a left shift.
 * src/core/utils/quantization/AsymmHelpers.cpp:43-115 (calculate_quantized_multiplier and the
 * less_than_one / greater_than_one helpers).  Returns 0 on success. */
ORC_EXPORT int orc_calculate_quantized_multiplier(float multiplier, int32_t *quant_multiplier, int32_t *shift)
{
    int          e       = 0;
    const double q       = frexp((double)multiplier, &e);
    int64_t      q_fixed = (int64_t)llround(q * (double)(1ll << 31));
    if (multiplier >= 1.f)
    {
        int left = e;
        if (q_fixed > (1ll << 31))
        {
            return 1;
        }
        if (q_fixed == (1ll << 31))
        {
            q_fixed /= 2;
            ++left;
        }
        if (left < 0 || q_fixed > INT32_MAX)
        {
            return 1;
        }
        *quant_multiplier = (int32_t)q_fixed;
        *shift            = -left;
        return 0;
    }
    if (multiplier < -0.00001f || multiplier > 1.0f + 0.00001f)
    {
        return 1;
    }
    int right = -e;
    if (q_fixed > (1ll << 31))
    {
        return 1;
    }
    if (q_fixed == (1ll << 31))
    {
        q_fixed /= 2;
        --right;
    }
    if (right < 0 || q_fixed > INT32_MAX)
    {
        return 1;
    }
    *quant_multiplier = (int32_t)q_fixed;
    *shift            = right;
    return 0;
}

/* Per-channel multipliers: multiplier[i] = i_scale * w_scale[i] / o_scale evaluated in float32 in that
 * order.  src/core/utils/quantization/AsymmHelpers.cpp:117-152. */
ORC_EXPORT int orc_calculate_quantized_multipliers(float i_scale, const float *w_scales, int n, float o_scale,
                                                   int32_t *mults, int32_t *shifts)
{
    for (int i = 0; i < n; ++i)
    {
        const float m = i_scale * w_scales[i] / o_scale;
        if (orc_calculate_quantized_multiplier(m, &mults[i], &shifts[i]) != 0)
        {
            return 1;
        }
    }
    return 0;
}

static inline int32_t load8(const void *p, size_t idx, int is_signed)
{
    return is_signed ? (int32_t)((const int8_t *)p)[idx] : (int32_t)((const uint8_t *)p)[idx];
}

/* c[m,n] = sum_k (a[m,k] + a_off) * (b[k,n] + b_off): the offsets are ADDED as given.
 * tests/validation/reference/GEMMLowp.cpp:202-255.  a: [batch][M][K], b: [K][N] or [batch][K][N]
 * (b_batch_stride 0 = shared), c: [batch][M][N] int32.  Row-parallel; the k-outer / j-inner loop
 * order of the reference is kept so gcc can vectorise the j loop. */
ORC_EXPORT void orc_gemmlowp_core(const void *a, int a_signed, const void *b, int b_signed, int32_t *c, int M, int N,
                                  int K, int batch, int b_batched, int32_t a_off, int32_t b_off)
{
    for (int d = 0; d < batch; ++d)
    {
        const size_t abase = (size_t)d * M * K;
        const size_t bbase = b_batched ? (size_t)d * K * N : 0;
        int32_t     *cd    = c + (size_t)d * M * N;
        /* widen B once so the inner loop is a plain int32 multiply-add */
        int32_t *bw = (int32_t *)malloc((size_t)K * N * sizeof(int32_t));
        for (size_t i = 0; i < (size_t)K * N; ++i)
        {
            bw[i] = wrap_add(load8(b, bbase + i, b_signed), b_off);
        }
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
        for (int i = 0; i < M; ++i)
        {
            int32_t *acc = cd + (size_t)i * N;
            for (int j = 0; j < N; ++j)
            {
                acc[j] = 0;
            }
            for (int k = 0; k < K; ++k)
            {
                const int32_t  av  = wrap_add(load8(a, abase + (size_t)i * K + k, a_signed), a_off);
                const int32_t *brw = bw + (size_t)k * N;
                for (int j = 0; j < N; ++j)
                {
                    acc[j] = (int32_t)((uint32_t)acc[j] + (uint32_t)av * (uint32_t)brw[j]);
                }
            }
        }
        free(bw);
    }
}

/* rowsum[m] = sum_k a[m,k]   src/cpu/kernels/CpuGemmLowpMatrixReductionKernel.cpp:133-204 */
ORC_EXPORT void orc_reduce_rows(const void *a, int a_signed, int M, int K, int32_t *out)
{
    for (int i = 0; i < M; ++i)
    {
        int32_t s = 0;
        for (int k = 0; k < K; ++k)
        {
            s = wrap_add(s, load8(a, (size_t)i * K + k, a_signed));
        }
        out[i] = s;
    }
}

/* colsum[n] = sum_k b[k,n]   src/cpu/kernels/CpuGemmLowpMatrixReductionKernel.cpp:273-446 */
ORC_EXPORT void orc_reduce_cols(const void *b, int b_signed, int K, int N, int32_t *out)
{
    for (int j = 0; j < N; ++j)
    {
        out[j] = 0;
    }
    for (int k = 0; k < K; ++k)
    {
        for (int j = 0; j < N; ++j)
        {
            out[j] = wrap_add(out[j], load8(b, (size_t)k * N + j, b_signed));
        }
    }
}

/* In-place offset contribution on the raw product sum_k a*b (output stage NONE):
 *   + a_off * colsum[n] + b_off * rowsum[m] + K * a_off * b_off
 * src/cpu/kernels/CpuGemmLowpOffsetContributionKernel.cpp:116-229. */
ORC_EXPORT void orc_offset_contribution(int32_t *mm, int M, int N, int K, const int32_t *colsum,
                                        const int32_t *rowsum, int32_t a_off, int32_t b_off)
{
    const int32_t k_term = wrap_mul(wrap_mul(a_off, b_off), K);
    for (int i = 0; i < M; ++i)
    {
        for (int j = 0; j < N; ++j)
        {
            int32_t v = mm[(size_t)i * N + j];
            if (a_off != 0)
            {
                v = wrap_add(v, wrap_mul(a_off, colsum[j]));
            }
            if (b_off != 0)
            {
                v = wrap_add(v, wrap_mul(b_off, rowsum[i]));
            }
            if (a_off != 0 && b_off != 0)
            {
                v = wrap_add(v, k_term);
            }
            mm[(size_t)i * N + j] = v;
        }
    }
}

/* Standalone / fused output stage QUANTIZE_DOWN_FIXEDPOINT over an int32 [M,N] matrix.
 * tests/validation/reference/GEMMLowp.cpp:106-158.  n_mult == 1: per-tensor, else per-column.
 * The oracle clamps to [lo,hi] and saturates to the 8-bit type; callers always pass bounds inside the
 * type range (or the type range itself), for which this is identical to the reference. */
ORC_EXPORT void orc_output_stage(const int32_t *in, const int32_t *bias, void *out, int out_signed, int M, int N,
                                 const int32_t *mult, const int32_t *shift, int n_mult, int32_t offset, int32_t lo,
                                 int32_t hi)
{
    const int32_t tmin = out_signed ? -128 : 0;
    const int32_t tmax = out_signed ? 127 : 255;
    const int32_t l    = lo > tmin ? lo : tmin;
    const int32_t h    = hi < tmax ? hi : tmax;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (int i = 0; i < M; ++i)
    {
        for (int j = 0; j < N; ++j)
        {
            int32_t v = in[(size_t)i * N + j];
            if (bias != NULL)
            {
                v = wrap_add(v, bias[j]);
            }
            const int32_t m = n_mult > 1 ? mult[j] : mult[0];
            const int32_t s = n_mult > 1 ? shift[j] : shift[0];
            const int32_t r = orc_quantize_down_fixedpoint(v, m, s, offset, l, h);
            if (out_signed)
            {
                ((int8_t *)out)[(size_t)i * N + j] = (int8_t)r;
            }
            else
            {
                ((uint8_t *)out)[(size_t)i * N + j] = (uint8_t)r;
            }
        }
    }
}

/* The same stage with a QSYMM16 destination (CpuGemmLowpQuantizeDownInt32ToInt16ScaleByFixedPointKernel;
 * tests/validation/reference/GEMMLowp.cpp:106-157 instantiated for int16_t, :423-436): identical arithmetic,
 * bounds intersected with the int16 range. */
ORC_EXPORT void orc_output_stage_s16(const int32_t *in, const int32_t *bias, int16_t *out, int M, int N,
                                     const int32_t *mult, const int32_t *shift, int n_mult, int32_t offset, int32_t lo,
                                     int32_t hi)
{
    const int32_t l = lo > -32768 ? lo : -32768;
    const int32_t h = hi < 32767 ? hi : 32767;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (int i = 0; i < M; ++i)
    {
        for (int j = 0; j < N; ++j)
        {
            int32_t v = in[(size_t)i * N + j];
            if (bias != NULL)
            {
                v = wrap_add(v, bias[j]);
            }
            const int32_t m = n_mult > 1 ? mult[j] : mult[0];
            const int32_t s = n_mult > 1 ? shift[j] : shift[0];
            out[(size_t)i * N + j] = (int16_t)orc_quantize_down_fixedpoint(v, m, s, offset, l, h);
        }
    }
}

/* Output stage QUANTIZE_DOWN (integer multiply): ((in + offset + bias) * mult) >> shift in wrapping int32 with an
 * arithmetic shift, clamped to [lo, hi] only when lo != hi, then saturated to the 8-bit type.
 * tests/validation/reference/GEMMLowp.cpp:66-104.  n_mult == 1: per-tensor, else per-column. */
ORC_EXPORT void orc_output_stage_int(const int32_t *in, const int32_t *bias, void *out, int out_signed, int M, int N,
                                     const int32_t *mult, const int32_t *shift, int n_mult, int32_t offset, int32_t lo,
                                     int32_t hi)
{
    const int32_t tmin = out_signed ? -128 : 0;
    const int32_t tmax = out_signed ? 127 : 255;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
    for (int i = 0; i < M; ++i)
    {
        for (int j = 0; j < N; ++j)
        {
            int32_t v = wrap_add(in[(size_t)i * N + j], offset);
            if (bias != NULL)
            {
                v = wrap_add(v, bias[j]);
            }
            v = wrap_mul(v, n_mult > 1 ? mult[j] : mult[0]);
            v >>= (n_mult > 1 ? shift[j] : shift[0]); /* gcc: arithmetic shift on signed */
            if (lo != hi)
            {
                v = v < lo ? lo : (v > hi ? hi : v);
            }
            v = v < tmin ? tmin : (v > tmax ? tmax : v);
            if (out_signed)
            {
                ((int8_t *)out)[(size_t)i * N + j] = (int8_t)v;
            }
            else
            {
                ((uint8_t *)out)[(size_t)i * N + j] = (uint8_t)v;
            }
        }
    }
}

/* The fused function with the QUANTIZE_DOWN stage (CpuGemmLowpOffsetContributionOutputStageKernel.cpp with
 * is_fixed_point == false): raw product + offset contribution, then the stage above. */
ORC_EXPORT void orc_gemmlowp_fused_int(const void *a, int a_signed, const void *b, int b_signed, const int32_t *bias,
                                       void *out, int out_signed, int M, int N, int K, int32_t a_off, int32_t b_off,
                                       const int32_t *mult, const int32_t *shift, int n_mult, int32_t offset,
                                       int32_t lo, int32_t hi)
{
    int32_t *mm     = (int32_t *)malloc((size_t)M * N * sizeof(int32_t));
    int32_t *colsum = (int32_t *)malloc((size_t)N * sizeof(int32_t));
    int32_t *rowsum = (int32_t *)malloc((size_t)M * sizeof(int32_t));
    orc_gemmlowp_core(a, a_signed, b, b_signed, mm, M, N, K, 1, 0, 0, 0);
    orc_reduce_cols(b, b_signed, K, N, colsum);
    orc_reduce_rows(a, a_signed, M, K, rowsum);
    orc_offset_contribution(mm, M, N, K, colsum, rowsum, a_off, b_off);
    orc_output_stage_int(mm, bias, out, out_signed, M, N, mult, shift, n_mult, offset, lo, hi);
    free(mm);
    free(colsum);
    free(rowsum);
}

/* The fused function: NEGEMMLowpMatrixMultiplyCore with a QUANTIZE_DOWN_FIXEDPOINT output stage, built
 * the way the library builds it (raw product + offset contribution + bias + requantise):
 * src/cpu/kernels/CpuGemmLowpOffsetContributionOutputStageKernel.cpp:275-346. */
ORC_EXPORT void orc_gemmlowp_fused(const void *a, int a_signed, const void *b, int b_signed, const int32_t *bias,
                                   void *out, int out_signed, int M, int N, int K, int32_t a_off, int32_t b_off,
                                   const int32_t *mult, const int32_t *shift, int n_mult, int32_t offset, int32_t lo,
                                   int32_t hi)
{
    int32_t *mm     = (int32_t *)malloc((size_t)M * N * sizeof(int32_t));
    int32_t *colsum = (int32_t *)malloc((size_t)N * sizeof(int32_t));
    int32_t *rowsum = (int32_t *)malloc((size_t)M * sizeof(int32_t));
    orc_gemmlowp_core(a, a_signed, b, b_signed, mm, M, N, K, 1, 0, 0, 0);
    orc_reduce_cols(b, b_signed, K, N, colsum);
    orc_reduce_rows(a, a_signed, M, K, rowsum);
    orc_offset_contribution(mm, M, N, K, colsum, rowsum, a_off, b_off);
    orc_output_stage(mm, bias, out, out_signed, M, N, mult, shift, n_mult, offset, lo, hi);
    free(mm);
    free(colsum);
    free(rowsum);
}

/* NHWC im2col for 8-bit data: src [B][H][W][C] -> dst [B][Ho*Wo][kh*kw*C] with the (ky,kx,c) order
 * (c fastest) and out-of-image taps filled with pad_value (= the input zero point).
 * src/cpu/kernels/directconv2d/impl.h:148-220,307-388; tests/validation/reference/Im2Col.cpp:105-160.
 * dst_row_stride >= kh*kw*C lets the caller pad K; the padding bytes are written as zero. */
ORC_EXPORT void orc_im2col_nhwc(const uint8_t *src, uint8_t *dst, int C, int W, int H, int B, int kw, int kh, int sx,
                                int sy, int pad_l, int pad_t, int dil_x, int dil_y, int Wo, int Ho, int pad_value,
                                int dst_row_stride)
{
    const int K = kh * kw * C;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int b = 0; b < B; ++b)
    {
        for (int yo = 0; yo < Ho; ++yo)
        {
            for (int xo = 0; xo < Wo; ++xo)
            {
                uint8_t *row = dst + ((size_t)(b * Ho + yo) * Wo + xo) * dst_row_stride;
                for (int ky = 0; ky < kh; ++ky)
                {
                    for (int kx = 0; kx < kw; ++kx)
                    {
                        const int yi = yo * sy - pad_t + ky * dil_y;
                        const int xi = xo * sx - pad_l + kx * dil_x;
                        uint8_t  *d  = row + (ky * kw + kx) * C;
                        if (yi < 0 || yi >= H || xi < 0 || xi >= W)
                        {
                            memset(d, pad_value, (size_t)C);
                        }
                        else
                        {
                            memcpy(d, src + (((size_t)b * H + yi) * W + xi) * C, (size_t)C);
                        }
                    }
                }
                if (dst_row_stride > K)
                {
                    memset(row + K, 0, (size_t)(dst_row_stride - K));
                }
            }
        }
    }
}

/* Weights [OFM][kh][kw][C] (NHWC weights, TensorShape(C,kw,kh,OFM)) -> GEMM B matrix [K][OFM] with
 * row index (ky*kw+kx)*C+c.  src/cpu/kernels/CpuWeightsReshapeKernel.cpp:121-183. */
ORC_EXPORT void orc_weights_reshape_nhwc(const uint8_t *w, uint8_t *dst, int C, int kw, int kh, int OFM)
{
    const int K = kh * kw * C;
    for (int o = 0; o < OFM; ++o)
    {
        for (int r = 0; r < K; ++r)
        {
            dst[(size_t)r * OFM + o] = w[(size_t)o * K + r];
        }
    }
}

/* NEGEMMConvolutionLayer for 8-bit NHWC tensors, built the way CpuGemmConv2d builds it
 * (src/cpu/operators/CpuGemmConv2d.cpp:243-332,910-1009): im2col (pad = input zero point) ->
 * GEMMLowp core with NEGATED zero points -> bias + fixed-point requantise + clamp.
 * src [B][H][W][C]; weights [OFM][kh][kw][C]; dst [B][Ho][Wo][OFM]. */
ORC_EXPORT void orc_conv2d_nhwc(const void *src, int src_signed, const void *weights, int w_signed,
                                const int32_t *bias, void *dst, int C, int W, int H, int B, int kw, int kh, int OFM,
                                int sx, int sy, int pad_l, int pad_t, int dil_x, int dil_y, int Wo, int Ho,
                                int32_t in_zp, int32_t w_zp, const int32_t *mult, const int32_t *shift, int n_mult,
                                int32_t out_offset, int32_t lo, int32_t hi)
{
    const int K    = kh * kw * C;
    const int M    = B * Ho * Wo;
    uint8_t  *cols = (uint8_t *)malloc((size_t)M * K);
    uint8_t  *bmat = (uint8_t *)malloc((size_t)K * OFM);
    orc_im2col_nhwc((const uint8_t *)src, cols, C, W, H, B, kw, kh, sx, sy, pad_l, pad_t, dil_x, dil_y, Wo, Ho,
                    in_zp & 0xff, K);
    orc_weights_reshape_nhwc((const uint8_t *)weights, bmat, C, kw, kh, OFM);
    orc_gemmlowp_fused(cols, src_signed, bmat, w_signed, bias, dst, src_signed, M, OFM, K, -in_zp, -w_zp, mult, shift,
                       n_mult, out_offset, lo, hi);
    free(cols);
    free(bmat);
}

/* Layout helpers used only by the tests to compare NHWC results with the NCHW reference oracle. */
ORC_EXPORT void orc_nhwc_to_nchw(const uint8_t *src, uint8_t *dst, int B, int H, int W, int C)
{
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x)
                for (int c = 0; c < C; ++c)
                    dst[(((size_t)b * C + c) * H + y) * W + x] = src[(((size_t)b * H + y) * W + x) * C + c];
}

ORC_EXPORT int orc_num_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
