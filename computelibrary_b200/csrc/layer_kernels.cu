// QASYMM8 layers between the convolutions of a quantized network: pooling, element-wise addition,
// ReLU-family activation and softmax on uint8 NHWC tensors.  All of them are HBM-bound byte kernels.
//
// The arithmetic is Compute Library's scalar oracle, operation by operation: dequantize
// ((q - zero_point) * scale), the float operator, quantize (lround(v / scale) + zero_point, clamped).  Every
// float operation is an explicit round-to-nearest intrinsic so that the compiler cannot contract or
// reorder them; where an operator is a function of ONE byte (activation, the requantisation after a
// maximum) the 256 possible results are computed once per block into shared memory with that same
// arithmetic and the kernel becomes a table look-up.
#include "common.cuh"
#include "kernels.cuh"

#include <cmath>
#include <cstring>
#include <map>
#include <mutex>

namespace cugl
{
namespace
{
constexpr int kThreads = 256;

// arm_compute/core/QuantizationInfo.h:342-345
__device__ __forceinline__ float dequantize(int q, float scale, int zp)
{
    return __fmul_rn(static_cast<float>(q - zp), scale);
}
// arm_compute/core/QuantizationInfo.h:268-273: lround(value / scale) + offset, clamped to the type.
// roundf rounds halves away from zero like lround; the clamp before the integer conversion only affects
// values that saturate anyway.
__device__ __forceinline__ int quantize_u8(float v, float scale, int zp)
{
    float r = roundf(__fdiv_rn(v, scale));
    r       = fminf(fmaxf(r, -1.0e6f), 1.0e6f);
    return min(max(static_cast<int>(r) + zp, 0), 255);
}
// tests/validation/reference/ActivationLayer.h:54-62
__device__ __forceinline__ float activate(float x, int act, float a, float b)
{
    switch (act)
    {
        case CUGL_ACT_RELU:
            return fmaxf(0.f, x);
        case CUGL_ACT_BOUNDED_RELU:
            return fminf(a, fmaxf(0.f, x));
        case CUGL_ACT_LU_BOUNDED_RELU:
            return fminf(a, fmaxf(b, x));
        default:
            return x;
    }
}

struct QInfo
{
    float scale;
    int   zp;
};

// table[q] = quantize(activate(dequantize(q))) for every byte value; blockDim.x >= 256 is not required
__device__ __forceinline__ void build_table(uint8_t *table, QInfo in, QInfo out, int act, float a, float b)
{
    for (int q = threadIdx.x; q < 256; q += blockDim.x)
    {
        table[q] = static_cast<uint8_t>(quantize_u8(activate(dequantize(q, in.scale, in.zp), act, a, b), out.scale, out.zp));
    }
    __syncthreads();
}
__device__ __forceinline__ uint32_t map4(const uint8_t *table, uint32_t w)
{
    return static_cast<uint32_t>(table[w & 0xff]) | (static_cast<uint32_t>(table[(w >> 8) & 0xff]) << 8) |
           (static_cast<uint32_t>(table[(w >> 16) & 0xff]) << 16) | (static_cast<uint32_t>(table[w >> 24]) << 24);
}

// ---- activation ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
    activation_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int64_t n, bool vec, QInfo in,
                      QInfo out, int act, float a, float b)
{
    __shared__ uint8_t table[256];
    build_table(table, in, out, act, a, b);
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t nth = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (vec)
    {
        const int64_t nv = n >> 4;
        for (int64_t i = tid; i < nv; i += nth)
        {
            uint4 v = __ldg(reinterpret_cast<const uint4 *>(src) + i);
            v.x     = map4(table, v.x);
            v.y     = map4(table, v.y);
            v.z     = map4(table, v.z);
            v.w     = map4(table, v.w);
            reinterpret_cast<uint4 *>(dst)[i] = v;
        }
        for (int64_t i = (nv << 4) + tid; i < n; i += nth)
        {
            dst[i] = table[src[i]];
        }
    }
    else
    {
        for (int64_t i = tid; i < n; i += nth)
        {
            dst[i] = table[src[i]];
        }
    }
}

// ---- addition --------------------------------------------------------------------------------------
// tests/validation/reference/ArithmeticOperations.cpp:40-53, 124-151.  The oracle adds the two floats in
// double and casts back: one rounding of the exact sum, which a float addition also gives as long as the
// operands' exponents are within 28 of each other (the exact sum then fits a double); the entry point
// enforces that through the scale ratio.
__device__ __forceinline__ uint32_t add_byte(uint32_t qa, uint32_t qb, QInfo ia, QInfo ib, QInfo o, const uint8_t *post)
{
    const float s = __fadd_rn(dequantize(static_cast<int>(qa), ia.scale, ia.zp), dequantize(static_cast<int>(qb), ib.scale, ib.zp));
    return post[quantize_u8(s, o.scale, o.zp)];
}
__device__ __forceinline__ uint32_t add4(uint32_t wa, uint32_t wb, QInfo ia, QInfo ib, QInfo o, const uint8_t *post)
{
    uint32_t r = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        r |= add_byte((wa >> (8 * j)) & 0xff, (wb >> (8 * j)) & 0xff, ia, ib, o, post) << (8 * j);
    }
    return r;
}
__global__ void __launch_bounds__(kThreads)
    add_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ b, uint8_t *__restrict__ dst, int64_t n,
               bool vec, QInfo ia, QInfo ib, QInfo o, int act, float act_a, float act_b)
{
    __shared__ uint8_t post[256]; // the activation on the quantized sum (identity table for CUGL_ACT_NONE)
    build_table(post, o, o, act, act_a, act_b);
    if (act == CUGL_ACT_NONE)
    {
        for (int q = threadIdx.x; q < 256; q += blockDim.x) post[q] = static_cast<uint8_t>(q);
        __syncthreads();
    }
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t nth = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t nv  = vec ? (n >> 4) : 0;
    for (int64_t i = tid; i < nv; i += nth)
    {
        const uint4 va = __ldg(reinterpret_cast<const uint4 *>(a) + i);
        const uint4 vb = __ldg(reinterpret_cast<const uint4 *>(b) + i);
        uint4       r;
        r.x = add4(va.x, vb.x, ia, ib, o, post);
        r.y = add4(va.y, vb.y, ia, ib, o, post);
        r.z = add4(va.z, vb.z, ia, ib, o, post);
        r.w = add4(va.w, vb.w, ia, ib, o, post);
        reinterpret_cast<uint4 *>(dst)[i] = r;
    }
    for (int64_t i = (nv << 4) + tid; i < n; i += nth)
    {
        dst[i] = static_cast<uint8_t>(add_byte(a[i], b[i], ia, ib, o, post));
    }
}

// Saturating form of the addition: for many quantizations (always when the three scales and zero points are
// equal, as in a residual network whose tensors share one quantization) the oracle's result over all 65536
// byte pairs is exactly min(max(min(a + b, 255), floor), cap).  The host proves that by enumeration
// (classify_add, below) and this kernel then needs seven to nine instructions per four elements (add_clamp_u8x4).
__global__ void __launch_bounds__(kThreads)
    add_saturating_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ b, uint8_t *__restrict__ dst,
                          int64_t n, bool vec, uint32_t floor4, uint32_t cap4)
{
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t nth = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t nv  = vec ? (n >> 4) : 0;
    for (int64_t i = tid; i < nv; i += nth)
    {
        const uint4 va = __ldg(reinterpret_cast<const uint4 *>(a) + i);
        const uint4 vb = __ldg(reinterpret_cast<const uint4 *>(b) + i);
        uint4       r;
        r.x = add_clamp_u8x4(va.x, vb.x, floor4, cap4);
        r.y = add_clamp_u8x4(va.y, vb.y, floor4, cap4);
        r.z = add_clamp_u8x4(va.z, vb.z, floor4, cap4);
        r.w = add_clamp_u8x4(va.w, vb.w, floor4, cap4);
        reinterpret_cast<uint4 *>(dst)[i] = r;
    }
    for (int64_t i = (nv << 4) + tid; i < n; i += nth)
    {
        const uint32_t v = min(static_cast<uint32_t>(a[i]) + b[i], 255u);
        dst[i]           = static_cast<uint8_t>(min(max(v, floor4 & 0xffu), cap4 & 0xffu));
    }
}

// ---- pooling ---------------------------------------------------------------------------------------
struct PoolGeom
{
    int B, H, W, C, Wo, Ho, pw, ph, sx, sy, pl, pr, pt, pb, exclude_padding;
};

// MAX (tests/validation/reference/PoolingLayer.cpp:78-134): window clipped to the image.  Dequantisation is
// monotonic (scale > 0), so the float maximum is the dequantized byte maximum and the result is
// table[max byte].  One thread per output pixel and 16 channels (kVec) or per single channel.
template <bool kVec>
__global__ void __launch_bounds__(kThreads)
    maxpool_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, PoolGeom g, QInfo in, QInfo out)
{
    __shared__ uint8_t table[256];
    build_table(table, in, out, CUGL_ACT_NONE, 0.f, 0.f);
    const int     cv    = kVec ? g.C >> 4 : g.C;
    const int64_t total = static_cast<int64_t>(g.B) * g.Ho * g.Wo * cv;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        int c, w, h, b;
        if (total <= 0x7fffffff) // 32-bit divisions: a 64-bit one costs more than the whole pooling window
        {
            uint32_t q = static_cast<uint32_t>(i);
            c          = static_cast<int>(q % static_cast<uint32_t>(cv));
            q /= static_cast<uint32_t>(cv);
            w = static_cast<int>(q % static_cast<uint32_t>(g.Wo));
            q /= static_cast<uint32_t>(g.Wo);
            h = static_cast<int>(q % static_cast<uint32_t>(g.Ho));
            b = static_cast<int>(q / static_cast<uint32_t>(g.Ho));
        }
        else
        {
            c         = static_cast<int>(i % cv);
            int64_t p = i / cv;
            w         = static_cast<int>(p % g.Wo);
            p /= g.Wo;
            h = static_cast<int>(p % g.Ho);
            b = static_cast<int>(p / g.Ho);
        }
        const int ws = max(w * g.sx - g.pl, 0), we = min(w * g.sx - g.pl + g.pw, g.W);
        const int hs = max(h * g.sy - g.pt, 0), he = min(h * g.sy - g.pt + g.ph, g.H);
        if (kVec)
        {
            // running maxima as halfword pairs (even bytes / odd bytes of each word): the 16-bit pair maximum is one
            // instruction, the byte-wise __vmaxu4 is not
            uint32_t me[4] = {0, 0, 0, 0}, mo[4] = {0, 0, 0, 0};
            for (int y = hs; y < he; ++y)
            {
                for (int x = ws; x < we; ++x)
                {
                    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src + ((static_cast<int64_t>(b) * g.H + y) * g.W + x) * g.C) + c);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                    {
                        const uint32_t e = __byte_perm(w[k], 0, 0x4240), o = __byte_perm(w[k], 0, 0x4341);
                        me[k]            = __vimax3_u16x2(me[k], e, e);
                        mo[k]            = __vimax3_u16x2(mo[k], o, o);
                    }
                }
            }
            uint4 m;
            m.x = __byte_perm(me[0], mo[0], 0x6240);
            m.y = __byte_perm(me[1], mo[1], 0x6240);
            m.z = __byte_perm(me[2], mo[2], 0x6240);
            m.w = __byte_perm(me[3], mo[3], 0x6240);
            m.x = map4(table, m.x);
            m.y = map4(table, m.y);
            m.z = map4(table, m.z);
            m.w = map4(table, m.w);
            reinterpret_cast<uint4 *>(dst + ((static_cast<int64_t>(b) * g.Ho + h) * g.Wo + w) * g.C)[c] = m;
        }
        else
        {
            int m = 0;
            for (int y = hs; y < he; ++y)
            {
                for (int x = ws; x < we; ++x)
                {
                    m = max(m, static_cast<int>(src[((static_cast<int64_t>(b) * g.H + y) * g.W + x) * g.C + c]));
                }
            }
            dst[((static_cast<int64_t>(b) * g.Ho + h) * g.Wo + w) * g.C + c] = table[m];
        }
    }
}

// The same for the window sizes a network uses (3x3, 2x2, and the 1x1 / stride 2 "subsampling" pool of ResNet's
// shortcuts), 16 channels per thread: the window is unrolled, taps outside the image load nothing and count as 0 (the
// identity of an unsigned maximum), so there is no loop and no branch per tap; two taps go into every three-operand
// maximum; and when the table is the identity (equal input and output quantization, checked entry by entry) the
// bytes are stored as they are.  About a third of the general kernel's instructions per output.
template <int N>
__device__ __forceinline__ uint32_t max_u16x2_of(const uint32_t (&v)[N])
{
    uint32_t m = v[0];
#pragma unroll
    for (int j = 1; j + 1 < N; j += 2)
    {
        m = __vimax3_u16x2(m, v[j], v[j + 1]);
    }
    if ((N & 1) == 0)
    {
        m = __vimax3_u16x2(m, v[N - 1], v[N - 1]);
    }
    return m;
}

template <int PW, int PH>
__global__ void __launch_bounds__(kThreads)
    maxpool_window_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, PoolGeom g, QInfo in, QInfo out)
{
    __shared__ uint8_t table[256];
    build_table(table, in, out, CUGL_ACT_NONE, 0.f, 0.f);
    bool same = true;
    for (int q = threadIdx.x; q < 256; q += blockDim.x)
    {
        same = same && table[q] == q;
    }
    const bool     identity = __syncthreads_and(same) != 0;
    constexpr int  kTaps    = PW * PH;
    const uint32_t cv       = static_cast<uint32_t>(g.C >> 4);
    const uint32_t total    = static_cast<uint32_t>(g.B) * g.Ho * g.Wo * cv; // the launcher keeps this below 2^31
    const int64_t  row_pitch = static_cast<int64_t>(g.W) * g.C;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
    {
        uint32_t       q = i;
        const uint32_t c = q % cv;
        q /= cv;
        const int w = static_cast<int>(q % static_cast<uint32_t>(g.Wo));
        q /= static_cast<uint32_t>(g.Wo);
        const int h = static_cast<int>(q % static_cast<uint32_t>(g.Ho));
        const int b = static_cast<int>(q / static_cast<uint32_t>(g.Ho));
        const int x0 = w * g.sx - g.pl, y0 = h * g.sy - g.pt;
        // tap (0, 0): outside the tensor for border pixels, where it is only used after the bounds test
        const uint8_t *p = src + (static_cast<int64_t>(b) * g.H + y0) * row_pitch + static_cast<int64_t>(x0) * g.C + 16 * c;
        uint4 t[kTaps];
#pragma unroll
        for (int y = 0; y < PH; ++y)
        {
            const bool y_in = static_cast<unsigned>(y0 + y) < static_cast<unsigned>(g.H);
#pragma unroll
            for (int x = 0; x < PW; ++x)
            {
                const bool tap_in = y_in && static_cast<unsigned>(x0 + x) < static_cast<unsigned>(g.W);
                t[y * PW + x]     = make_uint4(0, 0, 0, 0);
                if (tap_in)
                {
                    t[y * PW + x] = __ldg(reinterpret_cast<const uint4 *>(p + y * row_pitch + static_cast<int64_t>(x) * g.C));
                }
            }
        }
        uint32_t m[4];
        if (kTaps == 1)
        {
            m[0] = t[0].x, m[1] = t[0].y, m[2] = t[0].z, m[3] = t[0].w;
        }
        else
        {
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                // even and odd bytes as halfword pairs: the 16-bit pair maximum is one instruction
                uint32_t e[kTaps], o[kTaps];
#pragma unroll
                for (int j = 0; j < kTaps; ++j)
                {
                    const uint32_t word = k == 0 ? t[j].x : (k == 1 ? t[j].y : (k == 2 ? t[j].z : t[j].w));
                    e[j]                = __byte_perm(word, 0, 0x4240);
                    o[j]                = __byte_perm(word, 0, 0x4341);
                }
                m[k] = __byte_perm(max_u16x2_of(e), max_u16x2_of(o), 0x6240);
            }
        }
        if (!identity)
        {
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                m[k] = map4(table, m[k]);
            }
        }
        reinterpret_cast<uint4 *>(dst + ((static_cast<int64_t>(b) * g.Ho + h) * g.Wo + w) * g.C)[c] = make_uint4(m[0], m[1], m[2], m[3]);
    }
}

// AVG (tests/validation/reference/PoolingLayer.cpp:137-172): float sum in window order (y outer, x inner),
// divided by the window area with or without the padding.  One thread per output element; consecutive
// threads take consecutive channels.
// kVec = channels per thread (4: one 32-bit load per tap; every channel keeps its own sum in window order).
template <int kVec>
__global__ void __launch_bounds__(kThreads)
    avgpool_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, PoolGeom g, QInfo in, QInfo out)
{
    const int     cv    = g.C / kVec;
    const int64_t total = static_cast<int64_t>(g.B) * g.Ho * g.Wo * cv;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int c = static_cast<int>(i % cv) * kVec;
        int64_t   p = i / cv;
        const int w = static_cast<int>(p % g.Wo);
        p /= g.Wo;
        const int h = static_cast<int>(p % g.Ho);
        const int b = static_cast<int>(p / g.Ho);
        int       ws = w * g.sx - g.pl, hs = h * g.sy - g.pt;
        int       we = min(ws + g.pw, g.W + g.pr), he = min(hs + g.ph, g.H + g.pb);
        int       pool = (he - hs) * (we - ws);
        ws = max(ws, 0);
        hs = max(hs, 0);
        we = min(we, g.W);
        he = min(he, g.H);
        if (g.exclude_padding) pool = (he - hs) * (we - ws);
        float sum[kVec];
#pragma unroll
        for (int k = 0; k < kVec; ++k) sum[k] = 0.f;
        // the additions stay in window order (the float sum must round as the reference's does); the loads of a window
        // row are independent of them, so the row is walked by pointer and unrolled to keep several loads in flight
        // (a window as wide as the image, e.g. the global pool, is one run of pixels)
        const bool whole_rows = kVec == 4 && ws == 0 && we == g.W; // (one channel per thread: measured slower that way)
        const int  y_end = whole_rows ? hs + 1 : he, run = whole_rows ? (he - hs) * g.W : we - ws;
        for (int y = hs; y < y_end; ++y)
        {
            const uint8_t *px = src + ((static_cast<int64_t>(b) * g.H + y) * g.W + ws) * g.C + c;
#pragma unroll(kVec == 4 ? 8 : 1)
            for (int x = 0; x < run; ++x, px += g.C)
            {
                if (kVec == 4)
                {
                    const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(px));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                    {
                        sum[k] = __fadd_rn(sum[k], dequantize(static_cast<uint8_t>(v >> (8 * k)), in.scale, in.zp));
                    }
                }
                else
                {
                    sum[0] = __fadd_rn(sum[0], dequantize(__ldg(px), in.scale, in.zp));
                }
            }
        }
        uint8_t *o = dst + ((static_cast<int64_t>(b) * g.Ho + h) * g.Wo + w) * g.C + c;
        if (kVec == 4)
        {
            uint32_t r = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                r |= static_cast<uint32_t>(quantize_u8(__fdiv_rn(sum[k], static_cast<float>(pool)), out.scale, out.zp) & 0xff) << (8 * k);
            }
            *reinterpret_cast<uint32_t *>(o) = r;
        }
        else
        {
            o[0] = static_cast<uint8_t>(quantize_u8(__fdiv_rn(sum[0], static_cast<float>(pool)), out.scale, out.zp));
        }
    }
}

// ---- softmax ---------------------------------------------------------------------------------------
// tests/validation/reference/SoftmaxLayer.cpp:39-107: max, exp((x - max) * beta), sum, divide; quantized with
// (1/256, 0).  One block per row; the sum is a tree reduction and exp is expf, so the result may differ from
// the oracle's sequential sum by one quantization step.
__global__ void __launch_bounds__(kThreads)
    softmax_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int cols, float beta, QInfo in)
{
    __shared__ float red[kThreads];
    __shared__ float etab[256]; // exp of every possible byte value relative to the row maximum
    const uint8_t *s = src + static_cast<int64_t>(blockIdx.x) * cols;
    uint8_t       *d = dst + static_cast<int64_t>(blockIdx.x) * cols;
    int            m = 0;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) m = max(m, static_cast<int>(s[i]));
    red[threadIdx.x] = static_cast<float>(m);
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1)
    {
        if (threadIdx.x < o) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    const float fmax_ = dequantize(static_cast<int>(red[0]), in.scale, in.zp);
    __syncthreads();
    for (int q = threadIdx.x; q < 256; q += blockDim.x)
    {
        etab[q] = expf(__fmul_rn(__fsub_rn(dequantize(q, in.scale, in.zp), fmax_), beta));
    }
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) sum += etab[s[i]];
    red[threadIdx.x] = sum;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1)
    {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    const float total = red[0];
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
    {
        d[i] = static_cast<uint8_t>(quantize_u8(__fdiv_rn(etab[s[i]], total), 1.f / 256.f, 0));
    }
}

// Host copy of the oracle arithmetic (same expressions, evaluated by the host compiler without contraction:
// x86-64 baseline has no fused multiply-add) used to classify an addition.
inline float h_dequantize(int q, float scale, int zp)
{
    return static_cast<float>(q - zp) * scale;
}
inline int h_quantize_u8(float v, float scale, int zp)
{
    const long q = lroundf(v / scale) + zp;
    return static_cast<int>(q < 0 ? 0 : (q > 255 ? 255 : q));
}
inline float h_activate(float x, int act, float a, float b)
{
    switch (act)
    {
        case CUGL_ACT_RELU:
            return x > 0.f ? x : 0.f;
        case CUGL_ACT_BOUNDED_RELU:
        {
            const float t = x > 0.f ? x : 0.f;
            return t < a ? t : a;
        }
        case CUGL_ACT_LU_BOUNDED_RELU:
        {
            const float t = x > b ? x : b;
            return t < a ? t : a;
        }
        default:
            return x;
    }
}
} // namespace

// True when act(quantize(dequantize(a) + dequantize(b))) == min(max(min(a + b, 255), floor), cap) for all 65536
// byte pairs; floor and cap are returned.  Results are remembered per parameter set.
bool classify_add(float a_scale, int a_zp, float b_scale, int b_zp, float o_scale, int o_zp, int act, float act_a,
                  float act_b, int *floor_out, int *cap_out)
{
    struct Key
    {
        float as, bs, os, aa, ab;
        int   az, bz, oz, act;
        bool  operator<(const Key &o) const
        {
            return std::memcmp(this, &o, sizeof(Key)) < 0;
        }
    };
    struct Form
    {
        bool saturating;
        int  floor, cap;
    };
    static std::mutex          mu;
    static std::map<Key, Form> cache;
    Key                        key;
    std::memset(&key, 0, sizeof(key));
    key.as = a_scale, key.bs = b_scale, key.os = o_scale, key.aa = act_a, key.ab = act_b;
    key.az = a_zp, key.bz = b_zp, key.oz = o_zp, key.act = act;
    std::lock_guard<std::mutex> lock(mu);
    auto                        it = cache.find(key);
    if (it == cache.end())
    {
        auto eval = [&](int qa, int qb)
        {
            const double s = static_cast<double>(h_dequantize(qa, a_scale, a_zp)) + static_cast<double>(h_dequantize(qb, b_scale, b_zp));
            const int    q = h_quantize_u8(static_cast<float>(s), o_scale, o_zp);
            return act == CUGL_ACT_NONE ? q : h_quantize_u8(h_activate(h_dequantize(q, o_scale, o_zp), act, act_a, act_b), o_scale, o_zp);
        };
        Form f{true, eval(0, 0), eval(255, 255)};
        for (int qa = 0; qa < 256 && f.saturating; ++qa)
        {
            for (int qb = 0; qb < 256; ++qb)
            {
                const int sum  = qa + qb > 255 ? 255 : qa + qb;
                const int want = sum < f.floor ? f.floor : (sum > f.cap ? f.cap : sum);
                if (eval(qa, qb) != want)
                {
                    f.saturating = false;
                    break;
                }
            }
        }
        it = cache.emplace(key, f).first;
    }
    *floor_out = it->second.floor;
    *cap_out   = it->second.cap;
    return it->second.saturating;
}

namespace
{
int grid_for(int64_t work_items, int sm_count)
{
    const int64_t blocks = (work_items + kThreads - 1) / kThreads;
    const int64_t cap    = static_cast<int64_t>(sm_count) * 8; // whole multiples of the SM count
    return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

bool valid_scale(float s)
{
    return s > 0.f && s < 1.0e30f;
}
bool valid_act(int act)
{
    return act >= CUGL_ACT_NONE && act <= CUGL_ACT_LU_BOUNDED_RELU;
}
bool aligned16(const void *p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}
} // namespace
} // namespace cugl

using namespace cugl;

extern "C"
{
    void cugl_pool2d_out_dims(const cugl_pool_desc *d, int32_t *Wo, int32_t *Ho)
    {
        int32_t w = 1, h = 1;
        if (d != nullptr && !d->is_global && d->stride_x > 0 && d->stride_y > 0)
        {
            w = (d->W + d->pad_left + d->pad_right - d->pool_w) / d->stride_x + 1;
            h = (d->H + d->pad_top + d->pad_bottom - d->pool_h) / d->stride_y + 1;
        }
        if (Wo) *Wo = w;
        if (Ho) *Ho = h;
    }

    cugl_status cugl_pool2d_validate(const cugl_pool_desc *d)
    {
        if (d == nullptr || d->B < 1 || d->H < 1 || d->W < 1 || d->C < 1 ||
            (d->pool_type != CUGL_POOL_MAX && d->pool_type != CUGL_POOL_AVG) || !valid_scale(d->src_scale) ||
            !valid_scale(d->dst_scale))
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "pooling: bad tensor, pooling type or quantization scale");
        }
        if (!d->is_global)
        {
            if (d->pool_w < 1 || d->pool_h < 1 || d->stride_x < 1 || d->stride_y < 1 || d->pad_left < 0 ||
                d->pad_right < 0 || d->pad_top < 0 || d->pad_bottom < 0)
            {
                return fail(nullptr, CUGL_INVALID_ARGUMENT, "pooling: bad window, stride or padding");
            }
            // src/cpu/kernels/CpuPool2dKernel.cpp: the padding must be smaller than the window
            if (d->pad_left >= d->pool_w || d->pad_right >= d->pool_w || d->pad_top >= d->pool_h || d->pad_bottom >= d->pool_h)
            {
                return fail(nullptr, CUGL_INVALID_ARGUMENT, "pooling: padding must be smaller than the pooling window");
            }
            int32_t wo, ho;
            cugl_pool2d_out_dims(d, &wo, &ho);
            if (wo < 1 || ho < 1)
            {
                return fail(nullptr, CUGL_INVALID_ARGUMENT, "pooling: window larger than the padded input");
            }
        }
        return CUGL_SUCCESS;
    }

    cugl_status cugl_pool2d_nhwc(cugl_context *ctx, const cugl_pool_desc *d, const void *d_src, void *d_dst)
    {
        if (ctx == nullptr || d_src == nullptr || d_dst == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_pool2d_nhwc: null argument");
        }
        CUGL_TRY(cugl_pool2d_validate(d));
        PoolGeom g;
        g.B = d->B;
        g.H = d->H;
        g.W = d->W;
        g.C = d->C;
        if (d->is_global)
        {
            g.pw = d->W;
            g.ph = d->H;
            g.sx = g.sy = 1;
            g.pl = g.pr = g.pt = g.pb = 0;
            g.Wo = g.Ho = 1;
        }
        else
        {
            g.pw = d->pool_w;
            g.ph = d->pool_h;
            g.sx = d->stride_x;
            g.sy = d->stride_y;
            g.pl = d->pad_left;
            g.pr = d->pad_right;
            g.pt = d->pad_top;
            g.pb = d->pad_bottom;
            cugl_pool2d_out_dims(d, &g.Wo, &g.Ho);
        }
        g.exclude_padding = d->exclude_padding;
        const QInfo   in{d->src_scale, d->src_zero_point}, out{d->dst_scale, d->dst_zero_point};
        const int64_t pixels = static_cast<int64_t>(g.B) * g.Ho * g.Wo;
        if (d->pool_type == CUGL_POOL_MAX)
        {
            const bool vec = (g.C % 16) == 0 && aligned16(d_src) && aligned16(d_dst);
            const int64_t items = pixels * (g.C / 16);
            const auto   *s8    = static_cast<const uint8_t *>(d_src);
            auto         *d8    = static_cast<uint8_t *>(d_dst);
            if (vec && items <= 0x7fffffff && g.pw == 3 && g.ph == 3)
            {
                maxpool_window_kernel<3, 3><<<grid_for(items, ctx->sm_count), kThreads, 0, ctx->stream>>>(s8, d8, g, in, out);
            }
            else if (vec && items <= 0x7fffffff && g.pw == 2 && g.ph == 2)
            {
                maxpool_window_kernel<2, 2><<<grid_for(items, ctx->sm_count), kThreads, 0, ctx->stream>>>(s8, d8, g, in, out);
            }
            else if (vec && items <= 0x7fffffff && g.pw == 1 && g.ph == 1)
            {
                maxpool_window_kernel<1, 1><<<grid_for(items, ctx->sm_count), kThreads, 0, ctx->stream>>>(s8, d8, g, in, out);
            }
            else if (vec)
            {
                maxpool_kernel<true><<<grid_for(items, ctx->sm_count), kThreads, 0, ctx->stream>>>(s8, d8, g, in, out);
            }
            else
            {
                maxpool_kernel<false><<<grid_for(pixels * g.C, ctx->sm_count), kThreads, 0, ctx->stream>>>(
                    static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), g, in, out);
            }
            return check_cuda(ctx, cudaGetLastError(), "maxpool_kernel");
        }
        // four channels per thread once that still leaves every SM a hundred threads or more (global pool of
        // 7 x 7 x 2048: batch 256 32 -> 18 us, batch 64 21 -> 14 us); below that the one-channel form has the parallelism
        const bool vec4 = (g.C % 4) == 0 && pixels * (g.C / 4) >= static_cast<int64_t>(ctx->sm_count) * 128 &&
                          ((reinterpret_cast<uintptr_t>(d_src) | reinterpret_cast<uintptr_t>(d_dst)) & 3) == 0;
        if (vec4)
        {
            avgpool_kernel<4><<<grid_for(pixels * (g.C / 4), ctx->sm_count), kThreads, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), g, in, out);
        }
        else
        {
            avgpool_kernel<1><<<grid_for(pixels * g.C, ctx->sm_count), kThreads, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), g, in, out);
        }
        return check_cuda(ctx, cudaGetLastError(), "avgpool_kernel");
    }

    cugl_status cugl_add_qasymm8(cugl_context *ctx, const void *d_a, const void *d_b, void *d_dst, int64_t n,
                                 float a_scale, int32_t a_zp, float b_scale, int32_t b_zp, float o_scale, int32_t o_zp,
                                 int32_t activation, float act_a, float act_b)
    {
        if (ctx == nullptr || d_a == nullptr || d_b == nullptr || d_dst == nullptr || n < 0 || !valid_scale(a_scale) ||
            !valid_scale(b_scale) || !valid_scale(o_scale) || !valid_act(activation))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_add_qasymm8: bad argument");
        }
        const float ratio = a_scale / b_scale;
        if (!(ratio > 9.5367431640625e-07f && ratio < 1048576.f))
        {
            return fail(ctx, CUGL_UNSUPPORTED_CONFIG, "cugl_add_qasymm8: input scales more than 2^20 apart");
        }
        if (n == 0) return CUGL_SUCCESS;
        const bool vec = aligned16(d_a) && aligned16(d_b) && aligned16(d_dst);
        int        floor_q = 0, cap_q = 255;
        if (classify_add(a_scale, a_zp, b_scale, b_zp, o_scale, o_zp, activation, act_a, act_b, &floor_q, &cap_q))
        {
            add_saturating_kernel<<<grid_for((n + 15) / 16, ctx->sm_count), kThreads, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(d_a), static_cast<const uint8_t *>(d_b), static_cast<uint8_t *>(d_dst), n,
                vec, static_cast<uint32_t>(floor_q) * 0x01010101u, static_cast<uint32_t>(cap_q) * 0x01010101u);
            return check_cuda(ctx, cudaGetLastError(), "add_saturating_kernel");
        }
        add_kernel<<<grid_for((n + 15) / 16, ctx->sm_count), kThreads, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(d_a), static_cast<const uint8_t *>(d_b), static_cast<uint8_t *>(d_dst), n, vec,
            QInfo{a_scale, a_zp}, QInfo{b_scale, b_zp}, QInfo{o_scale, o_zp}, activation, act_a, act_b);
        return check_cuda(ctx, cudaGetLastError(), "add_kernel");
    }

    cugl_status cugl_activation_qasymm8(cugl_context *ctx, const void *d_src, void *d_dst, int64_t n,
                                        int32_t activation, float act_a, float act_b, float src_scale, int32_t src_zp,
                                        float dst_scale, int32_t dst_zp)
    {
        if (ctx == nullptr || d_src == nullptr || d_dst == nullptr || n < 0 || !valid_scale(src_scale) ||
            !valid_scale(dst_scale) || !valid_act(activation))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_activation_qasymm8: bad argument");
        }
        if (n == 0) return CUGL_SUCCESS;
        const bool vec = aligned16(d_src) && aligned16(d_dst);
        activation_kernel<<<grid_for((n + 15) / 16, ctx->sm_count), kThreads, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), n, vec, QInfo{src_scale, src_zp},
            QInfo{dst_scale, dst_zp}, activation, act_a, act_b);
        return check_cuda(ctx, cudaGetLastError(), "activation_kernel");
    }

    cugl_status cugl_softmax_qasymm8(cugl_context *ctx, const void *d_src, void *d_dst, int32_t rows, int32_t cols,
                                     float beta, float src_scale, int32_t src_zp)
    {
        if (ctx == nullptr || d_src == nullptr || d_dst == nullptr || rows < 0 || cols < 1 || !valid_scale(src_scale))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_softmax_qasymm8: bad argument");
        }
        if (rows == 0) return CUGL_SUCCESS;
        softmax_kernel<<<rows, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_src),
                                                           static_cast<uint8_t *>(d_dst), cols, beta,
                                                           QInfo{src_scale, src_zp});
        return check_cuda(ctx, cudaGetLastError(), "softmax_kernel");
    }
}
