// Shared declarations of the cugl CUDA backend: context object, error plumbing and the integer
// requantisation primitives every epilogue uses.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

#include "cugl.h"

struct cugl_context
{
    int          device      = 0;
    int          sm_count    = 0;
    cudaStream_t stream      = nullptr;
    bool         owns_stream = false;
    int32_t     *d_status    = nullptr; // device word written by kernels whose bounded waits ran out
    int32_t     *h_status    = nullptr; // pinned mirror read in cugl_sync
    long long   *d_trace     = nullptr; // optional event-timestamp buffer for the tensor-core GEMM kernels
    long long    spin_limit  = 4000000000ll; // clock64 ticks a device-side wait may last (about two seconds)
    int          withhold_kb = -1;      // one-shot test instrument, see cugl_context_withhold_copy_once
    int          dependent_launch = 1;  // tensor-core kernels launch with programmatic stream serialization
    std::string  last_error;
};

namespace cugl
{
void        set_global_error(const std::string &msg);
cugl_status fail(cugl_context *ctx, cugl_status code, const std::string &msg);
cugl_status check_cuda(cugl_context *ctx, cudaError_t e, const char *what);

#define CUGL_CUDA_TRY(ctx, expr)                                     \
    do                                                               \
    {                                                                \
        cudaError_t _e = (expr);                                     \
        if (_e != cudaSuccess)                                       \
        {                                                            \
            return ::cugl::check_cuda((ctx), _e, #expr);             \
        }                                                            \
    } while (0)

#define CUGL_TRY(expr)                   \
    do                                   \
    {                                    \
        cugl_status _s = (expr);         \
        if (_s != CUGL_SUCCESS)          \
        {                                \
            return _s;                   \
        }                                \
    } while (0)

// Device status codes (written to cugl_context::d_status)
enum : int32_t
{
    DEV_OK               = 0,
    DEV_TIMEOUT_PRODUCER = 1,
    DEV_TIMEOUT_MMA      = 2,
    DEV_TIMEOUT_EPILOGUE = 3,
    DEV_TIMEOUT_DRAIN    = 4
};

// Everything an epilogue needs to turn a raw sum_k A*B accumulator into the function's output.
// Follows CpuGemmLowpOffsetContributionOutputStageKernel.cpp:275-346 (term assembly) and
// tests/validation/reference/GEMMLowp.cpp:122-157 (requantisation).
struct EpilogueParams
{
    const int32_t *colsum; // [N]  sum_k B[k,n]           (nullptr when a_offset == 0)
    const int32_t *rowsum; // [M]  sum_k A[m,k]           (nullptr when b_offset == 0)
    const int32_t *bias;   // [N]                          (nullptr when absent)
    const int32_t *mults;  // [N] per-channel multipliers  (nullptr: per-tensor)
    const int32_t *shifts; // [N] per-channel shifts
    int32_t        mult, shift;
    int32_t        a_off, b_off;
    int32_t        k_term;        // K * a_off * b_off
    int32_t        result_offset; // gemmlowp_offset
    int32_t        lo, hi;        // bounds already intersected with the 8-bit type range
    int32_t        stage;         // cugl_stage
    int32_t        out_signed;    // unused for S32
    // stage NONE only: out_f32 != 0 writes float(result) * dq_scale instead of the int32 result; accumulate != 0 adds
    // the value to what dst holds (int32 addition, or one float addition for a float destination)
    int32_t        out_f32;
    int32_t        accumulate;
    float          dq_scale;
};

// The 32-bit word a stage-NONE epilogue stores for the int32 result v, given the word dst holds now.
__device__ __forceinline__ uint32_t raw_result_word(int32_t v, uint32_t old, const EpilogueParams &ep)
{
    if (ep.out_f32 != 0)
    {
        float f = __fmul_rn(__int2float_rn(v), ep.dq_scale);
        if (ep.accumulate != 0)
        {
            f = __fadd_rn(__uint_as_float(old), f);
        }
        return __float_as_uint(f);
    }
    return ep.accumulate != 0 ? old + static_cast<uint32_t>(v) : static_cast<uint32_t>(v);
}

// SQDMULH: (int64(a) * b * 2) >> 32, i.e. floor(a*b / 2^31); saturates only for INT32_MIN^2.
// tests/validation/reference/UtilsQuantizedAsymm.h:60-67.
__device__ __forceinline__ int32_t sqdmulh(int32_t a, int32_t b)
{
    const int32_t  hi = __mulhi(a, b);
    const uint32_t lo = static_cast<uint32_t>(a) * static_cast<uint32_t>(b);
    int32_t        r  = static_cast<int32_t>(__funnelshift_l(lo, static_cast<uint32_t>(hi), 1));
    if (a == INT32_MIN && b == INT32_MIN)
    {
        r = INT32_MAX;
    }
    return r;
}

// Requantise one accumulator.  left = max(-shift, 0), right = max(shift, 0); exactly one is non-zero,
// so this single expression covers both branches of the reference:
//   shift <  0 : sqdmulh(acc * (1 << -shift), mult)
//   shift >= 0 : (sqdmulh(acc, mult) + (1 << (shift-1))) >> shift      (round-half-up, SRSHL)
__device__ __forceinline__ int32_t requantize(int32_t acc, int32_t mult, int32_t left, int32_t right)
{
    const int32_t  x     = static_cast<int32_t>(static_cast<uint32_t>(acc) << left);
    const int32_t  q     = sqdmulh(x, mult);
    const uint32_t round = (1u << right) >> 1; // 0 when right == 0
    return static_cast<int32_t>(static_cast<uint32_t>(q) + round) >> right;
}

__device__ __forceinline__ int32_t finalize(int32_t acc, int32_t mult, int32_t left, int32_t right, int32_t offset,
                                            int32_t lo, int32_t hi)
{
    const int32_t r = static_cast<int32_t>(static_cast<uint32_t>(requantize(acc, mult, left, right)) +
                                           static_cast<uint32_t>(offset));
    return min(max(r, lo), hi);
}

// Four unsigned bytes at once: min(max(min(a + b, 255), floor), cap) with floor <= cap <= 255, floor4 / cap4 holding the
// bound in every byte.  The byte-wise SIMD intrinsics (__vaddus4, __vmaxu4, __vminu4) have no instruction on
// sm_100 and expand to about seven instructions per element; the 16-bit pair forms of add-then-min and max do, so
// the bytes are widened into two words of halfword pairs (four byte permutes), added and bounded there (two or
// four instructions) and narrowed again (one permute).
__device__ __forceinline__ uint32_t add_clamp_u8x4(uint32_t a, uint32_t b, uint32_t floor4, uint32_t cap4)
{
    const uint32_t cap2 = cap4 & 0x00ff00ffu;
    uint32_t lo = __viaddmin_u16x2(__byte_perm(a, 0, 0x4140), __byte_perm(b, 0, 0x4140), cap2);
    uint32_t hi = __viaddmin_u16x2(__byte_perm(a, 0, 0x4342), __byte_perm(b, 0, 0x4342), cap2);
    if (floor4 != 0) // uniform over the launch
    {
        const uint32_t floor2 = floor4 & 0x00ff00ffu;
        lo = __vimax3_u16x2(lo, floor2, floor2);
        hi = __vimax3_u16x2(hi, floor2, floor2);
    }
    return __byte_perm(lo, hi, 0x6420);
}

// Output stage QUANTIZE_DOWN (tests/validation/reference/GEMMLowp.cpp:66-104): x already holds
// accumulator + offset + bias; wrapping multiply, arithmetic shift, clamp (bounds pre-intersected with the type).
__device__ __forceinline__ int32_t finalize_int(int32_t x, int32_t mult, int32_t shift, int32_t lo, int32_t hi)
{
    const int32_t r = static_cast<int32_t>(static_cast<uint32_t>(x) * static_cast<uint32_t>(mult)) >> shift;
    return min(max(r, lo), hi);
}

// Division by a run-time constant as multiply-high and shift (round-up method): with p = 31 + ceil(log2 d),
// mul = ceil(2^p / d) fits 32 bits and n / d == umulhi(n, mul) >> (p - 32) for every 0 <= n < 2^31.
struct FastDiv
{
    uint32_t mul, shr, d;
};

inline FastDiv make_fastdiv(int d)
{
    FastDiv f;
    f.d = static_cast<uint32_t>(d);
    if (d <= 1)
    {
        f.mul = 0;
        f.shr = 0;
        return f;
    }
    int l = 0;
    while ((1ll << l) < d) ++l;
    const int p = 31 + l;
    f.mul       = static_cast<uint32_t>(((1ull << p) + static_cast<uint64_t>(d) - 1) / static_cast<uint64_t>(d));
    f.shr       = static_cast<uint32_t>(p - 32);
    return f;
}

__device__ __forceinline__ int fast_div(int n, const FastDiv &f)
{
    return f.d <= 1 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), f.mul) >> f.shr);
}

__device__ __forceinline__ int32_t load_q8(const void *p, size_t idx, bool is_signed)
{
    return is_signed ? static_cast<int32_t>(static_cast<const int8_t *>(p)[idx])
                     : static_cast<int32_t>(static_cast<const uint8_t *>(p)[idx]);
}
} // namespace cugl
