// TEST INFRASTRUCTURE ONLY — not part of the shipped library.
//
// Second translation unit of oracle/_ref/libacl_ref.so: C-ABI wrappers around the scalar test oracles of
// the quantized layers that sit between the convolutions of a QASYMM8 network.  As in ref_shim.cpp the
// reference translation units are #included in place from an unmodified Compute Library tree; nothing is copied.
//
// Wrapped reference entry points (all QASYMM8 = uint8_t: dequantize -> float operator -> quantize):
//   reference::pooling_layer<uint8_t>            tests/validation/reference/PoolingLayer.cpp:40-196, 218-230
//   reference::arithmetic_operation<uint8_t>     tests/validation/reference/ArithmeticOperations.cpp:124-151
//   reference::activation_layer<uint8_t>         tests/validation/reference/ActivationLayer.cpp:61-71
//   reference::softmax_layer<uint8_t>            tests/validation/reference/SoftmaxLayer.cpp:39-107, 201-213
//   convert_from_asymmetric / convert_to_asymmetric  tests/validation/Helpers.cpp:89-102 and the header
#include "tests/framework/Asserts.h"
// The reference files use the test framework's assertion macros on a few indices; replace only the
// mechanism so that the test runner is not dragged into the link.
#undef ARM_COMPUTE_ASSERT
#define ARM_COMPUTE_ASSERT(X)                        \
    do                                               \
    {                                                \
        if (!(X))                                    \
        {                                            \
            throw std::runtime_error("assert: " #X); \
        }                                            \
    } while (false)
#undef ARM_COMPUTE_EXPECT
#define ARM_COMPUTE_EXPECT(X, LEVEL)                 \
    do                                               \
    {                                                \
        if (!(X))                                    \
        {                                            \
            throw std::runtime_error("expect: " #X); \
        }                                            \
    } while (false)
#include "tests/validation/Helpers.cpp"                        // NOLINT: in-place inclusion on purpose
#include "tests/validation/reference/ActivationLayer.cpp"      // NOLINT
#include "tests/validation/reference/ArithmeticOperations.cpp" // NOLINT
#include "tests/validation/reference/DequantizationLayer.cpp"  // NOLINT
#include "tests/validation/reference/PoolingLayer.cpp"         // NOLINT
#include "tests/validation/reference/SoftmaxLayer.cpp"         // NOLINT

#include <cstring>

using namespace arm_compute;
using namespace arm_compute::test;
using namespace arm_compute::test::validation;

// Link-only definitions: Helpers.cpp refers to the CPU feature probe and to the test runner's global
// assets library in functions that are never called through this file.
namespace arm_compute
{
CPUInfo &CPUInfo::get()
{
    throw std::runtime_error("CPUInfo is not part of this oracle build");
}
bool CPUInfo::has_bf16() const
{
    return false;
}
bool CPUInfo::has_fp16() const
{
    return false;
}
namespace test
{
std::unique_ptr<AssetsLibrary>  library;
std::random_device::result_type AssetsLibrary::seed() const
{
    return 0;
}
} // namespace test
} // namespace arm_compute

namespace
{
// [B][H][W][C] bytes <-> the oracle's NCHW SimpleTensor (shape [W,H,C,B], x fastest)
SimpleTensor<uint8_t> nhwc_to_tensor(const uint8_t *src, int C, int W, int H, int B, float scale, int zp)
{
    SimpleTensor<uint8_t> t(TensorShape(W, H, C, B), DataType::QASYMM8, 1, QuantizationInfo(scale, zp));
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x)
                for (int c = 0; c < C; ++c)
                    t[((size_t(b) * C + c) * H + y) * W + x] = src[((size_t(b) * H + y) * W + x) * C + c];
    return t;
}
void tensor_to_nhwc(const SimpleTensor<uint8_t> &t, uint8_t *dst, int C, int W, int H, int B)
{
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x)
                for (int c = 0; c < C; ++c)
                    dst[((size_t(b) * H + y) * W + x) * C + c] = t[((size_t(b) * C + c) * H + y) * W + x];
}
} // namespace

extern "C"
{
    // pool_type: 0 = MAX, 1 = AVG.  global != 0: the window is the whole image (pw, ph, strides and pads ignored).
    // dst is [B][Ho][Wo][C] with the reference's own output-shape rule (floor rounding).
    void ref_pool_nhwc_u8(const uint8_t *src, uint8_t *dst, int C, int W, int H, int B, int pool_type, int pw, int ph,
                          int sx, int sy, int pl, int pr, int pt, int pb, int exclude_padding, int global,
                          float in_scale, int in_zp, float out_scale, int out_zp, int *out_w, int *out_h)
    {
        SimpleTensor<uint8_t> ts = nhwc_to_tensor(src, C, W, H, B, in_scale, in_zp);
        const PoolingType     pt_ = pool_type == 0 ? PoolingType::MAX : PoolingType::AVG;
        PoolingLayerInfo      info =
            global ? PoolingLayerInfo(pt_, DataLayout::NCHW)
                        : PoolingLayerInfo(pt_, Size2D(pw, ph), DataLayout::NCHW,
                                           PadStrideInfo(sx, sy, pl, pr, pt, pb, DimensionRoundingType::FLOOR),
                                           exclude_padding != 0);
        SimpleTensor<uint8_t> td =
            reference::pooling_layer<uint8_t>(ts, info, QuantizationInfo(out_scale, out_zp), nullptr, DataLayout::NCHW);
        const int Wo = td.shape()[0], Ho = td.shape()[1];
        if (out_w) *out_w = Wo;
        if (out_h) *out_h = Ho;
        if (dst) tensor_to_nhwc(td, dst, C, Wo, Ho, B);
    }

    void ref_add_qasymm8(const uint8_t *a, const uint8_t *b, uint8_t *dst, long long n, float a_scale, int a_zp,
                         float b_scale, int b_zp, float o_scale, int o_zp)
    {
        SimpleTensor<uint8_t> ta(TensorShape(n), DataType::QASYMM8, 1, QuantizationInfo(a_scale, a_zp));
        SimpleTensor<uint8_t> tb(TensorShape(n), DataType::QASYMM8, 1, QuantizationInfo(b_scale, b_zp));
        SimpleTensor<uint8_t> td(TensorShape(n), DataType::QASYMM8, 1, QuantizationInfo(o_scale, o_zp));
        std::memcpy(ta.data(), a, n);
        std::memcpy(tb.data(), b, n);
        reference::arithmetic_operation<uint8_t>(reference::ArithmeticOperation::ADD, ta, tb, td, ConvertPolicy::SATURATE);
        std::memcpy(dst, td.data(), n);
    }

    // act: 0 = RELU, 1 = BOUNDED_RELU(a), 2 = LU_BOUNDED_RELU(a upper, b lower)
    void ref_activation_qasymm8(const uint8_t *src, uint8_t *dst, long long n, int act, float a, float b,
                                float in_scale, int in_zp, float out_scale, int out_zp)
    {
        SimpleTensor<uint8_t> ts(TensorShape(n), DataType::QASYMM8, 1, QuantizationInfo(in_scale, in_zp));
        std::memcpy(ts.data(), src, n);
        const ActivationLayerInfo::ActivationFunction f =
            act == 0   ? ActivationLayerInfo::ActivationFunction::RELU
            : act == 1 ? ActivationLayerInfo::ActivationFunction::BOUNDED_RELU
                       : ActivationLayerInfo::ActivationFunction::LU_BOUNDED_RELU;
        SimpleTensor<uint8_t> td =
            reference::activation_layer<uint8_t>(ts, ActivationLayerInfo(f, a, b), QuantizationInfo(out_scale, out_zp));
        std::memcpy(dst, td.data(), n);
    }

    // rows x cols, softmax along the contiguous axis; output quantization is the reference's fixed (1/256, 0)
    void ref_softmax_qasymm8(const uint8_t *src, uint8_t *dst, int rows, int cols, float beta, float in_scale, int in_zp)
    {
        SimpleTensor<uint8_t> ts(TensorShape(cols, rows), DataType::QASYMM8, 1, QuantizationInfo(in_scale, in_zp));
        std::memcpy(ts.data(), src, size_t(rows) * cols);
        SimpleTensor<uint8_t> td = reference::softmax_layer<uint8_t>(ts, beta, 0, false);
        std::memcpy(dst, td.data(), size_t(rows) * cols);
    }
    // The dequantised GEMMLowp output as the reference's fixture computes it (GEMMLowpFixture.h:898-921):
    // reference::dequantization_layer<float, int32_t> of the S32 result carrying (scale, 0), then -- accumulate != 0 --
    // reference::arithmetic_operation<float>(ADD, previous, result, SATURATE).  inout holds the previous output on
    // entry when accumulating and the result on return.
    void ref_dequantize_s32_f32(const int32_t *acc, float *inout, long long n, float scale, int accumulate)
    {
        SimpleTensor<int32_t> in{TensorShape(static_cast<size_t>(n)), DataType::S32, 1, QuantizationInfo(scale, 0)};
        std::memcpy(in.data(), acc, sizeof(int32_t) * n);
        SimpleTensor<float> deq = reference::dequantization_layer<float, int32_t>(in);
        if (accumulate != 0)
        {
            SimpleTensor<float> prev{TensorShape(static_cast<size_t>(n)), DataType::F32, 1};
            std::memcpy(prev.data(), inout, sizeof(float) * n);
            SimpleTensor<float> sum{TensorShape(static_cast<size_t>(n)), DataType::F32, 1};
            reference::arithmetic_operation<float>(reference::ArithmeticOperation::ADD, prev, deq, sum, ConvertPolicy::SATURATE);
            std::memcpy(inout, sum.data(), sizeof(float) * n);
        }
        else
        {
            std::memcpy(inout, deq.data(), sizeof(float) * n);
        }
    }
}
