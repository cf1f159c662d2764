// Self-test of the C++ function family, written the way the reference's own examples / fixtures drive the NE
// functions (examples/neon_gemm_qasymm8.cpp:200-246, tests/validation/fixtures/GEMMLowpFixture.h:239-346):
// configure -> allocate -> fill (std::mt19937) -> run -> compare with the CPU oracle (oracle/gemmlowp_oracle.c).
//   test_cu_functions --validate   host-only checks of validate() (no GPU needed)
//   test_cu_functions              everything, on cuda:0
#include "arm_compute/core/Utils.h"
#include "arm_compute/runtime/CUDA/CUAllocator.h"
#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"
#include "arm_compute/runtime/MemoryGroup.h"
#include "arm_compute/runtime/Tensor.h"
#include "arm_compute/runtime/CUDA/functions/CUFullyConnectedLayer.h"
#include "arm_compute/runtime/CUDA/functions/CUGEMMConvolutionLayer.h"
#include "arm_compute/runtime/CUDA/functions/CUGEMMLowpMatrixMultiplyCore.h"
#include "arm_compute/runtime/CUDA/functions/CUGEMMLowpOutputStage.h"
#include "arm_compute/runtime/CUDA/functions/CUQuantizedLayers.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

using namespace arm_compute;

extern "C"
{
    // test oracle (oracle/gemmlowp_oracle.c)
    void orc_gemmlowp_core(const void *a, int a_signed, const void *b, int b_signed, int32_t *c, int M, int N, int K,
                           int batch, int b_batched, int32_t a_off, int32_t b_off);
    void orc_gemmlowp_fused(const void *a, int a_signed, const void *b, int b_signed, const int32_t *bias, void *out,
                            int out_signed, int M, int N, int K, int32_t a_off, int32_t b_off, const int32_t *mult,
                            const int32_t *shift, int n_mult, int32_t offset, int32_t lo, int32_t hi);
    void orc_output_stage_s16(const int32_t *in, const int32_t *bias, int16_t *out, int M, int N, const int32_t *mult,
                              const int32_t *shift, int n_mult, int32_t offset, int32_t lo, int32_t hi);
    void orc_conv2d_nhwc(const void *src, int src_signed, const void *weights, int w_signed, const int32_t *bias,
                         void *dst, int C, int W, int H, int B, int kw, int kh, int OFM, int sx, int sy, int pad_l,
                         int pad_t, int dil_x, int dil_y, int Wo, int Ho, int32_t in_zp, int32_t w_zp,
                         const int32_t *mult, const int32_t *shift, int n_mult, int32_t out_offset, int32_t lo,
                         int32_t hi);
    // oracle/layers_oracle.c
    void orc_pool_nhwc_u8(const uint8_t *src, uint8_t *dst, int C, int W, int H, int B, int pool_type, int pw, int ph,
                          int sx, int sy, int pl, int pr, int pt, int pb, int exclude_padding, int Wo, int Ho,
                          float in_scale, int in_zp, float out_scale, int out_zp);
    void orc_add_qasymm8(const uint8_t *a, const uint8_t *b, uint8_t *dst, long long n, float a_scale, int a_zp,
                         float b_scale, int b_zp, float o_scale, int o_zp);
    void orc_activation_qasymm8(const uint8_t *src, uint8_t *dst, long long n, int act, float a, float b,
                                float in_scale, int in_zp, float out_scale, int out_zp);
    void orc_softmax_qasymm8(const uint8_t *src, uint8_t *dst, int rows, int cols, float beta, float in_scale,
                             int in_zp);
}

static int g_failures = 0;
#define CHECK(cond)                                                        \
    do                                                                     \
    {                                                                      \
        if (!(cond))                                                       \
        {                                                                  \
            std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond);  \
            ++g_failures;                                                  \
        }                                                                  \
    } while (false)

template <typename T>
static void fill_uniform(std::vector<T> &v, int lo, int hi, unsigned seed)
{
    std::mt19937                       gen(seed);
    std::uniform_int_distribution<int> dist(lo, hi);
    for (auto &x : v) x = static_cast<T>(dist(gen));
}

template <typename T>
static void upload(CUTensor &t, const std::vector<T> &v)
{
    t.map();
    std::memcpy(t.buffer(), v.data(), v.size() * sizeof(T));
    t.unmap();
}

template <typename T>
static std::vector<T> download(CUTensor &t, size_t n)
{
    std::vector<T> v(n);
    t.map();
    std::memcpy(v.data(), t.buffer(), n * sizeof(T));
    return v;
}

static void test_validate()
{
    const TensorInfo a(TensorShape(256U, 64U), 1, DataType::QASYMM8, QuantizationInfo(0.02f, -128));
    const TensorInfo b(TensorShape(128U, 256U), 1, DataType::QASYMM8, QuantizationInfo(0.005f, -120));
    const TensorInfo bias(TensorShape(128U), 1, DataType::S32);
    const TensorInfo out_s32(TensorShape(128U, 64U), 1, DataType::S32);
    const TensorInfo out_u8(TensorShape(128U, 64U), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 10));
    GEMMInfo         plain;
    CHECK(bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b, nullptr, &out_s32, plain)));
    // bias without an output stage (CpuGemmLowpMatrixMultiplyCore.cpp:376-378)
    CHECK(!bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b, &bias, &out_s32, plain)));
    // K mismatch
    const TensorInfo b_bad(TensorShape(128U, 255U), 1, DataType::QASYMM8);
    CHECK(!bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b_bad, nullptr, &out_s32, plain)));
    // reshaped operands are refused
    const GEMMInfo reshaped(true, false, false);
    CHECK(!bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b, nullptr, &out_s32, reshaped)));
    // fused stage
    GEMMLowpOutputStageInfo stage;
    stage.type                = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    stage.gemmlowp_multiplier = 1099511552;
    stage.gemmlowp_shift      = 8;
    stage.gemmlowp_offset     = 10;
    stage.gemmlowp_min_bound  = 0;
    stage.gemmlowp_max_bound  = 255;
    GEMMInfo fused;
    fused.set_gemmlowp_output_stage(stage);
    CHECK(bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b, &bias, &out_u8, fused)));
    CHECK(!bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b, &bias, &out_s32, fused))); // stage needs 8-bit dst
    stage.gemmlowp_min_bound = 300;
    fused.set_gemmlowp_output_stage(stage);
    CHECK(!bool(CUGEMMLowpMatrixMultiplyCore::validate(&a, &b, &bias, &out_u8, fused))); // min > max
    // stand-alone output stage
    stage.gemmlowp_min_bound = 0;
    CHECK(bool(CUGEMMLowpOutputStage::validate(&out_s32, &bias, &out_u8, stage)));
    CHECK(!bool(CUGEMMLowpOutputStage::validate(&out_u8, &bias, &out_u8, stage)));
    // convolution
    TensorInfo src(TensorShape(64U, 56U, 56U, 2U), 1, DataType::QASYMM8, QuantizationInfo(0.03f, 128));
    src.set_data_layout(DataLayout::NHWC);
    TensorInfo wgt(TensorShape(64U, 3U, 3U, 64U), 1, DataType::QSYMM8_PER_CHANNEL, QuantizationInfo(std::vector<float>(64, 0.004f)));
    wgt.set_data_layout(DataLayout::NHWC);
    TensorInfo cb(TensorShape(64U), 1, DataType::S32);
    TensorInfo dst(TensorShape(64U, 56U, 56U, 2U), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 0));
    dst.set_data_layout(DataLayout::NHWC);
    CHECK(bool(CUGEMMConvolutionLayer::validate(&src, &wgt, &cb, &dst, PadStrideInfo(1, 1, 1, 1))));
    CHECK(!bool(CUGEMMConvolutionLayer::validate(&src, &wgt, &cb, &dst, PadStrideInfo(1, 1, 0, 0)))); // wrong out shape
    CHECK(!bool(CUGEMMConvolutionLayer::validate(&src, &wgt, &cb, &dst, PadStrideInfo(1, 1, 1, 1), WeightsInfo(),
                                                 Size2D(1U, 1U), ActivationLayerInfo(), false, 2))); // groups
    const auto mm = get_quantized_activation_min_max(
        ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::LU_BOUNDED_RELU, 6.f, 1.f), DataType::QASYMM8,
        UniformQuantizationInfo(0.05f, 10));
    CHECK(mm.first == 30 && mm.second == 130);
}

// examples/neon_gemm_qasymm8.cpp: core to S32, then the output stage; and the fused form.
static void test_gemmlowp_config1()
{
    const int            M = 64, N = 128, K = 256;
    std::vector<uint8_t> ha(size_t(M) * K), hb(size_t(K) * N);
    std::vector<int32_t> hbias(N);
    fill_uniform(ha, 0, 255, 1);
    fill_uniform(hb, 0, 255, 2);
    fill_uniform(hbias, -2000, 2000, 3);
    int32_t mult = 0, shift = 0;
    CHECK(cugl_calculate_quantized_multiplier(0.02f * 0.005f / 0.05f, &mult, &shift) == CUGL_SUCCESS);
    CHECK(mult == 1099511552 && shift == 8);

    CUTensor a, b, bias, acc, out, out_fused;
    a.allocator()->init(TensorInfo(TensorShape(K, M), 1, DataType::QASYMM8, QuantizationInfo(0.02f, -128)));
    b.allocator()->init(TensorInfo(TensorShape(N, K), 1, DataType::QASYMM8, QuantizationInfo(0.005f, -120)));
    bias.allocator()->init(TensorInfo(TensorShape(N), 1, DataType::S32));
    acc.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::S32));
    out.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 10)));
    out_fused.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 10)));

    GEMMLowpOutputStageInfo stage;
    stage.type                = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    stage.gemmlowp_multiplier = mult;
    stage.gemmlowp_shift      = shift;
    stage.gemmlowp_offset     = 10;
    stage.gemmlowp_min_bound  = 0;
    stage.gemmlowp_max_bound  = 255;
    stage.output_data_type    = DataType::QASYMM8;

    // the same accumulators through the QSYMM16 variant of the stage (no offset, whole int16 range)
    CUTensor out16;
    out16.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::QSYMM16, QuantizationInfo(0.001f, 0)));
    GEMMLowpOutputStageInfo stage16 = stage;
    stage16.gemmlowp_shift          = 2;
    stage16.gemmlowp_offset         = 0;
    stage16.gemmlowp_min_bound      = -32768;
    stage16.gemmlowp_max_bound      = 32767;
    stage16.output_data_type        = DataType::QSYMM16;
    GEMMLowpOutputStageInfo bad16   = stage16;
    bad16.type                      = GEMMLowpOutputStageType::QUANTIZE_DOWN;
    CHECK(bool(CUGEMMLowpOutputStage::validate(acc.info(), bias.info(), out16.info(), stage16)));
    CHECK(!bool(CUGEMMLowpOutputStage::validate(acc.info(), bias.info(), out16.info(), bad16)));

    CUGEMMLowpMatrixMultiplyCore core;
    core.configure(&a, &b, nullptr, &acc);
    CUGEMMLowpOutputStage os, os16;
    os.configure(&acc, &bias, &out, stage);
    os16.configure(&acc, &bias, &out16, stage16);
    CUGEMMLowpMatrixMultiplyCore fused;
    GEMMInfo                     info;
    info.set_gemmlowp_output_stage(stage);
    fused.configure(&a, &b, &bias, &out_fused, info);

    // allocation after configure, as the library requires
    for (CUTensor *t : {&a, &b, &bias, &acc, &out, &out_fused, &out16}) t->allocator()->allocate();
    upload(a, ha);
    upload(b, hb);
    upload(bias, hbias);
    core.run();
    os.run();
    os16.run();
    fused.run();
    fused.run(); // MultipleExecution: same output
    CUScheduler::get().sync();

    std::vector<int32_t> want_acc(size_t(M) * N);
    orc_gemmlowp_core(ha.data(), 0, hb.data(), 0, want_acc.data(), M, N, K, 1, 0, -128, -120);
    std::vector<uint8_t> want(size_t(M) * N);
    orc_gemmlowp_fused(ha.data(), 0, hb.data(), 0, hbias.data(), want.data(), 0, M, N, K, -128, -120, &mult, &shift, 1,
                       10, 0, 255);
    CHECK(download<int32_t>(acc, want_acc.size()) == want_acc);
    CHECK(download<uint8_t>(out, want.size()) == want);
    CHECK(download<uint8_t>(out_fused, want.size()) == want);
    std::vector<int16_t> want16(size_t(M) * N);
    const int32_t        shift16 = 2;
    orc_output_stage_s16(want_acc.data(), hbias.data(), want16.data(), M, N, &mult, &shift16, 1, 0, -32768, 32767);
    CHECK(download<int16_t>(out16, want16.size()) == want16);

    // update_quantization_parameters: new scales / offsets, recomputed stage
    a.info()->set_quantization_info(QuantizationInfo(0.03f, -100));
    b.info()->set_quantization_info(QuantizationInfo(0.004f, -90));
    out_fused.info()->set_quantization_info(QuantizationInfo(0.07f, 3));
    fused.update_quantization_parameters();
    fused.run();
    CUScheduler::get().sync();
    int32_t m2 = 0, s2 = 0;
    cugl_calculate_quantized_multiplier(0.03f * 0.004f / 0.07f, &m2, &s2);
    orc_gemmlowp_fused(ha.data(), 0, hb.data(), 0, hbias.data(), want.data(), 0, M, N, K, -100, -90, &m2, &s2, 1, 3, 0,
                       255);
    CHECK(download<uint8_t>(out_fused, want.size()) == want);
}

// Config-3-shaped convolution at a small batch with a fused ReLU (NEGEMMConvolutionLayer).
static void test_convolution()
{
    const int            B = 2, H = 28, W = 28, C = 64, OFM = 64, k = 3;
    std::vector<uint8_t> hsrc(size_t(B) * H * W * C);
    std::vector<int8_t>  hw(size_t(OFM) * k * k * C);
    std::vector<int32_t> hbias(OFM);
    std::vector<float>   scales(OFM);
    fill_uniform(hsrc, 0, 255, 11);
    fill_uniform(hw, -127, 127, 12);
    fill_uniform(hbias, -5000, 5000, 13);
    std::mt19937                          gen(14);
    std::uniform_real_distribution<float> sd(2e-3f, 8e-3f);
    for (auto &s : scales) s = sd(gen);

    CUTensor   src, wgt, bias, dst;
    TensorInfo si(TensorShape(C, W, H, B), 1, DataType::QASYMM8, QuantizationInfo(0.03f, 128));
    si.set_data_layout(DataLayout::NHWC);
    TensorInfo wi(TensorShape(C, k, k, OFM), 1, DataType::QSYMM8_PER_CHANNEL, QuantizationInfo(scales));
    wi.set_data_layout(DataLayout::NHWC);
    TensorInfo di(TensorShape(OFM, W, H, B), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 0));
    di.set_data_layout(DataLayout::NHWC);
    src.allocator()->init(si);
    wgt.allocator()->init(wi);
    bias.allocator()->init(TensorInfo(TensorShape(OFM), 1, DataType::S32));
    dst.allocator()->init(di);

    CUGEMMConvolutionLayer conv;
    conv.configure(&src, &wgt, &bias, &dst, PadStrideInfo(1, 1, 1, 1), WeightsInfo(), Size2D(1U, 1U),
                   ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU));
    for (CUTensor *t : {&src, &wgt, &bias, &dst}) t->allocator()->allocate();
    upload(src, hsrc);
    upload(wgt, hw);
    upload(bias, hbias);
    conv.run();
    CUScheduler::get().sync();
    CHECK(!wgt.is_used()); // weights are consumed by prepare()

    std::vector<int32_t> mult(OFM), shift(OFM);
    cugl_calculate_quantized_multipliers(0.03f, scales.data(), OFM, 0.05f, mult.data(), shift.data());
    std::vector<uint8_t> want(size_t(B) * H * W * OFM);
    orc_conv2d_nhwc(hsrc.data(), 0, hw.data(), 1, hbias.data(), want.data(), C, W, H, B, k, k, OFM, 1, 1, 1, 1, 1, 1, W,
                    H, 128, 0, mult.data(), shift.data(), OFM, 0, 0, 255);
    CHECK(download<uint8_t>(dst, want.size()) == want);
}

static TensorInfo u8_nhwc(const TensorShape &shape, float scale, int zp)
{
    TensorInfo t(shape, 1, DataType::QASYMM8, QuantizationInfo(scale, zp));
    t.set_data_layout(DataLayout::NHWC);
    return t;
}

static void test_validate_layers()
{
    TensorInfo in  = u8_nhwc(TensorShape(64, 112, 112, 2), 0.05f, 0);
    TensorInfo out = u8_nhwc(TensorShape(64, 56, 56, 2), 0.05f, 0);
    const PoolingLayerInfo pool1(PoolingType::MAX, 3, DataLayout::NHWC, PadStrideInfo(2, 2, 0, 1, 0, 1, DimensionRoundingType::FLOOR));
    CHECK(bool(CUPoolingLayer::validate(&in, &out, pool1)));
    CHECK(!bool(CUPoolingLayer::validate(&in, &in, pool1)));                                   // wrong output shape
    CHECK(!bool(CUPoolingLayer::validate(&in, &out, PoolingLayerInfo(PoolingType::L2, 3, DataLayout::NHWC,
                                                                     PadStrideInfo(2, 2, 0, 1, 0, 1, DimensionRoundingType::FLOOR)))));
    TensorInfo g_out = u8_nhwc(TensorShape(64, 1, 1, 2), 0.05f, 0);
    CHECK(bool(CUPoolingLayer::validate(&in, &g_out, PoolingLayerInfo(PoolingType::AVG, DataLayout::NHWC))));
    CHECK(bool(CUArithmeticAddition::validate(&in, &in, &in, ConvertPolicy::SATURATE,
                                              ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU))));
    CHECK(!bool(CUArithmeticAddition::validate(&in, &in, &in, ConvertPolicy::WRAP)));
    CHECK(!bool(CUArithmeticAddition::validate(&in, &out, &in, ConvertPolicy::SATURATE)));      // no broadcasting
    CHECK(bool(CUActivationLayer::validate(&in, nullptr, ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::BOUNDED_RELU, 6.f))));
    CHECK(!bool(CUActivationLayer::validate(&in, nullptr, ActivationLayerInfo())));
    TensorInfo logits(TensorShape(1000, 4), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 0));
    TensorInfo probs(TensorShape(1000, 4), 1, DataType::QASYMM8, QuantizationInfo(1.f / 256.f, 0));
    CHECK(bool(CUSoftmaxLayer::validate(&logits, &probs)));
    CHECK(!bool(CUSoftmaxLayer::validate(&logits, &logits)));                                   // output quantization is fixed
    CHECK(!bool(CUSoftmaxLayer::validate(&logits, &probs, 1.f, 1)));
}

// pool1 -> (x + x') -> ReLU -> bounded ReLU -> global average -> softmax, every step against the oracle
static void test_layers()
{
    const int C = 32, W = 20, H = 18, B = 2, Wo = 10, Ho = 9;
    const float s = 0.05f;
    CUTensor src, pooled, other, sum, act, avg, probs;
    src.allocator()->init(u8_nhwc(TensorShape(C, W, H, B), s, 3));
    pooled.allocator()->init(u8_nhwc(TensorShape(C, Wo, Ho, B), 0.06f, 5));
    other.allocator()->init(u8_nhwc(TensorShape(C, Wo, Ho, B), 0.04f, 9));
    sum.allocator()->init(u8_nhwc(TensorShape(C, Wo, Ho, B), 0.07f, 12));
    act.allocator()->init(u8_nhwc(TensorShape(C, Wo, Ho, B), 0.07f, 12));
    avg.allocator()->init(u8_nhwc(TensorShape(C, 1, 1, B), 0.07f, 12));
    TensorInfo pinfo(TensorShape(C, B), 1, DataType::QASYMM8, QuantizationInfo(1.f / 256.f, 0));
    probs.allocator()->init(pinfo);
    CUPoolingLayer       pool, gap;
    CUArithmeticAddition add;
    CUActivationLayer    relu6;
    CUSoftmaxLayer       softmax;
    pool.configure(&src, &pooled, PoolingLayerInfo(PoolingType::MAX, 3, DataLayout::NHWC,
                                                   PadStrideInfo(2, 2, 0, 1, 0, 1, DimensionRoundingType::FLOOR)));
    add.configure(&pooled, &other, &sum, ConvertPolicy::SATURATE,
                  ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU));
    relu6.configure(&sum, &act, ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::BOUNDED_RELU, 6.f));
    gap.configure(&act, &avg, PoolingLayerInfo(PoolingType::AVG, DataLayout::NHWC));
    // softmax over the channels of the pooled vector: view avg [C,1,1,B] as [C,B]
    CUTensor avg2d;
    TensorInfo a2(TensorShape(C, B), 1, DataType::QASYMM8, QuantizationInfo(0.07f, 12));
    avg2d.allocator()->init(a2);
    for (CUTensor *t : {&src, &pooled, &other, &sum, &act, &avg, &probs}) t->allocator()->allocate();
    avg2d.allocator()->import_memory(avg.device_ptr());
    softmax.configure(&avg2d, &probs);
    std::vector<uint8_t> hsrc(size_t(B) * H * W * C), hother(size_t(B) * Ho * Wo * C);
    fill_uniform(hsrc, 0, 255, 11);
    fill_uniform(hother, 0, 255, 12);
    upload(src, hsrc);
    upload(other, hother);
    pool.run();
    add.run();
    relu6.run();
    gap.run();
    softmax.run();
    CUScheduler::get().sync();

    const size_t n = size_t(B) * Ho * Wo * C;
    std::vector<uint8_t> w_pool(n), w_sum(n), w_relu(n), w_act(n), w_avg(size_t(B) * C), w_probs(size_t(B) * C);
    orc_pool_nhwc_u8(hsrc.data(), w_pool.data(), C, W, H, B, 0, 3, 3, 2, 2, 0, 1, 0, 1, 0, Wo, Ho, s, 3, 0.06f, 5);
    orc_add_qasymm8(w_pool.data(), hother.data(), w_sum.data(), (long long)n, 0.06f, 5, 0.04f, 9, 0.07f, 12);
    orc_activation_qasymm8(w_sum.data(), w_relu.data(), (long long)n, 0, 0.f, 0.f, 0.07f, 12, 0.07f, 12);
    orc_activation_qasymm8(w_relu.data(), w_act.data(), (long long)n, 1, 6.f, 0.f, 0.07f, 12, 0.07f, 12);
    orc_pool_nhwc_u8(w_act.data(), w_avg.data(), C, Wo, Ho, B, 1, Wo, Ho, 1, 1, 0, 0, 0, 0, 0, 1, 1, 0.07f, 12, 0.07f, 12);
    orc_softmax_qasymm8(w_avg.data(), w_probs.data(), B, C, 1.f, 0.07f, 12);
    CHECK(download<uint8_t>(pooled, n) == w_pool);
    CHECK(download<uint8_t>(sum, n) == w_relu);
    CHECK(download<uint8_t>(act, n) == w_act);
    CHECK(download<uint8_t>(avg, w_avg.size()) == w_avg);
    const std::vector<uint8_t> got = download<uint8_t>(probs, w_probs.size());
    int worst = 0;
    for (size_t i = 0; i < got.size(); ++i) worst = std::max(worst, std::abs(int(got[i]) - int(w_probs[i])));
    CHECK(worst <= 1);
}

// NEFullyConnectedLayer semantics: logits = x * W^T + b on a [num_inputs, batch] input, both weight layouts
static void test_fully_connected()
{
    const int K = 512, N = 200, B = 37;
    std::vector<uint8_t> hx(size_t(B) * K);
    std::vector<int8_t>  hw(size_t(N) * K); // one row per output neuron
    std::vector<int32_t> hb(N);
    fill_uniform(hx, 0, 255, 21);
    fill_uniform(hw, -127, 127, 22);
    fill_uniform(hb, -3000, 3000, 23);
    std::vector<int8_t> hw_t(size_t(K) * N), b_kn(size_t(K) * N); // [K][N]
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) b_kn[size_t(k) * N + n] = hw_t[size_t(k) * N + n] = hw[size_t(n) * K + k];
    int32_t mult = 0, shift = 0;
    CHECK(cugl_calculate_quantized_multiplier(0.05f * 0.004f / 0.1f, &mult, &shift) == CUGL_SUCCESS);
    std::vector<uint8_t> want(size_t(B) * N);
    // offsets as the operator passes them to the core: negated zero points; ReLU = clamp at the output zero point
    orc_gemmlowp_fused(hx.data(), 0, b_kn.data(), 1, hb.data(), want.data(), 0, B, N, K, -7, 0, &mult, &shift, 1, 20, 20, 255);
    for (int transposed = 1; transposed >= 0; --transposed)
    {
        CUTensor x, w, b, y;
        x.allocator()->init(TensorInfo(TensorShape(K, B), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 7)));
        w.allocator()->init(TensorInfo(transposed ? TensorShape(K, N) : TensorShape(N, K), 1, DataType::QSYMM8,
                                       QuantizationInfo(0.004f, 0)));
        b.allocator()->init(TensorInfo(TensorShape(N), 1, DataType::S32));
        y.allocator()->init(TensorInfo(TensorShape(N, B), 1, DataType::QASYMM8, QuantizationInfo(0.1f, 20)));
        FullyConnectedLayerInfo info;
        info.transpose_weights = transposed != 0;
        info.activation_info   = ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU);
        CHECK(bool(CUFullyConnectedLayer::validate(x.info(), w.info(), b.info(), y.info(), info)));
        CUFullyConnectedLayer fc;
        fc.configure(&x, &w, &b, &y, info);
        for (CUTensor *t : {&x, &w, &b, &y}) t->allocator()->allocate();
        upload(x, hx);
        upload(w, transposed ? hw : hw_t);
        upload(b, hb);
        fc.run();
        fc.run();
        CUScheduler::get().sync();
        CHECK(download<uint8_t>(y, want.size()) == want);
    }
    TensorInfo bad_w(TensorShape(K + 16, N), 1, DataType::QSYMM8, QuantizationInfo(0.004f, 0));
    TensorInfo xi(TensorShape(K, B), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 7));
    TensorInfo yi(TensorShape(N, B), 1, DataType::QASYMM8, QuantizationInfo(0.1f, 20));
    CHECK(!bool(CUFullyConnectedLayer::validate(&xi, &bad_w, nullptr, &yi)));
}


// ---- host tensors with padding: the fixtures add padding after configure() (GEMMLowpFixture.h:302) -----------------
// element (x, y) of a 2-D host tensor
template <typename T>
static T &at(Tensor &t, int x, int y)
{
    return *reinterpret_cast<T *>(t.ptr_to_element(Coordinates(x, y)));
}

static void test_host_tensors_with_padding()
{
    const int            M = 37, N = 72, K = 96;
    std::vector<uint8_t> ha(size_t(M) * K), hb(size_t(K) * N);
    std::vector<int32_t> hbias(N);
    fill_uniform(ha, 0, 255, 31);
    fill_uniform(hb, 0, 255, 32);
    fill_uniform(hbias, -2000, 2000, 33);
    GEMMLowpOutputStageInfo stage;
    stage.type                = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    stage.gemmlowp_multiplier = 1099511552;
    stage.gemmlowp_shift      = 8;
    stage.gemmlowp_offset     = 10;
    stage.gemmlowp_min_bound  = 0;
    stage.gemmlowp_max_bound  = 255;
    stage.output_data_type    = DataType::QASYMM8;
    Tensor a, b, bias, out; // plain host tensors: the function stages them
    a.allocator()->init(TensorInfo(TensorShape(K, M), 1, DataType::QASYMM8, QuantizationInfo(0.02f, -128)));
    b.allocator()->init(TensorInfo(TensorShape(N, K), 1, DataType::QASYMM8, QuantizationInfo(0.005f, -120)));
    bias.allocator()->init(TensorInfo(TensorShape(N), 1, DataType::S32));
    out.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 10)));
    CUGEMMLowpMatrixMultiplyCore fused;
    GEMMInfo                     info;
    info.set_gemmlowp_output_stage(stage);
    fused.configure(&a, &b, &bias, &out, info);
    // padding appears after configure, as in the validation fixtures: row pitches and the first-element offset change
    a.info()->extend_padding(PaddingSize(0, 5, 0, 3));
    b.info()->extend_padding(PaddingSize(0, 11, 0, 0));
    out.info()->extend_padding(PaddingSize(0, 7, 0, 2));
    for (Tensor *t : {&a, &b, &bias, &out}) t->allocator()->allocate();
    std::memset(out.buffer(), 0xEE, out.info()->total_size());
    for (int m = 0; m < M; ++m)
        for (int k = 0; k < K; ++k) at<uint8_t>(a, k, m) = ha[size_t(m) * K + k];
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; ++n) at<uint8_t>(b, n, k) = hb[size_t(k) * N + n];
    std::memcpy(bias.buffer(), hbias.data(), hbias.size() * 4);
    fused.run(); // blocks for a host output
    std::vector<uint8_t> want(size_t(M) * N);
    const int32_t        mult = 1099511552, shift = 8;
    orc_gemmlowp_fused(ha.data(), 0, hb.data(), 0, hbias.data(), want.data(), 0, M, N, K, -128, -120, &mult, &shift, 1,
                       10, 0, 255);
    bool equal = true;
    for (int m = 0; m < M && equal; ++m)
        for (int n = 0; n < N; ++n) equal = equal && at<uint8_t>(out, n, m) == want[size_t(m) * N + n];
    CHECK(equal);
    // the padding bytes of the host output were left alone
    const size_t pitch = out.info()->strides_in_bytes()[1], off0 = out.info()->offset_first_element_in_bytes();
    bool padding_untouched = true;
    for (size_t i = 0; i < off0; ++i) padding_untouched = padding_untouched && out.buffer()[i] == 0xEE;
    for (int m = 0; m + 1 < M; ++m)
        for (size_t x = N; x < pitch; ++x) padding_untouched = padding_untouched && out.buffer()[off0 + m * pitch + x] == 0xEE;
    CHECK(padding_untouched);
}

// ---- rest of the function's type table: S32 accumulation, F32 dequantised output, 3-D reinterpretation, odd K -------
static void test_type_table()
{
    const int           M = 70, N = 130, K = 221; // K and the row pitch are no multiples of 16
    std::vector<int8_t> ha(size_t(M) * K), hb(size_t(K) * N);
    fill_uniform(ha, -128, 127, 41);
    fill_uniform(hb, -128, 127, 42);
    std::vector<int32_t> want(size_t(M) * N);
    orc_gemmlowp_core(ha.data(), 1, hb.data(), 1, want.data(), M, N, K, 1, 0, 3, -4);
    CUTensor a, b, acc, accf;
    a.allocator()->init(TensorInfo(TensorShape(K, M), 1, DataType::QASYMM8_SIGNED, QuantizationInfo(1.f / 255, 3)));
    b.allocator()->init(TensorInfo(TensorShape(N, K), 1, DataType::QASYMM8_SIGNED, QuantizationInfo(5.f / 255, -4)));
    acc.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::S32));
    accf.allocator()->init(TensorInfo(TensorShape(N, M), 1, DataType::F32));
    // GEMMInfo(..., accumulate = true): dst += A * B (CpuGemmLowpMatrixMultiplyCore.cpp:393-401)
    const GEMMInfo accumulate(false, false, false, 0, false, false, GEMMLowpOutputStageInfo(), false, false, false,
                              ActivationLayerInfo(), false, arm_compute::WeightFormat::UNSPECIFIED, false, true);
    CUGEMMLowpMatrixMultiplyCore plain, acc_fn, f32_fn, f32_acc_fn;
    plain.configure(&a, &b, nullptr, &acc);
    acc_fn.configure(&a, &b, nullptr, &acc, accumulate);
    f32_fn.configure(&a, &b, nullptr, &accf);
    f32_acc_fn.configure(&a, &b, nullptr, &accf, accumulate);
    for (CUTensor *t : {&a, &b, &acc, &accf}) t->allocator()->allocate();
    upload(a, ha);
    upload(b, hb);
    plain.run();
    CUScheduler::get().sync();
    CHECK(download<int32_t>(acc, want.size()) == want);
    acc_fn.run();
    acc_fn.run();
    CUScheduler::get().sync();
    std::vector<int32_t> want3(want);
    for (auto &v : want3) v *= 3;
    CHECK(download<int32_t>(acc, want.size()) == want3);
    // dequantised output (the s8 -> f32 rows of the type table): float(int32) * (scale_a * scale_b), as
    // dequantize_s32 of arm_compute/core/QuantizationInfo.h:639-642 computes it
    f32_fn.run();
    CUScheduler::get().sync();
    const float        scale = (1.f / 255) * (5.f / 255);
    std::vector<float> wantf(want.size());
    for (size_t i = 0; i < want.size(); ++i) wantf[i] = static_cast<float>(want[i]) * scale;
    CHECK(download<float>(accf, wantf.size()) == wantf);
    f32_acc_fn.run();
    CUScheduler::get().sync();
    for (size_t i = 0; i < want.size(); ++i) wantf[i] = wantf[i] + static_cast<float>(want[i]) * scale;
    CHECK(download<float>(accf, wantf.size()) == wantf);

    // reinterpret_input_as_3d + depth_output_gemm3d: A [K, 7, 10, 2] is a batch of two 70-row matrices
    CUTensor a3, o3;
    a3.allocator()->init(TensorInfo(TensorShape(K, 7, 10, 2), 1, DataType::QASYMM8_SIGNED, QuantizationInfo(1.f / 255, 3)));
    o3.allocator()->init(TensorInfo(TensorShape(N, 7, 10, 2), 1, DataType::S32));
    const GEMMInfo               as3d(false, false, false, 10, true);
    CUGEMMLowpMatrixMultiplyCore fn3d;
    fn3d.configure(&a3, &b, nullptr, &o3, as3d);
    a3.allocator()->allocate();
    o3.allocator()->allocate();
    std::vector<int8_t> ha2(ha);
    ha2.insert(ha2.end(), ha.rbegin(), ha.rend()); // second batch: other data
    upload(a3, ha2);
    fn3d.run();
    CUScheduler::get().sync();
    std::vector<int32_t> want2(2 * want.size());
    orc_gemmlowp_core(ha2.data(), 1, hb.data(), 1, want2.data(), M, N, K, 2, 0, 3, -4);
    CHECK(download<int32_t>(o3, want2.size()) == want2);
}

// ---- NCHW convolution and update_quantization_parameters --------------------------------------------------------------
static void test_convolution_nchw_and_requantisation()
{
    const int            B = 2, H = 11, W = 13, C = 16, OFM = 24, k = 3;
    std::vector<uint8_t> nhwc(size_t(B) * H * W * C), nchw(nhwc.size());
    std::vector<int8_t>  w_nhwc(size_t(OFM) * k * k * C), w_nchw(w_nhwc.size());
    std::vector<int32_t> hbias(OFM);
    std::vector<float>   scales(OFM);
    fill_uniform(nhwc, 0, 255, 51);
    fill_uniform(w_nhwc, -127, 127, 52);
    fill_uniform(hbias, -3000, 3000, 53);
    std::mt19937                          gen(54);
    std::uniform_real_distribution<float> sd(2e-3f, 8e-3f);
    for (auto &s : scales) s = sd(gen);
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x)
                for (int c = 0; c < C; ++c)
                    nchw[((size_t(b) * C + c) * H + y) * W + x] = nhwc[((size_t(b) * H + y) * W + x) * C + c];
    for (int o = 0; o < OFM; ++o)
        for (int y = 0; y < k; ++y)
            for (int x = 0; x < k; ++x)
                for (int c = 0; c < C; ++c)
                    w_nchw[((size_t(o) * C + c) * k + y) * k + x] = w_nhwc[((size_t(o) * k + y) * k + x) * C + c];
    const int Wo = (W + 2 - k) / 2 + 1, Ho = (H + 2 - k) / 2 + 1;
    CUTensor   src, wgt, bias, dst;
    TensorInfo si(TensorShape(W, H, C, B), 1, DataType::QASYMM8, QuantizationInfo(0.03f, 128));
    TensorInfo wi(TensorShape(k, k, C, OFM), 1, DataType::QSYMM8_PER_CHANNEL, QuantizationInfo(scales));
    TensorInfo di(TensorShape(Wo, Ho, OFM, B), 1, DataType::QASYMM8, QuantizationInfo(0.05f, 4));
    si.set_data_layout(DataLayout::NCHW);
    wi.set_data_layout(DataLayout::NCHW);
    di.set_data_layout(DataLayout::NCHW);
    src.allocator()->init(si);
    wgt.allocator()->init(wi);
    bias.allocator()->init(TensorInfo(TensorShape(OFM), 1, DataType::S32));
    dst.allocator()->init(di);
    CUGEMMConvolutionLayer conv;
    conv.configure(&src, &wgt, &bias, &dst, PadStrideInfo(2, 2, 1, 1));
    for (CUTensor *t : {&src, &wgt, &bias, &dst}) t->allocator()->allocate();
    upload(src, nchw);
    upload(wgt, w_nchw);
    upload(bias, hbias);
    conv.run();
    CUScheduler::get().sync();
    auto check = [&](float in_scale, int in_zp, float out_scale, int out_zp) {
        std::vector<int32_t> mult(OFM), shift(OFM);
        cugl_calculate_quantized_multipliers(in_scale, scales.data(), OFM, out_scale, mult.data(), shift.data());
        std::vector<uint8_t> want(size_t(B) * Ho * Wo * OFM), want_nchw(want.size());
        orc_conv2d_nhwc(nhwc.data(), 0, w_nhwc.data(), 1, hbias.data(), want.data(), C, W, H, B, k, k, OFM, 2, 2, 1, 1, 1,
                        1, Wo, Ho, in_zp, 0, mult.data(), shift.data(), OFM, out_zp, 0, 255);
        for (int b = 0; b < B; ++b)
            for (int p = 0; p < Ho * Wo; ++p)
                for (int o = 0; o < OFM; ++o) want_nchw[(size_t(b) * OFM + o) * Ho * Wo + p] = want[(size_t(b) * Ho * Wo + p) * OFM + o];
        CHECK(download<uint8_t>(dst, want_nchw.size()) == want_nchw);
    };
    check(0.03f, 128, 0.05f, 4);
    // NEGEMMConvolutionLayer::update_quantization_parameters: new input / output quantization, same prepared weights
    src.info()->set_quantization_info(QuantizationInfo(0.02f, 100));
    dst.info()->set_quantization_info(QuantizationInfo(0.04f, 9));
    conv.update_quantization_parameters();
    conv.run();
    CUScheduler::get().sync();
    check(0.02f, 100, 0.04f, 9);
}

// ---- memory manager: two convolutions on the explicit lowering share one pool ----------------------------------------
static size_t run_two_convolutions(std::shared_ptr<IMemoryManager> mm, std::vector<uint8_t> &result)
{
    // C = 3 keeps both layers on the explicit im2col lowering: each needs a [M][Kp] patch matrix per run
    const int  B = 4, H = 40, W = 40, C = 3, OFM = 3, k = 5;
    CUAllocator allocator;
    const size_t before = CUAllocator::bytes_in_use();
    CUAllocator::reset_peak();
    {
        CUTensor   x, w1, w2, mid, y;
        TensorInfo xi(TensorShape(C, W, H, B), 1, DataType::QASYMM8, QuantizationInfo(0.03f, 120));
        TensorInfo wi(TensorShape(C, k, k, OFM), 1, DataType::QASYMM8, QuantizationInfo(0.004f, 130));
        TensorInfo yi(TensorShape(OFM, W, H, B), 1, DataType::QASYMM8, QuantizationInfo(0.1f, 12));
        xi.set_data_layout(DataLayout::NHWC), wi.set_data_layout(DataLayout::NHWC), yi.set_data_layout(DataLayout::NHWC);
        x.allocator()->init(xi), w1.allocator()->init(wi), w2.allocator()->init(wi), mid.allocator()->init(yi), y.allocator()->init(yi);
        CUGEMMConvolutionLayer c1(mm), c2(mm);
        c1.configure(&x, &w1, nullptr, &mid, PadStrideInfo(1, 1, 2, 2));
        c2.configure(&mid, &w2, nullptr, &y, PadStrideInfo(1, 1, 2, 2));
        for (CUTensor *t : {&x, &w1, &w2, &mid, &y}) t->allocator()->allocate();
        if (mm)
        {
            mm->populate(allocator, 1); // one pool: the two workspaces never live at the same time
        }
        std::vector<uint8_t> hx(size_t(B) * H * W * C), hw(size_t(OFM) * k * k * C);
        fill_uniform(hx, 0, 255, 61);
        fill_uniform(hw, 100, 160, 62);
        upload(x, hx);
        upload(w1, hw);
        upload(w2, hw);
        c1.run();
        c2.run();
        CUScheduler::get().sync();
        result = download<uint8_t>(y, size_t(B) * H * W * OFM);
    }
    if (mm)
    {
        mm->clear();
    }
    return CUAllocator::peak_bytes() - before;
}

static void test_memory_manager()
{
    std::vector<uint8_t> plain, managed;
    const size_t         peak_plain   = run_two_convolutions(nullptr, plain);
    const size_t         peak_managed = run_two_convolutions(cu_create_memory_manager(), managed);
    CHECK(plain == managed);
    // without a manager each function holds its own patch matrix (4*40*40 rows x 80 bytes = 512 KB each)
    std::printf("peak device bytes of the tensors and workspaces: %zu without a memory manager, %zu with one\n", peak_plain,
                peak_managed);
    CHECK(peak_managed + 400 * 1024 < peak_plain);
}

int main(int argc, char **argv)
{
    const bool validate_only = argc > 1 && std::strcmp(argv[1], "--validate") == 0;
    try
    {
        test_validate();
        test_validate_layers();
        if (!validate_only)
        {
            CUScheduler::get().default_init(0);
            test_gemmlowp_config1();
            test_convolution();
            test_layers();
            test_fully_connected();
            test_host_tensors_with_padding();
            test_type_table();
            test_convolution_nchw_and_requantisation();
            test_memory_manager();
        }
    }
    catch (const std::exception &e)
    {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%s (%d failure%s)\n", g_failures == 0 ? "OK" : "FAILED", g_failures, g_failures == 1 ? "" : "s");
    return g_failures == 0 ? 0 : 1;
}
