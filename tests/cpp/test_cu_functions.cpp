// Self-test of the C++ function family, written the way the reference's own examples / fixtures drive the NE
// functions (examples/neon_gemm_qasymm8.cpp:200-246, tests/validation/fixtures/GEMMLowpFixture.h:239-346):
// configure -> allocate -> fill (std::mt19937) -> run -> compare with the CPU oracle (oracle/gemmlowp_oracle.c).
//   test_cu_functions --validate   host-only checks of validate() (no GPU needed)
//   test_cu_functions              everything, on cuda:0
#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"
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
    GEMMInfo reshaped;
    reshaped.set_is_a_reshaped(true);
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
    const auto mm = cu_quantized_activation_min_max(
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
