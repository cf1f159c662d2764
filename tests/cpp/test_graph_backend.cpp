// The graph frontend of Compute Library (arm_compute/graph/frontend/Stream.h, the API of examples/graph_resnet50.cpp)
// driving the CUDA backend: a reduced ResNet -- stem convolution + ReLU, max pooling, one bottleneck unit with a
// shortcut convolution and the residual addition + ReLU, global average pooling, 1x1 logits convolution, flatten,
// softmax -- on QASYMM8 tensors with seeded weights, compared with the CPU oracle layer by layer.
#include "arm_compute/graph.h"
#include "arm_compute/graph/backends/CUDA/CUDeviceBackend.h"
#include "arm_compute/runtime/CUDA/CUAllocator.h"
#include "arm_compute/runtime/CUDA/CUScheduler.h"

#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

using namespace arm_compute;
using namespace arm_compute::graph;
using namespace arm_compute::graph::frontend;

extern "C"
{
    void orc_conv2d_nhwc(const void *src, int src_signed, const void *weights, int w_signed, const int32_t *bias,
                         void *dst, int C, int W, int H, int B, int kw, int kh, int OFM, int sx, int sy, int pad_l,
                         int pad_t, int dil_x, int dil_y, int Wo, int Ho, int32_t in_zp, int32_t w_zp,
                         const int32_t *mult, const int32_t *shift, int n_mult, int32_t out_offset, int32_t lo,
                         int32_t hi);
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

namespace
{
int g_failures = 0;
#define CHECK(cond)                                                       \
    do                                                                    \
    {                                                                     \
        if (!(cond))                                                      \
        {                                                                 \
            std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); \
            ++g_failures;                                                 \
        }                                                                 \
    } while (false)

// feeds a dense tensor from a byte vector (weights, biases, the input image)
class VectorAccessor final : public ITensorAccessor
{
public:
    explicit VectorAccessor(const void *data, size_t bytes) : _data(static_cast<const uint8_t *>(data), static_cast<const uint8_t *>(data) + bytes) {}
    bool access_tensor(ITensor &tensor) override
    {
        if (tensor.info()->total_size() != _data.size())
        {
            std::printf("accessor size mismatch: tensor %zu bytes, data %zu bytes\n", tensor.info()->total_size(), _data.size());
            ++g_failures;
            return false;
        }
        std::memcpy(tensor.buffer(), _data.data(), _data.size());
        return true;
    }

private:
    std::vector<uint8_t> _data;
};

// copies a dense output tensor into a vector the test keeps
class CaptureAccessor final : public ITensorAccessor
{
public:
    explicit CaptureAccessor(std::vector<uint8_t> &out) : _out(out) {}
    bool access_tensor(ITensor &tensor) override
    {
        _out.assign(tensor.buffer(), tensor.buffer() + tensor.info()->total_size());
        return false; // one run
    }

private:
    std::vector<uint8_t> &_out;
};

template <typename T>
std::unique_ptr<ITensorAccessor> feed(const std::vector<T> &v)
{
    return std::make_unique<VectorAccessor>(v.data(), v.size() * sizeof(T));
}

struct Conv
{
    int                  C, OFM, k, stride, pad;
    std::vector<uint8_t> w; // [OFM][k][k][C]
    std::vector<int32_t> b;
    Conv(int C_, int OFM_, int k_, int stride_, int pad_, unsigned seed) : C(C_), OFM(OFM_), k(k_), stride(stride_), pad(pad_)
    {
        std::mt19937                       gen(seed);
        std::uniform_int_distribution<int> wd(90, 150), bd(-3000, 3000);
        w.resize(size_t(OFM) * k * k * C);
        b.resize(OFM);
        for (auto &x : w) x = static_cast<uint8_t>(wd(gen));
        for (auto &x : b) x = bd(gen);
    }
};

constexpr float kActScale = 0.05f, kWScale = 0.004f;
constexpr int   kWZp = 120;

ConvolutionLayer conv_layer(const Conv &c)
{
    // NHWC graph weights are [C, kw, kh, OFM]: exactly the [OFM][kh][kw][C] byte order the vectors hold
    return ConvolutionLayer(c.k, c.k, c.OFM, feed(c.w), feed(c.b), PadStrideInfo(c.stride, c.stride, c.pad, c.pad), 1,
                            QuantizationInfo(kWScale, kWZp), QuantizationInfo(kActScale, 0));
}

std::vector<uint8_t> conv_oracle(const Conv &c, const std::vector<uint8_t> &x, int B, int H, int W, bool relu, int &Ho, int &Wo)
{
    Ho = (H + 2 * c.pad - c.k) / c.stride + 1;
    Wo = (W + 2 * c.pad - c.k) / c.stride + 1;
    int32_t mult = 0, shift = 0;
    cugl_calculate_quantized_multiplier(kActScale * kWScale / kActScale, &mult, &shift);
    std::vector<uint8_t> y(size_t(B) * Ho * Wo * c.OFM);
    orc_conv2d_nhwc(x.data(), 0, c.w.data(), 0, c.b.data(), y.data(), c.C, W, H, B, c.k, c.k, c.OFM, c.stride, c.stride, c.pad, c.pad,
                    1, 1, Wo, Ho, 0, kWZp, &mult, &shift, 1, 0, 0, 255);
    (void)relu; // zero point 0: the ReLU clamp [0, 255] is the type range
    return y;
}
} // namespace

int main()
{
    try
    {
        const int            B = 2, H = 32, W = 32;
        std::vector<uint8_t> image(size_t(B) * H * W * 3);
        std::mt19937         gen(7);
        for (auto &p : image) p = static_cast<uint8_t>(gen() & 0xff);
        const Conv stem(3, 16, 7, 2, 3, 11), shortcut(16, 32, 1, 1, 0, 12), c1(16, 16, 1, 1, 0, 13), c2(16, 16, 3, 1, 1, 14),
            c3(16, 32, 1, 1, 0, 15), logits(32, 10, 1, 1, 0, 16);

        std::vector<uint8_t> got_sum, got_probs;
        {
            Stream           graph(0, "reduced_resnet");
            TensorDescriptor in_desc(TensorShape(3U, W, H, B), DataType::QASYMM8, QuantizationInfo(kActScale, 0), DataLayout::NHWC);
            graph << backends::CUDATarget << FastMathHint::Disabled << InputLayer(in_desc, feed(image)) << conv_layer(stem).set_name("conv1")
                  << ActivationLayer(ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU)).set_name("conv1/Relu")
                  << PoolingLayer(PoolingLayerInfo(PoolingType::MAX, 3, DataLayout::NHWC,
                                                   PadStrideInfo(2, 2, 0, 1, 0, 1, DimensionRoundingType::FLOOR)))
                         .set_name("pool1");
            SubStream left(graph), right(graph);
            left << conv_layer(shortcut).set_name("unit/shortcut");
            right << conv_layer(c1).set_name("unit/conv1")
                  << ActivationLayer(ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU))
                  << conv_layer(c2).set_name("unit/conv2")
                  << ActivationLayer(ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU))
                  << conv_layer(c3).set_name("unit/conv3");
            graph << EltwiseLayer(std::move(left), std::move(right), EltwiseOperation::Add).set_name("unit/add")
                  << ActivationLayer(ActivationLayerInfo(ActivationLayerInfo::ActivationFunction::RELU)).set_name("unit/Relu");
            SubStream tap(graph);
            tap << OutputLayer(std::make_unique<CaptureAccessor>(got_sum));
            graph << PoolingLayer(PoolingLayerInfo(PoolingType::AVG, DataLayout::NHWC)).set_name("pool5") << conv_layer(logits).set_name("logits")
                  << FlattenLayer().set_name("flatten") << SoftmaxLayer().set_name("softmax")
                  << OutputLayer(std::make_unique<CaptureAccessor>(got_probs));
            GraphConfig config;
            config.use_tuner = false;
            graph.finalize(backends::CUDATarget, config);
            graph.run();
            std::printf("device bytes held by the graph's tensors and workspaces at peak: %zu\n", CUAllocator::peak_bytes());
        }

        // ---- the same network on the oracle -------------------------------------------------------------------------
        int  h1, w1, hp, wp, hh, ww;
        auto x  = conv_oracle(stem, image, B, H, W, true, h1, w1);
        hp      = (h1 + 1 - 3) / 2 + 1;
        wp      = (w1 + 1 - 3) / 2 + 1;
        std::vector<uint8_t> p1(size_t(B) * hp * wp * 16);
        orc_pool_nhwc_u8(x.data(), p1.data(), 16, w1, h1, B, 0, 3, 3, 2, 2, 0, 1, 0, 1, 0, wp, hp, kActScale, 0, kActScale, 0);
        auto l  = conv_oracle(shortcut, p1, B, hp, wp, false, hh, ww);
        auto r  = conv_oracle(c1, p1, B, hp, wp, true, hh, ww);
        r       = conv_oracle(c2, r, B, hp, wp, true, hh, ww);
        r       = conv_oracle(c3, r, B, hp, wp, false, hh, ww);
        std::vector<uint8_t> sum(l.size()), sum_relu(l.size());
        orc_add_qasymm8(l.data(), r.data(), sum.data(), (long long)sum.size(), kActScale, 0, kActScale, 0, kActScale, 0);
        orc_activation_qasymm8(sum.data(), sum_relu.data(), (long long)sum.size(), 0, 0.f, 0.f, kActScale, 0, kActScale, 0);
        std::vector<uint8_t> avg(size_t(B) * 32);
        orc_pool_nhwc_u8(sum_relu.data(), avg.data(), 32, wp, hp, B, 1, wp, hp, 1, 1, 0, 0, 0, 0, 0, 1, 1, kActScale, 0, kActScale, 0);
        auto lg = conv_oracle(logits, avg, B, 1, 1, false, hh, ww);
        std::vector<uint8_t> probs(lg.size());
        orc_softmax_qasymm8(lg.data(), probs.data(), B, 10, 1.f, kActScale, 0);

        CHECK(got_sum == sum_relu);
        CHECK(got_probs.size() == probs.size());
        int worst = 0;
        for (size_t i = 0; i < probs.size() && i < got_probs.size(); ++i) worst = std::max(worst, std::abs(int(got_probs[i]) - int(probs[i])));
        CHECK(worst <= 1); // softmax: within one step, the tolerance of the reference's own quantized softmax tests
    }
    catch (const std::exception &e)
    {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%s (%d failure%s)\n", g_failures == 0 ? "OK" : "FAILED", g_failures, g_failures == 1 ? "" : "s");
    return g_failures == 0 ? 0 : 1;
}
