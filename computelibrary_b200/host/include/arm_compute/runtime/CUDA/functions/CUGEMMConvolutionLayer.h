// CUDA counterpart of NEGEMMConvolutionLayer for 8-bit NHWC tensors
// (src/runtime/NEON/functions/NEGEMMConvolutionLayer.cpp:60-145; operator src/cpu/operators/CpuGemmConv2d.cpp).
// NHWC: input [C, W, H, B] QASYMM8 / QASYMM8_SIGNED, weights [C, kw, kh, OFM] same type or QSYMM8_PER_CHANNEL,
// biases S32 [OFM] or nullptr, output [OFM, Wo, Ho, B] of the input's type.  NCHW ([W, H, C, B], weights
// [kw, kh, C, OFM], output [Wo, Ho, OFM, B]) runs on NHWC copies made by a device transpose before and after the
// convolution (the weights once, in prepare()).  Quantisation infos carry TRUE zero points; RELU / BOUNDED_RELU /
// LU_BOUNDED_RELU are folded into the clamp of the output stage.
#pragma once
#include "arm_compute/core/ITensor.h"
#include "arm_compute/core/Types.h"
#include "arm_compute/function_info/ActivationLayerInfo.h"
#include "arm_compute/function_info/GEMMInfo.h"
#include "arm_compute/runtime/IFunction.h"
#include "arm_compute/runtime/IMemoryManager.h"
#include "arm_compute/runtime/IWeightsManager.h"

#include <memory>

struct cugl_conv_plan;

namespace arm_compute
{
class CUGEMMConvolutionLayer : public IFunction
{
public:
    CUGEMMConvolutionLayer(const std::shared_ptr<IMemoryManager> &memory_manager  = nullptr,
                           IWeightsManager                       *weights_manager = nullptr);
    CUGEMMConvolutionLayer(const CUGEMMConvolutionLayer &)            = delete;
    CUGEMMConvolutionLayer &operator=(const CUGEMMConvolutionLayer &) = delete;
    ~CUGEMMConvolutionLayer();
    void configure(const ITensor *input, const ITensor *weights, const ITensor *biases, ITensor *output,
                   const PadStrideInfo &conv_info, const WeightsInfo &weights_info = WeightsInfo(),
                   const Size2D &dilation = Size2D(1U, 1U), const ActivationLayerInfo &act_info = ActivationLayerInfo(),
                   bool enable_fast_math = false, unsigned int num_groups = 1);
    static Status validate(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                           const ITensorInfo *output, const PadStrideInfo &conv_info,
                           const WeightsInfo &weights_info = WeightsInfo(), const Size2D &dilation = Size2D(1U, 1U),
                           const ActivationLayerInfo &act_info = ActivationLayerInfo(), bool enable_fast_math = false,
                           unsigned int num_groups = 1);
    // As NEGEMMConvolutionLayer::update_quantization_parameters (NEGEMMConvolutionLayer.cpp:129-131,
    // CpuGemmConv2d.cpp:858-908): after the tensors' QuantizationInfo changed, re-derive the output stage and the
    // operand offsets.  The prepared weights stay valid.
    void update_quantization_parameters();
    void run() override;
    void prepare() override;

private:
    struct Impl;
    std::unique_ptr<Impl> _impl;
};
} // namespace arm_compute
