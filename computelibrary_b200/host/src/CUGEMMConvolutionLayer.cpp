#include "arm_compute/runtime/CUDA/functions/CUGEMMConvolutionLayer.h"

#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"

#include <algorithm>
#include <vector>

namespace arm_compute
{
std::pair<int32_t, int32_t> cu_quantized_activation_min_max(const ActivationLayerInfo &act, DataType dt,
                                                            UniformQuantizationInfo oq)
{
    const bool    is_signed = dt == DataType::QASYMM8_SIGNED;
    const int     a_int     = is_signed ? quantize_qasymm8_signed(act.a(), oq) : quantize_qasymm8(act.a(), oq);
    const int     b_int     = is_signed ? quantize_qasymm8_signed(act.b(), oq) : quantize_qasymm8(act.b(), oq);
    const int32_t type_max  = is_signed ? 127 : 255;
    const int32_t lo = act.activation() != ActivationLayerInfo::ActivationFunction::LU_BOUNDED_RELU
                           ? std::min(oq.offset, type_max)
                           : b_int;
    const int32_t hi = act.activation() == ActivationLayerInfo::ActivationFunction::RELU ? type_max : a_int;
    return {lo, hi};
}

namespace
{
struct ConvSetup
{
    cugl_conv_desc       desc{};
    std::vector<int32_t> mults, shifts;
};

Status make_conv(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                 const ITensorInfo *output, const PadStrideInfo &conv_info, const WeightsInfo &weights_info,
                 const Size2D &dilation, const ActivationLayerInfo &act_info, unsigned int num_groups, ConvSetup &out)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr || weights == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights_info.are_reshaped(), "Weights already reshaped are not supported!");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(num_groups != 1, "Grouping (num_groups != 1) is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input->data_layout() != DataLayout::NHWC, "the CUDA backend implements the NHWC layout");
    const DataType dt = input->data_type();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(dt != DataType::QASYMM8 && dt != DataType::QASYMM8_SIGNED, "input must be 8-bit quantized");
    const DataType wdt = weights->data_type();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!is_data_type_quantized(wdt), "weights must be 8-bit quantized");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_type() != dt, "output must have the input's data type");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights->dimension(0) != input->dimension(0), "weights and input channel counts differ");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(conv_info.round() != DimensionRoundingType::FLOOR, "only FLOOR rounding is implemented");
    if (biases != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(biases->data_type() != DataType::S32, "biases must be S32 for quantized convolution");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(biases->num_dimensions() > 1 || biases->dimension(0) != weights->dimension(3),
                                        "biases must be a vector of OFM elements");
    }
    cugl_conv_desc &d = out.desc;
    d                 = cugl_conv_desc{};
    d.C               = static_cast<int32_t>(input->dimension(0));
    d.W               = static_cast<int32_t>(input->dimension(1));
    d.H               = static_cast<int32_t>(input->dimension(2));
    d.B               = static_cast<int32_t>(input->tensor_shape().total_size_upper(3));
    d.kw              = static_cast<int32_t>(weights->dimension(1));
    d.kh              = static_cast<int32_t>(weights->dimension(2));
    d.OFM             = static_cast<int32_t>(weights->dimension(3));
    d.stride_x        = static_cast<int32_t>(conv_info.stride().first);
    d.stride_y        = static_cast<int32_t>(conv_info.stride().second);
    d.pad_left        = static_cast<int32_t>(conv_info.pad_left());
    d.pad_right       = static_cast<int32_t>(conv_info.pad_right());
    d.pad_top         = static_cast<int32_t>(conv_info.pad_top());
    d.pad_bottom      = static_cast<int32_t>(conv_info.pad_bottom());
    d.dil_x           = static_cast<int32_t>(dilation.x());
    d.dil_y           = static_cast<int32_t>(dilation.y());
    d.src_dtype       = dt == DataType::QASYMM8 ? CUGL_U8 : CUGL_S8;
    d.w_dtype         = wdt == DataType::QASYMM8 ? CUGL_U8 : CUGL_S8;
    const QuantizationInfo iq = input->quantization_info(), wq = weights->quantization_info();
    const QuantizationInfo oq = output->total_size() == 0 ? iq : output->quantization_info();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(iq.scale().empty() || wq.scale().empty() || oq.scale().empty(), "missing quantization scale");
    const bool per_channel = is_data_type_quantized_per_channel(wdt);
    d.src_zero_point       = iq.uniform().offset; // true zero points: negated inside the plan (CpuGemmConv2d.cpp:266-280)
    d.w_zero_point         = per_channel ? 0 : wq.uniform().offset;
    d.is_quantized_per_channel = per_channel ? 1 : 0;
    const size_t n_scales      = per_channel ? static_cast<size_t>(d.OFM) : 1;
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(wq.scale().size() < n_scales, "per-channel weights need OFM scales");
    out.mults.resize(n_scales);
    out.shifts.resize(n_scales);
    if (cugl_calculate_quantized_multipliers(iq.scale()[0], wq.scale().data(), static_cast<int>(n_scales), oq.scale()[0],
                                             out.mults.data(), out.shifts.data()) != CUGL_SUCCESS)
    {
        return Status(ErrorCode::RUNTIME_ERROR, cugl_last_error_string(nullptr));
    }
    d.gemmlowp_multiplier    = out.mults[0];
    d.gemmlowp_shift         = out.shifts[0];
    d.h_gemmlowp_multipliers = out.mults.data();
    d.h_gemmlowp_shifts      = out.shifts.data();
    d.dst_zero_point         = oq.uniform().offset;
    int32_t lo = dt == DataType::QASYMM8 ? 0 : -128, hi = dt == DataType::QASYMM8 ? 255 : 127;
    if (act_info.enabled())
    {
        using F = ActivationLayerInfo::ActivationFunction;
        const F f = act_info.activation();
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(f != F::RELU && f != F::BOUNDED_RELU && f != F::LU_BOUNDED_RELU,
                                        "only RELU, BOUNDED_RELU and LU_BOUNDED_RELU can be fused");
        std::tie(lo, hi) = cu_quantized_activation_min_max(act_info, dt, oq.uniform());
    }
    d.min_bound = lo;
    d.max_bound = hi;
    d.has_bias  = biases != nullptr ? 1 : 0;
    const char *why = nullptr;
    if (cugl_conv2d_validate(&d, &why) != CUGL_SUCCESS)
    {
        return Status(ErrorCode::RUNTIME_ERROR, why != nullptr ? why : "invalid convolution");
    }
    int32_t wo = 0, ho = 0;
    cugl_conv2d_out_dims(&d, &wo, &ho);
    if (output->total_size() != 0)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->dimension(0) != static_cast<size_t>(d.OFM) ||
                                            output->dimension(1) != static_cast<size_t>(wo) ||
                                            output->dimension(2) != static_cast<size_t>(ho),
                                        "output shape must be [OFM, Wo, Ho, B]");
    }
    return Status{};
}
} // namespace

struct CUGEMMConvolutionLayer::Impl
{
    const ITensor  *input{nullptr};
    const ITensor  *weights{nullptr};
    const ITensor  *biases{nullptr};
    ITensor        *output{nullptr};
    cugl_conv_plan *plan{nullptr};
    bool            is_prepared{false};
};

CUGEMMConvolutionLayer::CUGEMMConvolutionLayer(const std::shared_ptr<IMemoryManager> &memory_manager,
                                               IWeightsManager                       *weights_manager)
    : _impl(std::make_unique<Impl>())
{
    ARM_COMPUTE_UNUSED(memory_manager, weights_manager);
}

CUGEMMConvolutionLayer::~CUGEMMConvolutionLayer()
{
    if (_impl && _impl->plan != nullptr)
    {
        cugl_conv2d_plan_destroy(_impl->plan);
    }
}

Status CUGEMMConvolutionLayer::validate(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                                        const ITensorInfo *output, const PadStrideInfo &conv_info,
                                        const WeightsInfo &weights_info, const Size2D &dilation,
                                        const ActivationLayerInfo &act_info, bool enable_fast_math, unsigned int num_groups)
{
    ARM_COMPUTE_UNUSED(enable_fast_math);
    ConvSetup s;
    return make_conv(input, weights, biases, output, conv_info, weights_info, dilation, act_info, num_groups, s);
}

void CUGEMMConvolutionLayer::configure(const ITensor *input, const ITensor *weights, const ITensor *biases, ITensor *output,
                                       const PadStrideInfo &conv_info, const WeightsInfo &weights_info, const Size2D &dilation,
                                       const ActivationLayerInfo &act_info, bool enable_fast_math, unsigned int num_groups)
{
    ARM_COMPUTE_UNUSED(enable_fast_math);
    ARM_COMPUTE_ERROR_ON_NULLPTR(input, weights, output);
    ConvSetup s;
    ARM_COMPUTE_ERROR_THROW_ON(make_conv(input->info(), weights->info(), biases != nullptr ? biases->info() : nullptr,
                                         output->info(), conv_info, weights_info, dilation, act_info, num_groups, s));
    if (_impl->plan != nullptr)
    {
        cugl_conv2d_plan_destroy(_impl->plan);
        _impl->plan = nullptr;
    }
    _impl->input       = input;
    _impl->weights     = weights;
    _impl->biases      = biases;
    _impl->output      = output;
    _impl->is_prepared = false;
    cugl_context *ctx  = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_conv2d_plan_create(ctx, &s.desc, &_impl->plan), ctx, "CUGEMMConvolutionLayer::configure"));
}

void CUGEMMConvolutionLayer::prepare()
{
    if (_impl->is_prepared)
    {
        return;
    }
    ARM_COMPUTE_ERROR_ON_MSG(_impl->plan == nullptr, "prepare before configure");
    cugl_context *ctx = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_conv2d_prepare(_impl->plan, cu_device_ptr(_impl->weights)), ctx, "CUGEMMConvolutionLayer::prepare"));
    _impl->weights->mark_as_unused();
    _impl->is_prepared = true;
}

void CUGEMMConvolutionLayer::run()
{
    prepare();
    cugl_context *ctx = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_conv2d_run(_impl->plan, cu_device_ptr(_impl->input),
                                                         static_cast<const int32_t *>(cu_device_ptr(_impl->biases)),
                                                         cu_device_ptr(_impl->output)),
                                         ctx, "CUGEMMConvolutionLayer::run"));
}
} // namespace arm_compute
