#include "arm_compute/runtime/CUDA/functions/CUFullyConnectedLayer.h"

#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"
#include "arm_compute/runtime/CUDA/functions/CUGEMMConvolutionLayer.h"

#include <tuple>
#include <vector>

namespace arm_compute
{
namespace
{
struct FcSetup
{
    cugl_conv_desc       desc{};
    std::vector<int32_t> mults, shifts;
    size_t               num_inputs{0}, num_outputs{0};
};

Status make_fc(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases, const ITensorInfo *output,
               const FullyConnectedLayerInfo &fc, const WeightsInfo &weights_info, FcSetup &out)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr || weights == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights_info.are_reshaped() || fc.are_weights_reshaped,
                                    "Weights already reshaped are not supported!");
    const DataType dt = input->data_type();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(dt != DataType::QASYMM8 && dt != DataType::QASYMM8_SIGNED, "input must be 8-bit quantized");
    const DataType wdt = weights->data_type();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!is_data_type_quantized(wdt), "weights must be 8-bit quantized");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_type() != dt, "output must have the input's data type");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights->num_dimensions() > 2, "weights must be a matrix");
    out.num_inputs  = fc.transpose_weights ? weights->dimension(0) : weights->dimension(1);
    out.num_outputs = fc.transpose_weights ? weights->dimension(1) : weights->dimension(0);
    // CpuFullyConnected.cpp: a 4-D input is a convolution output whose first three dimensions are flattened
    const bool   is_conv_input = input->num_dimensions() > 2;
    const size_t flat          = is_conv_input ? input->dimension(0) * input->dimension(1) * input->dimension(2) : input->dimension(0);
    const size_t batch         = is_conv_input ? input->tensor_shape().total_size_upper(3) : input->tensor_shape().total_size_upper(1);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(flat != out.num_inputs, "input features and weights rows differ");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->dimension(0) != out.num_outputs || output->tensor_shape().total_size_upper(1) != batch,
                                    "output must be [num_outputs, batch]");
    if (biases != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(biases->data_type() != DataType::S32, "biases must be S32 for a quantized layer");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(biases->num_dimensions() > 1 || biases->dimension(0) != out.num_outputs,
                                        "biases must be a vector of num_outputs elements");
    }
    cugl_conv_desc &d = out.desc;
    d                 = cugl_conv_desc{};
    d.C               = static_cast<int32_t>(out.num_inputs);
    d.W = d.H = 1;
    d.B       = static_cast<int32_t>(batch);
    d.kw = d.kh = 1;
    d.OFM       = static_cast<int32_t>(out.num_outputs);
    d.stride_x = d.stride_y = d.dil_x = d.dil_y = 1;
    d.src_dtype = dt == DataType::QASYMM8 ? CUGL_U8 : CUGL_S8;
    d.w_dtype   = wdt == DataType::QASYMM8 ? CUGL_U8 : CUGL_S8;
    const QuantizationInfo iq = input->quantization_info(), wq = weights->quantization_info(), oq = output->quantization_info();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(iq.scale().empty() || wq.scale().empty() || oq.scale().empty(), "missing quantization scale");
    const bool per_channel     = is_data_type_quantized_per_channel(wdt);
    d.src_zero_point           = iq.uniform().offset; // true zero points; the plan negates them (CpuFullyConnected.cpp:97-102)
    d.w_zero_point             = per_channel ? 0 : wq.uniform().offset;
    d.is_quantized_per_channel = per_channel ? 1 : 0;
    const size_t n_scales      = per_channel ? out.num_outputs : 1;
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(wq.scale().size() < n_scales, "per-channel weights need num_outputs scales");
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
    if (fc.activation_info.enabled())
    {
        using F   = ActivationLayerInfo::ActivationFunction;
        const F f = fc.activation_info.activation();
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(f != F::RELU && f != F::BOUNDED_RELU && f != F::LU_BOUNDED_RELU,
                                        "only RELU, BOUNDED_RELU and LU_BOUNDED_RELU can be fused");
        std::tie(lo, hi) = cu_quantized_activation_min_max(fc.activation_info, dt, oq.uniform());
    }
    d.min_bound = lo;
    d.max_bound = hi;
    d.has_bias  = biases != nullptr ? 1 : 0;
    const char *why = nullptr;
    if (cugl_conv2d_validate(&d, &why) != CUGL_SUCCESS)
    {
        return Status(ErrorCode::RUNTIME_ERROR, why != nullptr ? why : "invalid fully connected layer");
    }
    return Status{};
}
} // namespace

struct CUFullyConnectedLayer::Impl
{
    const ITensor          *input{nullptr};
    const ITensor          *weights{nullptr};
    const ITensor          *biases{nullptr};
    ITensor                *output{nullptr};
    cugl_conv_plan         *plan{nullptr};
    FullyConnectedLayerInfo fc{};
    size_t                  num_inputs{0}, num_outputs{0};
    bool                    is_prepared{false};
};

CUFullyConnectedLayer::CUFullyConnectedLayer() : _impl(std::make_unique<Impl>())
{
}

CUFullyConnectedLayer::~CUFullyConnectedLayer()
{
    if (_impl && _impl->plan != nullptr)
    {
        cugl_conv2d_plan_destroy(_impl->plan);
    }
}

Status CUFullyConnectedLayer::validate(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                                       const ITensorInfo *output, FullyConnectedLayerInfo fc_info,
                                       const WeightsInfo &weights_info)
{
    FcSetup s;
    return make_fc(input, weights, biases, output, fc_info, weights_info, s);
}

void CUFullyConnectedLayer::configure(const ITensor *input, const ITensor *weights, const ITensor *biases, ITensor *output,
                                      FullyConnectedLayerInfo fc_info, const WeightsInfo &weights_info)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input, weights, output);
    FcSetup s;
    ARM_COMPUTE_ERROR_THROW_ON(make_fc(input->info(), weights->info(), biases != nullptr ? biases->info() : nullptr,
                                       output->info(), fc_info, weights_info, s));
    if (_impl->plan != nullptr)
    {
        cugl_conv2d_plan_destroy(_impl->plan);
        _impl->plan = nullptr;
    }
    _impl->input       = input;
    _impl->weights     = weights;
    _impl->biases      = biases;
    _impl->output      = output;
    _impl->fc          = fc_info;
    _impl->num_inputs  = s.num_inputs;
    _impl->num_outputs = s.num_outputs;
    _impl->is_prepared = false;
    cugl_context *ctx  = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_conv2d_plan_create(ctx, &s.desc, &_impl->plan), ctx, "CUFullyConnectedLayer::configure"));
}

void CUFullyConnectedLayer::prepare()
{
    if (_impl->is_prepared)
    {
        return;
    }
    ARM_COMPUTE_ERROR_ON_MSG(_impl->plan == nullptr, "prepare before configure");
    cugl_context *ctx = CUScheduler::get().context();
    const void   *w   = cu_device_ptr(_impl->weights);
    void         *tmp = nullptr;
    if (!_impl->fc.transpose_weights)
    {
        // weights arrive as [num_inputs][num_outputs] (num_outputs contiguous): bring them to one row per output
        const size_t bytes = _impl->num_inputs * _impl->num_outputs;
        ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_malloc(ctx, bytes, &tmp), ctx, "CUFullyConnectedLayer::prepare"));
        ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_weights_reshape_nhwc(ctx, w, tmp, static_cast<int32_t>(_impl->num_outputs),
                                                                       static_cast<int32_t>(_impl->num_inputs)),
                                             ctx, "CUFullyConnectedLayer::prepare"));
        w = tmp;
    }
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_conv2d_prepare(_impl->plan, w), ctx, "CUFullyConnectedLayer::prepare"));
    if (tmp != nullptr)
    {
        ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUFullyConnectedLayer::prepare"));
        cugl_free(ctx, tmp);
    }
    _impl->weights->mark_as_unused();
    _impl->is_prepared = true;
}

void CUFullyConnectedLayer::run()
{
    prepare();
    cugl_context *ctx = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_conv2d_run(_impl->plan, cu_device_ptr(_impl->input),
                                                         static_cast<const int32_t *>(cu_device_ptr(_impl->biases)),
                                                         cu_device_ptr(_impl->output)),
                                         ctx, "CUFullyConnectedLayer::run"));
}
} // namespace arm_compute
