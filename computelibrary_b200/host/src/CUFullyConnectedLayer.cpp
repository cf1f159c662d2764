#include "arm_compute/runtime/CUDA/functions/CUFullyConnectedLayer.h"

#include "arm_compute/core/Utils.h"
#include "arm_compute/core/utils/quantization/AsymmHelpers.h"

#include "CUHelpers.h"

#include <tuple>
#include <vector>

namespace arm_compute
{
namespace
{
struct FcSetup
{
    cugl_conv_desc          desc{};
    GEMMLowpOutputStageInfo stage{}; // owns the per-channel vectors the descriptor points into
    size_t                  num_inputs{0}, num_outputs{0};
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
    // CpuFullyConnected.cpp:290-304: when a convolution output with more than one pixel feeds the layer and the
    // weights were trained in the other layout, the reference permutes the weights (CpuConvertFullyConnectedWeights)
    const size_t pixels = !is_conv_input ? 1
                          : (input->data_layout() == DataLayout::NHWC ? input->dimension(1) * input->dimension(2)
                                                                      : input->dimension(0) * input->dimension(1));
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(pixels > 1 && fc.weights_trained_layout != input->data_layout(),
                                    "weights trained in another layout than the 4-D input's: the weight permutation of "
                                    "CpuConvertFullyConnectedWeights is not implemented (set weights_trained_layout)");
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
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(per_channel && wq.scale().size() < out.num_outputs, "per-channel weights need num_outputs scales");
    out.stage.type                     = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    out.stage.is_quantized_per_channel = per_channel;
    out.stage.gemmlowp_offset          = oq.uniform().offset;
    ARM_COMPUTE_RETURN_ON_ERROR(quantization::calculate_quantized_multipliers(iq, wq, oq, out.stage)); // CpuFullyConnected.cpp:165-170
    d.gemmlowp_multiplier    = out.stage.gemmlowp_multiplier;
    d.gemmlowp_shift         = out.stage.gemmlowp_shift;
    d.h_gemmlowp_multipliers = out.stage.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts      = out.stage.gemmlowp_shifts.data();
    d.dst_zero_point         = oq.uniform().offset;
    int32_t lo = dt == DataType::QASYMM8 ? 0 : -128, hi = dt == DataType::QASYMM8 ? 255 : 127;
    if (fc.activation_info.enabled())
    {
        using F   = ActivationLayerInfo::ActivationFunction;
        const F f = fc.activation_info.activation();
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(f != F::RELU && f != F::BOUNDED_RELU && f != F::LU_BOUNDED_RELU,
                                        "only RELU, BOUNDED_RELU and LU_BOUNDED_RELU can be fused");
        std::tie(lo, hi) = get_quantized_activation_min_max(fc.activation_info, dt, oq.uniform());
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
    CUOperand               input{}, weights{}, biases{}, output{};
    cugl_conv_plan         *plan{nullptr};
    FullyConnectedLayerInfo fc{};
    size_t                  num_inputs{0}, num_outputs{0};
    bool                    is_prepared{false};
};

CUFullyConnectedLayer::CUFullyConnectedLayer(std::shared_ptr<IMemoryManager> memory_manager, IWeightsManager *weights_manager)
    : _impl(std::make_unique<Impl>())
{
    // a fully connected layer on the plain-GEMM lowering needs no temporary memory (symmetric or per-tensor
    // weights alike: the row sums of a [batch, num_inputs] input are a few KB owned by the plan)
    ARM_COMPUTE_UNUSED(memory_manager, weights_manager);
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
    CU_THROW_ON(make_fc(input->info(), weights->info(), biases != nullptr ? biases->info() : nullptr,
                                       output->info(), fc_info, weights_info, s));
    if (_impl->plan != nullptr)
    {
        cugl_conv2d_plan_destroy(_impl->plan);
        _impl->plan = nullptr;
    }
    _impl->input.set(input);
    _impl->weights.set(weights);
    _impl->biases.set(biases);
    _impl->output.set(output);
    _impl->fc          = fc_info;
    _impl->num_inputs  = s.num_inputs;
    _impl->num_outputs = s.num_outputs;
    _impl->is_prepared = false;
    cugl_context *ctx  = CUScheduler::get().context();
    CU_THROW_ON(cu_status(cugl_conv2d_plan_create(ctx, &s.desc, &_impl->plan), ctx, "CUFullyConnectedLayer::configure"));
}

void CUFullyConnectedLayer::prepare()
{
    if (_impl->is_prepared)
    {
        return;
    }
    CU_ERROR_IF(_impl->plan == nullptr, "prepare before configure");
    cugl_context *ctx = CUScheduler::get().context();
    CU_ERROR_IF(!cu::is_dense(*_impl->weights.tensor()->info()), "CUFullyConnectedLayer: the weights tensor must be dense (no padding)");
    const void   *w   = _impl->weights.device(true);
    void         *tmp = nullptr;
    if (!_impl->fc.transpose_weights)
    {
        // weights arrive as [num_inputs][num_outputs] (num_outputs contiguous): bring them to one row per output
        const size_t bytes = _impl->num_inputs * _impl->num_outputs;
        CU_THROW_ON(cu_status(cugl_malloc(ctx, bytes, &tmp), ctx, "CUFullyConnectedLayer::prepare"));
        CU_THROW_ON(cu_status(cugl_weights_reshape_nhwc(ctx, w, tmp, static_cast<int32_t>(_impl->num_outputs),
                                                                       static_cast<int32_t>(_impl->num_inputs)),
                                             ctx, "CUFullyConnectedLayer::prepare"));
        w = tmp;
    }
    CU_THROW_ON(cu_status(cugl_conv2d_prepare(_impl->plan, w), ctx, "CUFullyConnectedLayer::prepare"));
    if (tmp != nullptr)
    {
        CU_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUFullyConnectedLayer::prepare"));
        cugl_free(ctx, tmp);
    }
    _impl->weights.tensor()->mark_as_unused();
    _impl->is_prepared = true;
}

void CUFullyConnectedLayer::run()
{
    prepare();
    cugl_context *ctx = CUScheduler::get().context();
    CU_ERROR_IF(!cu::is_dense(*_impl->input.tensor()->info()) || !cu::is_dense(*_impl->output.tensor()->info()) ||
                    (_impl->biases.tensor() != nullptr && !cu::is_dense(*_impl->biases.tensor()->info())),
                "CUFullyConnectedLayer: input, biases and output must be dense (no padding)");
    void *dst = _impl->output.device(false);
    CU_THROW_ON(cu_status(cugl_conv2d_run(_impl->plan, _impl->input.device(true),
                                          static_cast<const int32_t *>(_impl->biases.device(true)), dst),
                          ctx, "CUFullyConnectedLayer::run"));
    _impl->output.download();
}
} // namespace arm_compute
