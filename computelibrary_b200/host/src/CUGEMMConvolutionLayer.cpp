#include "arm_compute/runtime/CUDA/functions/CUGEMMConvolutionLayer.h"

#include "arm_compute/core/Utils.h"
#include "arm_compute/core/utils/quantization/AsymmHelpers.h"

#include "CUHelpers.h"

#include <algorithm>
#include <tuple>
#include <vector>

namespace arm_compute
{
namespace
{
struct ConvSetup
{
    cugl_conv_desc          desc{};
    GEMMLowpOutputStageInfo stage{}; // owns the per-channel vectors the descriptor points into
    bool                    nchw{false};
};

// Index of the width / height / channel dimension for the tensor's layout (get_data_layout_dimension_index)
struct Dims
{
    size_t w, h, c;
};
Dims dims_of(DataLayout layout)
{
    return layout == DataLayout::NHWC ? Dims{1, 2, 0} : Dims{0, 1, 2};
}

Status make_conv(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                 const ITensorInfo *output, const PadStrideInfo &conv_info, const WeightsInfo &weights_info,
                 const Size2D &dilation, const ActivationLayerInfo &act_info, unsigned int num_groups, ConvSetup &out)
{
    ARM_COMPUTE_RETURN_ERROR_ON_NULLPTR(input, weights, output);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights_info.are_reshaped(), "Weights already reshaped are not supported!");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(num_groups != 1, "Grouping (num_groups != 1) is not supported");
    const DataLayout layout = input->data_layout();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(layout != DataLayout::NHWC && layout != DataLayout::NCHW, "layout must be NHWC or NCHW");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights->data_layout() != layout, "weights and input layouts differ");
    const Dims     ix = dims_of(layout);
    const DataType dt = input->data_type();
    ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(input, 1, DataType::QASYMM8, DataType::QASYMM8_SIGNED);
    const DataType wdt = weights->data_type();
    ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(weights, 1, DataType::QASYMM8, DataType::QASYMM8_SIGNED,
                                                         DataType::QSYMM8_PER_CHANNEL);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(weights->dimension(ix.c) != input->dimension(ix.c), "weights and input channel counts differ");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(conv_info.round() != DimensionRoundingType::FLOOR, "only FLOOR rounding is implemented");
    if (biases != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(biases, 1, DataType::S32);
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(biases->num_dimensions() > 1 || biases->dimension(0) != weights->dimension(3),
                                        "biases must be a vector of OFM elements");
    }
    out.nchw          = layout == DataLayout::NCHW;
    cugl_conv_desc &d = out.desc;
    d                 = cugl_conv_desc{};
    d.C               = static_cast<int32_t>(input->dimension(ix.c));
    d.W               = static_cast<int32_t>(input->dimension(ix.w));
    d.H               = static_cast<int32_t>(input->dimension(ix.h));
    d.B               = static_cast<int32_t>(input->tensor_shape().total_size_upper(3));
    d.kw              = static_cast<int32_t>(weights->dimension(ix.w));
    d.kh              = static_cast<int32_t>(weights->dimension(ix.h));
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
    const bool per_channel     = is_data_type_quantized_per_channel(wdt);
    d.src_zero_point           = iq.uniform().offset; // true zero points: negated inside the plan (CpuGemmConv2d.cpp:266-280)
    d.w_zero_point             = per_channel ? 0 : wq.uniform().offset;
    d.is_quantized_per_channel = per_channel ? 1 : 0;
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(per_channel && wq.scale().size() < static_cast<size_t>(d.OFM),
                                    "per-channel weights need OFM scales");
    // the library's own multiplier derivation (src/core/utils/quantization/AsymmHelpers.cpp:117-152)
    out.stage.type                     = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    out.stage.is_quantized_per_channel = per_channel;
    out.stage.gemmlowp_offset          = oq.uniform().offset;
    ARM_COMPUTE_RETURN_ON_ERROR(quantization::calculate_quantized_multipliers(iq, wq, oq, out.stage));
    d.gemmlowp_multiplier    = out.stage.gemmlowp_multiplier;
    d.gemmlowp_shift         = out.stage.gemmlowp_shift;
    d.h_gemmlowp_multipliers = out.stage.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts      = out.stage.gemmlowp_shifts.data();
    d.dst_zero_point         = oq.uniform().offset;
    int32_t lo = dt == DataType::QASYMM8 ? 0 : -128, hi = dt == DataType::QASYMM8 ? 255 : 127;
    if (act_info.enabled())
    {
        using F   = ActivationLayerInfo::ActivationFunction;
        const F f = act_info.activation();
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(f != F::RELU && f != F::BOUNDED_RELU && f != F::LU_BOUNDED_RELU,
                                        "only RELU, BOUNDED_RELU and LU_BOUNDED_RELU can be fused");
        std::tie(lo, hi) = get_quantized_activation_min_max(act_info, dt, oq.uniform()); // src/core/Utils.cpp:442-460
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
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_type() != dt, "output must have the input's data type");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_layout() != layout, "output and input layouts differ");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->dimension(ix.c) != static_cast<size_t>(d.OFM) ||
                                            output->dimension(ix.w) != static_cast<size_t>(wo) ||
                                            output->dimension(ix.h) != static_cast<size_t>(ho),
                                        "output shape does not match the convolution");
    }
    return Status{};
}
} // namespace

struct CUGEMMConvolutionLayer::Impl
{
    explicit Impl(std::shared_ptr<IMemoryManager> mm) : memory_group(std::move(mm)) {}
    MemoryGroup            memory_group;
    CUOperand              input{}, weights{}, biases{}, output{};
    PadStrideInfo          conv_info{};
    Size2D                 dilation{1U, 1U};
    ActivationLayerInfo    act_info{};
    cugl_conv_plan        *plan{nullptr};
    cu::TemporaryWorkspace workspace{};
    // NCHW: the plan works on NHWC copies of the input and of the output that live in the workspace, behind the
    // plan's own temporaries
    bool   nchw{false};
    size_t plan_temp{0}, in_bytes{0}, out_bytes{0};
    int    B{0}, C{0}, HW{0}, OFM{0}, HoWo{0}, khkw{0};
    bool   is_prepared{false};
};

CUGEMMConvolutionLayer::CUGEMMConvolutionLayer(const std::shared_ptr<IMemoryManager> &memory_manager,
                                               IWeightsManager                       *weights_manager)
    : _impl(std::make_unique<Impl>(memory_manager))
{
    ARM_COMPUTE_UNUSED(weights_manager); // the weights are re-laid out on the device inside the plan
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
    CU_THROW_ON(make_conv(input->info(), weights->info(), biases != nullptr ? biases->info() : nullptr, output->info(),
                          conv_info, weights_info, dilation, act_info, num_groups, s));
    if (_impl->plan != nullptr)
    {
        cugl_conv2d_plan_destroy(_impl->plan);
        _impl->plan = nullptr;
    }
    _impl->input.set(input);
    _impl->weights.set(weights);
    _impl->biases.set(biases);
    _impl->output.set(output);
    _impl->conv_info   = conv_info;
    _impl->dilation    = dilation;
    _impl->act_info    = act_info;
    _impl->is_prepared = false;
    cugl_context *ctx  = CUScheduler::get().context();
    CU_THROW_ON(cu_status(cugl_conv2d_plan_create(ctx, &s.desc, &_impl->plan), ctx, "CUGEMMConvolutionLayer::configure"));
    int32_t wo = 0, ho = 0;
    cugl_conv2d_out_dims(&s.desc, &wo, &ho);
    _impl->nchw      = s.nchw;
    _impl->B         = s.desc.B;
    _impl->C         = s.desc.C;
    _impl->HW        = s.desc.H * s.desc.W;
    _impl->OFM       = s.desc.OFM;
    _impl->HoWo      = wo * ho;
    _impl->khkw      = s.desc.kh * s.desc.kw;
    _impl->plan_temp = (cugl_conv2d_plan_temp_bytes(_impl->plan) + 255) / 256 * 256;
    _impl->in_bytes  = s.nchw ? (static_cast<size_t>(_impl->B) * _impl->C * _impl->HW + 255) / 256 * 256 : 0;
    _impl->out_bytes = s.nchw ? (static_cast<size_t>(_impl->B) * _impl->OFM * _impl->HoWo + 255) / 256 * 256 : 0;
    // Temporary-lifetime memory (im2col matrix, folded input, row sums, NHWC copies): one slot managed by the
    // memory group, the protocol of CpuGemmConv2d's Im2ColOutput / GemmOutput workspace slots
    _impl->workspace.configure(_impl->memory_group, _impl->plan_temp + _impl->in_bytes + _impl->out_bytes);
}

void CUGEMMConvolutionLayer::update_quantization_parameters()
{
    CU_ERROR_IF(_impl->plan == nullptr, "update_quantization_parameters before configure");
    ConvSetup s;
    CU_THROW_ON(make_conv(_impl->input.tensor()->info(), _impl->weights.tensor()->info(),
                          _impl->biases.tensor() != nullptr ? _impl->biases.tensor()->info() : nullptr,
                          _impl->output.tensor()->info(), _impl->conv_info, WeightsInfo(), _impl->dilation, _impl->act_info, 1, s));
    cugl_context *ctx = CUScheduler::get().context();
    CU_THROW_ON(cu_status(cugl_conv2d_update_quantization(_impl->plan, &s.desc), ctx,
                          "CUGEMMConvolutionLayer::update_quantization_parameters"));
}

void CUGEMMConvolutionLayer::prepare()
{
    if (_impl->is_prepared)
    {
        return;
    }
    CU_ERROR_IF(_impl->plan == nullptr, "prepare before configure");
    CU_ERROR_IF(!cu::is_dense(*_impl->weights.tensor()->info()), "CUGEMMConvolutionLayer: the weights tensor must be dense (no padding)");
    cugl_context *ctx = CUScheduler::get().context();
    const void   *w   = _impl->weights.device(true);
    void         *tmp = nullptr;
    if (_impl->nchw)
    {
        // [OFM][C][kh*kw] -> [OFM][kh*kw][C]: the K-major operand the plan expects
        const size_t bytes = static_cast<size_t>(_impl->OFM) * _impl->C * _impl->khkw;
        CU_THROW_ON(cu_status(cugl_malloc(ctx, bytes, &tmp), ctx, "CUGEMMConvolutionLayer::prepare"));
        CU_THROW_ON(cu_status(cugl_transpose_batched(ctx, w, tmp, _impl->C, _impl->khkw, _impl->OFM), ctx,
                              "CUGEMMConvolutionLayer::prepare"));
        w = tmp;
    }
    CU_THROW_ON(cu_status(cugl_conv2d_prepare(_impl->plan, w), ctx, "CUGEMMConvolutionLayer::prepare"));
    if (tmp != nullptr)
    {
        CU_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUGEMMConvolutionLayer::prepare"));
        cugl_free(ctx, tmp);
    }
    _impl->weights.tensor()->mark_as_unused();
    _impl->is_prepared = true;
}

void CUGEMMConvolutionLayer::run()
{
    prepare();
    // the plan reads and writes dense tensors; padded ones (extend_padding after configure) are refused loudly
    CU_ERROR_IF(!cu::is_dense(*_impl->input.tensor()->info()) || !cu::is_dense(*_impl->output.tensor()->info()) ||
                    (_impl->biases.tensor() != nullptr && !cu::is_dense(*_impl->biases.tensor()->info())),
                "CUGEMMConvolutionLayer: input, biases and output must be dense (no padding)");
    MemoryGroupResourceScope scope_mg(_impl->memory_group);
    cugl_context *ctx = CUScheduler::get().context();
    uint8_t      *ws  = static_cast<uint8_t *>(_impl->workspace.device_ptr());
    if (ws != nullptr && _impl->plan_temp != 0)
    {
        CU_THROW_ON(cu_status(cugl_conv2d_plan_bind_temp(_impl->plan, ws, _impl->plan_temp), ctx, "CUGEMMConvolutionLayer::run"));
    }
    const void *src = _impl->input.device(true);
    void       *dst = _impl->output.device(false);
    if (_impl->nchw)
    {
        CU_ERROR_IF(ws == nullptr, "CUGEMMConvolutionLayer: NCHW workspace missing");
        uint8_t *in_nhwc = ws + _impl->plan_temp, *out_nhwc = in_nhwc + _impl->in_bytes;
        CU_THROW_ON(cu_status(cugl_transpose_batched(ctx, src, in_nhwc, _impl->C, _impl->HW, _impl->B), ctx, "NCHW -> NHWC"));
        CU_THROW_ON(cu_status(cugl_conv2d_run(_impl->plan, in_nhwc, static_cast<const int32_t *>(_impl->biases.device(true)), out_nhwc),
                              ctx, "CUGEMMConvolutionLayer::run"));
        CU_THROW_ON(cu_status(cugl_transpose_batched(ctx, out_nhwc, dst, _impl->HoWo, _impl->OFM, _impl->B), ctx, "NHWC -> NCHW"));
    }
    else
    {
        CU_THROW_ON(cu_status(cugl_conv2d_run(_impl->plan, src, static_cast<const int32_t *>(_impl->biases.device(true)), dst), ctx,
                              "CUGEMMConvolutionLayer::run"));
    }
    _impl->output.download();
}
} // namespace arm_compute
