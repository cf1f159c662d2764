#include "arm_compute/runtime/CUDA/functions/CUQuantizedLayers.h"

#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"

namespace arm_compute
{
namespace
{
bool is_u8_nhwc(const ITensorInfo *t)
{
    return t != nullptr && t->data_type() == DataType::QASYMM8 && t->data_layout() == DataLayout::NHWC;
}
int32_t to_cugl_activation(const ActivationLayerInfo &act)
{
    if (!act.enabled()) return CUGL_ACT_NONE;
    switch (act.activation())
    {
        case ActivationLayerInfo::ActivationFunction::RELU:
            return CUGL_ACT_RELU;
        case ActivationLayerInfo::ActivationFunction::BOUNDED_RELU:
            return CUGL_ACT_BOUNDED_RELU;
        case ActivationLayerInfo::ActivationFunction::LU_BOUNDED_RELU:
            return CUGL_ACT_LU_BOUNDED_RELU;
        default:
            return CUGL_ACT_NONE;
    }
}
bool dense(const ITensorInfo *t)
{
    // the byte kernels address tensors as contiguous NHWC arrays
    return t->strides_in_bytes()[1] == t->dimension(0) * t->element_size() &&
           t->total_size() == t->tensor_shape().total_size() * t->element_size();
}
// NHWC TensorShape(C, W, H, B)
cugl_pool_desc make_pool_desc(const ITensorInfo *in, const ITensorInfo *out, const PoolingLayerInfo &pi)
{
    cugl_pool_desc d{};
    d.C               = static_cast<int32_t>(in->dimension(0));
    d.W               = static_cast<int32_t>(in->dimension(1));
    d.H               = static_cast<int32_t>(in->dimension(2));
    d.B               = static_cast<int32_t>(in->tensor_shape().total_size_upper(3));
    d.pool_type       = pi.pool_type == PoolingType::MAX ? CUGL_POOL_MAX : CUGL_POOL_AVG;
    d.pool_w          = static_cast<int32_t>(pi.pool_size.width);
    d.pool_h          = static_cast<int32_t>(pi.pool_size.height);
    d.stride_x        = static_cast<int32_t>(pi.pad_stride_info.stride().first);
    d.stride_y        = static_cast<int32_t>(pi.pad_stride_info.stride().second);
    d.pad_left        = static_cast<int32_t>(pi.pad_stride_info.pad_left());
    d.pad_right       = static_cast<int32_t>(pi.pad_stride_info.pad_right());
    d.pad_top         = static_cast<int32_t>(pi.pad_stride_info.pad_top());
    d.pad_bottom      = static_cast<int32_t>(pi.pad_stride_info.pad_bottom());
    d.exclude_padding = pi.exclude_padding ? 1 : 0;
    d.is_global       = pi.is_global_pooling ? 1 : 0;
    const UniformQuantizationInfo qi = in->quantization_info().uniform();
    const UniformQuantizationInfo qo = out->quantization_info().uniform();
    d.src_scale = qi.scale, d.src_zero_point = qi.offset;
    d.dst_scale = qo.scale, d.dst_zero_point = qo.offset;
    return d;
}
} // namespace

// ---- pooling (src/cpu/kernels/CpuPool2dKernel.cpp: validate_arguments) ------------------------------------
Status CUPoolingLayer::validate(const ITensorInfo *input, const ITensorInfo *output, const PoolingLayerInfo &pool_info,
                                const ITensorInfo *indices)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(indices != nullptr, "pooling indices are not supported for quantized types");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!is_u8_nhwc(input) || !is_u8_nhwc(output), "QASYMM8 NHWC tensors only");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(pool_info.pool_type == PoolingType::L2, "L2 pooling is not supported for quantized types");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(pool_info.pad_stride_info.round() != DimensionRoundingType::FLOOR,
                                    "only FLOOR rounding of the output size is implemented");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!dense(input) || !dense(output), "padded tensors are not supported");
    const cugl_pool_desc d = make_pool_desc(input, output, pool_info);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(cugl_pool2d_validate(&d) != CUGL_SUCCESS, "invalid pooling window, stride or padding");
    int32_t wo = 1, ho = 1;
    cugl_pool2d_out_dims(&d, &wo, &ho);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->dimension(0) != input->dimension(0) ||
                                        output->dimension(1) != static_cast<size_t>(wo) ||
                                        output->dimension(2) != static_cast<size_t>(ho) ||
                                        output->tensor_shape().total_size_upper(3) != input->tensor_shape().total_size_upper(3),
                                    "output shape does not match the pooled input shape");
    return Status{};
}

void CUPoolingLayer::configure(ITensor *input, ITensor *output, const PoolingLayerInfo &pool_info, ITensor *indices)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input, output);
    CU_THROW_ON(validate(input->info(), output->info(), pool_info, indices != nullptr ? indices->info() : nullptr));
    _input  = input;
    _output = output;
    _info   = pool_info;
}

void CUPoolingLayer::run()
{
    cugl_context        *ctx = CUScheduler::get().context();
    const cugl_pool_desc d   = make_pool_desc(_input->info(), _output->info(), _info);
    CU_THROW_ON(
        cu_status(cugl_pool2d_nhwc(ctx, &d, cu_device_ptr(_input), cu_device_ptr(_output)), ctx, "CUPoolingLayer::run"));
}

// ---- addition (src/cpu/kernels/CpuAddKernel.cpp: validate_arguments) ---------------------------------------
Status CUArithmeticAddition::validate(const ITensorInfo *input1, const ITensorInfo *input2, const ITensorInfo *output,
                                      ConvertPolicy policy, const ActivationLayerInfo &act_info)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input1 == nullptr || input2 == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input1->data_type() != DataType::QASYMM8 || input2->data_type() != DataType::QASYMM8 ||
                                        output->data_type() != DataType::QASYMM8,
                                    "QASYMM8 tensors only");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(policy != ConvertPolicy::SATURATE, "quantized addition saturates (ConvertPolicy::SATURATE)");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input1->tensor_shape() != input2->tensor_shape() ||
                                        input1->tensor_shape() != output->tensor_shape(),
                                    "broadcasting is not implemented: shapes must be equal");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!dense(input1) || !dense(input2) || !dense(output), "padded tensors are not supported");
    if (act_info.enabled())
    {
        const auto f = act_info.activation();
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(f != ActivationLayerInfo::ActivationFunction::RELU &&
                                            f != ActivationLayerInfo::ActivationFunction::BOUNDED_RELU &&
                                            f != ActivationLayerInfo::ActivationFunction::LU_BOUNDED_RELU,
                                        "only the ReLU family can be fused");
    }
    return Status{};
}

void CUArithmeticAddition::configure(const ITensor *input1, const ITensor *input2, ITensor *output, ConvertPolicy policy,
                                     const ActivationLayerInfo &act_info)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input1, input2, output);
    CU_THROW_ON(validate(input1->info(), input2->info(), output->info(), policy, act_info));
    _input1 = input1;
    _input2 = input2;
    _output = output;
    _act    = act_info;
}

void CUArithmeticAddition::run()
{
    cugl_context                 *ctx = CUScheduler::get().context();
    const UniformQuantizationInfo q1  = _input1->info()->quantization_info().uniform();
    const UniformQuantizationInfo q2  = _input2->info()->quantization_info().uniform();
    const UniformQuantizationInfo qo  = _output->info()->quantization_info().uniform();
    CU_THROW_ON(cu_status(
        cugl_add_qasymm8(ctx, cu_device_ptr(_input1), cu_device_ptr(_input2), cu_device_ptr(_output),
                         static_cast<int64_t>(_output->info()->tensor_shape().total_size()), q1.scale, q1.offset, q2.scale,
                         q2.offset, qo.scale, qo.offset, to_cugl_activation(_act), _act.a(), _act.b()),
        ctx, "CUArithmeticAddition::run"));
}

// ---- activation (src/cpu/kernels/CpuActivationKernel.cpp: validate_arguments) ------------------------------
Status CUActivationLayer::validate(const ITensorInfo *input, const ITensorInfo *output, const ActivationLayerInfo &act_info)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input->data_type() != DataType::QASYMM8, "QASYMM8 tensors only");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!act_info.enabled() || to_cugl_activation(act_info) == CUGL_ACT_NONE,
                                    "only RELU, BOUNDED_RELU and LU_BOUNDED_RELU are implemented for QASYMM8");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!dense(input), "padded tensors are not supported");
    if (output != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_type() != DataType::QASYMM8, "QASYMM8 tensors only");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->tensor_shape() != input->tensor_shape(), "input and output shapes differ");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(!dense(output), "padded tensors are not supported");
    }
    return Status{};
}

void CUActivationLayer::configure(ITensor *input, ITensor *output, ActivationLayerInfo activation_info)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input);
    CU_THROW_ON(validate(input->info(), output != nullptr ? output->info() : nullptr, activation_info));
    _input  = input;
    _output = output != nullptr ? output : input;
    _act    = activation_info;
}

void CUActivationLayer::run()
{
    cugl_context                 *ctx = CUScheduler::get().context();
    const UniformQuantizationInfo qi  = _input->info()->quantization_info().uniform();
    const UniformQuantizationInfo qo  = _output->info()->quantization_info().uniform();
    CU_THROW_ON(cu_status(
        cugl_activation_qasymm8(ctx, cu_device_ptr(_input), cu_device_ptr(_output),
                                static_cast<int64_t>(_input->info()->tensor_shape().total_size()), to_cugl_activation(_act),
                                _act.a(), _act.b(), qi.scale, qi.offset, qo.scale, qo.offset),
        ctx, "CUActivationLayer::run"));
}

// ---- softmax (src/cpu/operators/CpuSoftmax.cpp: validate) -------------------------------------------------
Status CUSoftmaxLayer::validate(const ITensorInfo *input, const ITensorInfo *output, float beta, int32_t axis)
{
    (void)beta;
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input->data_type() != DataType::QASYMM8 || output->data_type() != DataType::QASYMM8,
                                    "QASYMM8 tensors only");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(axis != 0, "softmax along dimension 0 only");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->tensor_shape() != input->tensor_shape(), "input and output shapes differ");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!dense(input) || !dense(output), "padded tensors are not supported");
    // src/core/Utils.cpp:421-439: the output quantization of QASYMM8 softmax is fixed
    const UniformQuantizationInfo qo = output->quantization_info().uniform();
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(qo.scale != 1.f / 256.f || qo.offset != 0, "softmax output must be quantized with (1/256, 0)");
    return Status{};
}

void CUSoftmaxLayer::configure(ITensor *input, ITensor *output, float beta, int32_t axis)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input, output);
    CU_THROW_ON(validate(input->info(), output->info(), beta, axis));
    _input  = input;
    _output = output;
    _beta   = beta;
}

void CUSoftmaxLayer::run()
{
    cugl_context                 *ctx  = CUScheduler::get().context();
    const UniformQuantizationInfo qi   = _input->info()->quantization_info().uniform();
    const int32_t                 cols = static_cast<int32_t>(_input->info()->dimension(0));
    const int32_t                 rows = static_cast<int32_t>(_input->info()->tensor_shape().total_size_upper(1));
    CU_THROW_ON(cu_status(
        cugl_softmax_qasymm8(ctx, cu_device_ptr(_input), cu_device_ptr(_output), rows, cols, _beta, qi.scale, qi.offset), ctx,
        "CUSoftmaxLayer::run"));
}

// ---- flatten (src/cpu/operators/CpuFlatten.cpp) ------------------------------------------------------------------
Status CUFlattenLayer::validate(const ITensorInfo *input, const ITensorInfo *output)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input->data_type() != output->data_type(), "input and output data types differ");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input->tensor_shape().total_size() != output->tensor_shape().total_size(),
                                    "input and output hold different numbers of elements");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!dense(input) || !dense(output), "padded tensors are not supported");
    return Status{};
}

void CUFlattenLayer::configure(const ITensor *input, ITensor *output)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input, output);
    CU_THROW_ON(validate(input->info(), output->info()));
    _input  = input;
    _output = output;
}

void CUFlattenLayer::run()
{
    cugl_context *ctx = CUScheduler::get().context();
    CU_THROW_ON(cu_status(cugl_memcpy_d2d(ctx, cu_device_ptr(_output), cu_device_ptr(_input),
                                          _input->info()->tensor_shape().total_size() * _input->info()->element_size()),
                          ctx, "CUFlattenLayer::run"));
}
} // namespace arm_compute
