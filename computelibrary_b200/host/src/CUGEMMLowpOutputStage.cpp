#include "arm_compute/runtime/CUDA/functions/CUGEMMLowpOutputStage.h"

#include "CUHelpers.h"

namespace arm_compute
{
Status CUGEMMLowpOutputStage::validate(const ITensorInfo *input, const ITensorInfo *bias, const ITensorInfo *output,
                                       const GEMMLowpOutputStageInfo &info)
{
    // CpuGemmLowpOutputStage::validate (src/cpu/operators/CpuGemmLowpOutputStage.cpp:100-161)
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(input->data_type() != DataType::S32, "input must be S32");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_type() != DataType::QASYMM8 && output->data_type() != DataType::QASYMM8_SIGNED &&
                                        output->data_type() != DataType::QSYMM16,
                                    "output must be QASYMM8, QASYMM8_SIGNED or QSYMM16");
    // QSYMM16 exists for the fixed-point stage only (CpuGemmLowpOutputStage.cpp:73-80)
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->data_type() == DataType::QSYMM16 &&
                                        info.type != GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT,
                                    "a QSYMM16 output needs QUANTIZE_DOWN_FIXEDPOINT");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(info.type != GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT &&
                                        info.type != GEMMLowpOutputStageType::QUANTIZE_DOWN,
                                    "only QUANTIZE_DOWN and QUANTIZE_DOWN_FIXEDPOINT are implemented");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(info.gemmlowp_min_bound > info.gemmlowp_max_bound, "min bound above max bound");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->tensor_shape() != input->tensor_shape(), "input and output shapes differ");
    if (bias != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(bias->data_type() != DataType::S32, "bias must be S32");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(bias->num_dimensions() > 1 || bias->dimension(0) != input->dimension(0),
                                        "bias must be a vector of N elements");
    }
    if (info.is_quantized_per_channel)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(info.gemmlowp_multipliers.size() < input->dimension(0) ||
                                            info.gemmlowp_shifts.size() < input->dimension(0),
                                        "per-channel output stage needs N multipliers and shifts");
    }
    return Status{};
}

void CUGEMMLowpOutputStage::configure(const ITensor *input, const ITensor *bias, ITensor *output,
                                      const GEMMLowpOutputStageInfo &info)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(input, output);
    CU_THROW_ON(validate(input->info(), bias != nullptr ? bias->info() : nullptr, output->info(), info));
    _input.set(input);
    _bias.set(bias);
    _output.set(output);
    _info = info;
    if (info.is_quantized_per_channel)
    {
        cugl_context *ctx = CUScheduler::get().context();
        const size_t  n   = input->info()->dimension(0);
        CU_THROW_ON(cu_status(cugl_malloc(ctx, n * 4, &_d_mults), ctx, "CUGEMMLowpOutputStage::configure"));
        CU_THROW_ON(cu_status(cugl_malloc(ctx, n * 4, &_d_shifts), ctx, "CUGEMMLowpOutputStage::configure"));
        CU_THROW_ON(cu_status(cugl_memcpy_h2d(ctx, _d_mults, info.gemmlowp_multipliers.data(), n * 4), ctx, "copy"));
        CU_THROW_ON(cu_status(cugl_memcpy_h2d(ctx, _d_shifts, info.gemmlowp_shifts.data(), n * 4), ctx, "copy"));
        CU_THROW_ON(cu_status(cugl_sync(ctx), ctx, "sync"));
    }
}

void CUGEMMLowpOutputStage::run()
{
    cugl_context      *ctx = CUScheduler::get().context();
    const ITensorInfo *in  = _input.tensor()->info();
    const ITensorInfo *out = _output.tensor()->info();
    void              *dst = _output.device(false);
    const int32_t      N   = static_cast<int32_t>(in->dimension(0));
    const int32_t      M   = static_cast<int32_t>(in->tensor_shape().total_size_upper(1));
    const auto stage_fn = _info.type == GEMMLowpOutputStageType::QUANTIZE_DOWN ? cugl_output_stage_quantize_down : cugl_output_stage;
    CU_THROW_ON(cu_status(
        stage_fn(ctx, static_cast<const int32_t *>(_input.device(true)),
                          static_cast<int64_t>(in->strides_in_bytes()[1]), static_cast<const int32_t *>(_bias.device(true)),
                          dst, static_cast<int64_t>(out->strides_in_bytes()[1]), cu::to_cugl_dtype(out->data_type()),
                          M, N,
                          static_cast<const int32_t *>(_d_mults), static_cast<const int32_t *>(_d_shifts),
                          _info.gemmlowp_multiplier, _info.gemmlowp_shift, _info.is_quantized_per_channel ? N : 1,
                          _info.gemmlowp_offset, _info.gemmlowp_min_bound, _info.gemmlowp_max_bound),
        ctx, "CUGEMMLowpOutputStage::run"));
    _output.download();
}

CUGEMMLowpOutputStage::~CUGEMMLowpOutputStage()
{
    if (_d_mults != nullptr || _d_shifts != nullptr)
    {
        cugl_context *ctx = CUScheduler::get().context();
        cugl_sync(ctx);
        cugl_free(ctx, _d_mults);
        cugl_free(ctx, _d_shifts);
    }
}
} // namespace arm_compute
