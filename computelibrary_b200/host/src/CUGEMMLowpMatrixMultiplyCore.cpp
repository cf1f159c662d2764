#include "arm_compute/runtime/CUDA/functions/CUGEMMLowpMatrixMultiplyCore.h"

#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"

namespace arm_compute
{
namespace
{
int32_t to_cugl_dtype(DataType dt)
{
    switch (dt)
    {
        case DataType::QASYMM8:
            return CUGL_U8;
        case DataType::QASYMM8_SIGNED:
        case DataType::QSYMM8:
        case DataType::QSYMM8_PER_CHANNEL:
            return CUGL_S8;
        case DataType::S32:
            return CUGL_S32;
        default:
            return -1;
    }
}

// Translates the tensor infos + GEMMInfo into the C descriptor; the shape / type rules that cannot be
// expressed in the descriptor are checked here, the rest by cugl_gemmlowp_validate.
Status make_desc(const ITensorInfo *a, const ITensorInfo *b, const ITensorInfo *c, const ITensorInfo *output,
                 const GEMMInfo &gemm_info, cugl_gemm_desc &d)
{
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(a == nullptr || b == nullptr || output == nullptr, "nullptr tensor info");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(a->data_type() != DataType::QASYMM8 && a->data_type() != DataType::QASYMM8_SIGNED,
                                    "a: data type not in {QASYMM8, QASYMM8_SIGNED}");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(!is_data_type_quantized(b->data_type()),
                                    "b: data type not in {QASYMM8, QASYMM8_SIGNED, QSYMM8, QSYMM8_PER_CHANNEL}");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(to_cugl_dtype(output->data_type()) < 0,
                                    "output: data type not in {S32, QASYMM8, QASYMM8_SIGNED}");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(
        a->dimension(0) != b->dimension(1),
        "The product AB is defined only if the number of columns in A is equal to the number of rows in B");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.is_a_reshaped(), "Matrix A already reshaped is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.is_b_reshaped(), "Matrix B already reshaped is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.pretranspose_A(), "Matrix A already pretransposed is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.pretranspose_B(), "Matrix B already pretransposed is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.accumulate(), "Accumulation is not implemented by the CUDA backend");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->dimension(0) != b->dimension(0) || output->dimension(1) != a->dimension(1),
                                    "output shape must be [N, M]");
    const size_t batch_a = a->tensor_shape().total_size_upper(2);
    const size_t batch_b = b->tensor_shape().total_size_upper(2);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->tensor_shape().total_size_upper(2) != batch_a, "output batch differs from a");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(batch_b != 1 && batch_b != batch_a, "b must be 2-D or have a's batch count");
    const GEMMLowpOutputStageInfo s = gemm_info.gemmlowp_output_stage();
    if (c != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(c->data_type() != DataType::S32, "bias must be S32");
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(c->num_dimensions() > 1 || c->dimension(0) != b->dimension(0),
                                        "bias must be a vector of N elements");
    }
    if (s.type != GEMMLowpOutputStageType::NONE && s.is_quantized_per_channel)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(s.gemmlowp_multipliers.size() < b->dimension(0) ||
                                            s.gemmlowp_shifts.size() < b->dimension(0),
                                        "per-channel output stage needs N multipliers and shifts");
    }
    d                = cugl_gemm_desc{};
    d.M              = static_cast<int32_t>(a->dimension(1));
    d.N              = static_cast<int32_t>(b->dimension(0));
    d.K              = static_cast<int32_t>(a->dimension(0));
    d.batch          = static_cast<int32_t>(batch_a);
    d.lda            = static_cast<int64_t>(a->strides_in_bytes()[1]);
    d.ldb            = static_cast<int64_t>(b->strides_in_bytes()[1]);
    d.ldd            = static_cast<int64_t>(output->strides_in_bytes()[1]);
    d.a_batch_stride = static_cast<int64_t>(a->strides_in_bytes()[2]);
    d.b_batch_stride = batch_b > 1 ? static_cast<int64_t>(b->strides_in_bytes()[2]) : 0;
    d.d_batch_stride = static_cast<int64_t>(output->strides_in_bytes()[2]);
    d.a_dtype        = to_cugl_dtype(a->data_type());
    d.b_dtype        = to_cugl_dtype(b->data_type());
    d.dst_dtype      = to_cugl_dtype(output->data_type());
    d.a_offset       = a->quantization_info().uniform().offset; // added as given (CpuGemmLowpMatrixMultiplyCore.cpp:130-131)
    d.b_offset       = is_data_type_quantized_per_channel(b->data_type()) ? 0 : b->quantization_info().uniform().offset;
    switch (s.type)
    {
        case GEMMLowpOutputStageType::NONE:
            d.stage = CUGL_STAGE_NONE;
            break;
        case GEMMLowpOutputStageType::QUANTIZE_DOWN:
            d.stage = CUGL_STAGE_QUANTIZE_DOWN;
            break;
        case GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT:
            d.stage = CUGL_STAGE_QUANTIZE_DOWN_FIXEDPOINT;
            break;
        default:
            return Status(ErrorCode::RUNTIME_ERROR, "only output stages NONE, QUANTIZE_DOWN and QUANTIZE_DOWN_FIXEDPOINT are implemented");
    }
    d.is_quantized_per_channel   = s.is_quantized_per_channel ? 1 : 0;
    d.gemmlowp_multiplier        = s.gemmlowp_multiplier;
    d.gemmlowp_shift             = s.gemmlowp_shift;
    d.h_gemmlowp_multipliers     = s.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts          = s.gemmlowp_shifts.data();
    d.gemmlowp_offset            = s.gemmlowp_offset;
    d.gemmlowp_min_bound         = s.gemmlowp_min_bound;
    d.gemmlowp_max_bound         = s.gemmlowp_max_bound;
    d.has_bias                   = c != nullptr ? 1 : 0;
    d.reshape_b_only_on_first_run = gemm_info.reshape_b_only_on_first_run() ? 1 : 0;
    return Status{};
}
} // namespace

struct CUGEMMLowpMatrixMultiplyCore::Impl
{
    const ITensor  *a{nullptr};
    const ITensor  *b{nullptr};
    const ITensor  *c{nullptr};
    ITensor        *output{nullptr};
    GEMMInfo        gemm_info{};
    cugl_gemm_plan *plan{nullptr};
    bool            is_prepared{false};
};

CUGEMMLowpMatrixMultiplyCore::CUGEMMLowpMatrixMultiplyCore(std::shared_ptr<IMemoryManager> memory_manager,
                                                           IWeightsManager                *weights_manager)
    : _impl(std::make_unique<Impl>())
{
    // The workspace (K-major B, row / column sums, per-channel vectors) is owned by the cugl plan; the host
    // memory-manager hooks of the NE function have no device counterpart.
    ARM_COMPUTE_UNUSED(memory_manager, weights_manager);
}

CUGEMMLowpMatrixMultiplyCore::~CUGEMMLowpMatrixMultiplyCore()
{
    if (_impl && _impl->plan != nullptr)
    {
        cugl_gemmlowp_plan_destroy(_impl->plan);
    }
}

Status CUGEMMLowpMatrixMultiplyCore::validate(const ITensorInfo *a, const ITensorInfo *b, const ITensorInfo *c,
                                              const ITensorInfo *output, const GEMMInfo &gemm_info)
{
    cugl_gemm_desc d;
    ARM_COMPUTE_RETURN_ON_ERROR(make_desc(a, b, c, output, gemm_info, d));
    // the temporaries inside gemmlowp_output_stage() died with make_desc: validate without the vectors' contents
    const GEMMLowpOutputStageInfo s = gemm_info.gemmlowp_output_stage();
    d.h_gemmlowp_multipliers        = s.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts             = s.gemmlowp_shifts.data();
    const char *why = nullptr;
    if (cugl_gemmlowp_validate(&d, &why) != CUGL_SUCCESS)
    {
        return Status(ErrorCode::RUNTIME_ERROR, why != nullptr ? why : "invalid GEMMLowp configuration");
    }
    return Status{};
}

void CUGEMMLowpMatrixMultiplyCore::configure(const ITensor *a, const ITensor *b, const ITensor *c, ITensor *output,
                                             const GEMMInfo &gemm_info)
{
    ARM_COMPUTE_ERROR_ON_NULLPTR(a, b, output);
    ARM_COMPUTE_ERROR_THROW_ON(validate(a->info(), b->info(), c != nullptr ? c->info() : nullptr, output->info(), gemm_info));
    if (_impl->plan != nullptr)
    {
        cugl_gemmlowp_plan_destroy(_impl->plan);
        _impl->plan = nullptr;
    }
    _impl->a           = a;
    _impl->b           = b;
    _impl->c           = c;
    _impl->output      = output;
    _impl->gemm_info   = gemm_info;
    _impl->is_prepared = false;
    cugl_gemm_desc                 d;
    const GEMMLowpOutputStageInfo  s = gemm_info.gemmlowp_output_stage();
    ARM_COMPUTE_ERROR_THROW_ON(make_desc(a->info(), b->info(), c != nullptr ? c->info() : nullptr, output->info(), gemm_info, d));
    d.h_gemmlowp_multipliers = s.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts      = s.gemmlowp_shifts.data();
    cugl_context *ctx        = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_gemmlowp_plan_create(ctx, &d, &_impl->plan), ctx, "CUGEMMLowpMatrixMultiplyCore::configure"));
}

void CUGEMMLowpMatrixMultiplyCore::update_quantization_parameters(const GEMMLowpOutputStageInfo &output_stage)
{
    ARM_COMPUTE_ERROR_ON_MSG(_impl->plan == nullptr, "update_quantization_parameters before configure");
    _impl->gemm_info.set_gemmlowp_output_stage(output_stage);
    cugl_gemm_desc d;
    ARM_COMPUTE_ERROR_THROW_ON(make_desc(_impl->a->info(), _impl->b->info(), _impl->c != nullptr ? _impl->c->info() : nullptr,
                                         _impl->output->info(), _impl->gemm_info, d));
    d.h_gemmlowp_multipliers = output_stage.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts      = output_stage.gemmlowp_shifts.data();
    cugl_context *ctx        = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_gemmlowp_update_quantization(_impl->plan, &d), ctx, "CUGEMMLowpMatrixMultiplyCore::update_quantization_parameters"));
}

void CUGEMMLowpMatrixMultiplyCore::update_quantization_parameters()
{
    ARM_COMPUTE_ERROR_ON_MSG(_impl->plan == nullptr, "update_quantization_parameters before configure");
    const QuantizationInfo iq = _impl->a->info()->quantization_info();
    const QuantizationInfo wq = _impl->b->info()->quantization_info();
    const QuantizationInfo oq = _impl->output->info()->quantization_info();
    const DataType         dt = _impl->a->info()->data_type();
    GEMMLowpOutputStageInfo s;
    s.type                     = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    s.gemmlowp_offset          = oq.uniform().offset;
    s.gemmlowp_min_bound       = dt == DataType::QASYMM8 ? 0 : -128;
    s.gemmlowp_max_bound       = dt == DataType::QASYMM8 ? 255 : 127;
    s.is_quantized_per_channel = false;
    s.output_data_type         = _impl->output->info()->data_type();
    ARM_COMPUTE_ERROR_ON_MSG(iq.scale().empty() || wq.scale().empty() || oq.scale().empty(), "missing quantization scale");
    const float w0 = wq.scale()[0];
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_calculate_quantized_multipliers(iq.scale()[0], &w0, 1, oq.scale()[0],
                                                                              &s.gemmlowp_multiplier, &s.gemmlowp_shift),
                                         nullptr, "calculate_quantized_multipliers"));
    update_quantization_parameters(s);
}

void CUGEMMLowpMatrixMultiplyCore::prepare()
{
    if (_impl->is_prepared)
    {
        return;
    }
    ARM_COMPUTE_ERROR_ON_MSG(_impl->plan == nullptr, "prepare before configure");
    cugl_context *ctx = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_gemmlowp_prepare(_impl->plan, cu_device_ptr(_impl->b)), ctx, "CUGEMMLowpMatrixMultiplyCore::prepare"));
    if (_impl->gemm_info.reshape_b_only_on_first_run())
    {
        _impl->b->mark_as_unused(); // as NEGEMMLowpMatrixMultiplyCore.cpp:180-183
    }
    _impl->is_prepared = true;
}

void CUGEMMLowpMatrixMultiplyCore::run()
{
    prepare();
    cugl_context *ctx  = CUScheduler::get().context();
    const bool    need_b = !_impl->gemm_info.reshape_b_only_on_first_run();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(
        cugl_gemmlowp_run(_impl->plan, cu_device_ptr(_impl->a), need_b ? cu_device_ptr(_impl->b) : nullptr,
                          static_cast<const int32_t *>(cu_device_ptr(_impl->c)), cu_device_ptr(_impl->output)),
        ctx, "CUGEMMLowpMatrixMultiplyCore::run"));
}
} // namespace arm_compute
