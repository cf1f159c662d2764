#include "arm_compute/runtime/CUDA/functions/CUGEMMLowpMatrixMultiplyCore.h"

#include "arm_compute/core/Utils.h"
#include "arm_compute/core/utils/quantization/AsymmHelpers.h"

#include "CUHelpers.h"

namespace arm_compute
{
namespace
{
// [K, M, batch...] seen through GEMMInfo::reinterpret_input_as_3d / depth_output_gemm3d
// (CpuGemmLowpMatrixMultiplyCore.cpp:519-535): rows of the matrix are dimensions 1 and 2 folded together, which is
// only a change of index arithmetic when the planes follow each other without a gap.
struct MatrixView
{
    size_t  rows{0}, batch{1};
    int64_t ld{0}, batch_stride{0};
};

Status matrix_view(const ITensorInfo *t, bool fold_3d, const char *name, MatrixView &v)
{
    const Strides &st = t->strides_in_bytes();
    if (fold_3d)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_MSG_VAR(t->num_dimensions() > 2 && st[2] != st[1] * t->dimension(1),
                                            "%s: a 3-D reinterpreted matrix must have no padding between its planes", name);
        v.rows         = t->dimension(1) * t->dimension(2);
        v.batch        = t->tensor_shape().total_size_upper(3);
        v.batch_stride = static_cast<int64_t>(st[3]);
    }
    else
    {
        v.rows         = t->dimension(1);
        v.batch        = t->tensor_shape().total_size_upper(2);
        v.batch_stride = static_cast<int64_t>(st[2]);
    }
    v.ld = static_cast<int64_t>(st[1]);
    return Status{};
}

// Translates the tensor infos + GEMMInfo into the C descriptor; the shape / type rules that cannot be
// expressed in the descriptor are checked here (CpuGemmLowpMatrixMultiplyCore.cpp:362-401), the rest by
// cugl_gemmlowp_validate.  `s` must outlive `d`: the descriptor points into its per-channel vectors.
Status make_desc(const ITensorInfo *a, const ITensorInfo *b, const ITensorInfo *c, const ITensorInfo *output,
                 const GEMMInfo &gemm_info, const GEMMLowpOutputStageInfo &s, cugl_gemm_desc &d)
{
    ARM_COMPUTE_RETURN_ERROR_ON_NULLPTR(a, b, output);
    ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(a, 1, DataType::QASYMM8, DataType::QASYMM8_SIGNED);
    ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(b, 1, DataType::QASYMM8, DataType::QASYMM8_SIGNED, DataType::QSYMM8,
                                                         DataType::QSYMM8_PER_CHANNEL);
    ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(output, 1, DataType::S32, DataType::QASYMM8,
                                                         DataType::QASYMM8_SIGNED, DataType::F32);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(c != nullptr && s.type == GEMMLowpOutputStageType::NONE,
                                    "Bias addition not supported in NEGEMMLowpMatrixMultiplyCore for output S32");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(
        a->dimension(0) != b->dimension(1),
        "The product AB is defined only if the number of columns in A is equal to the number of rows in B");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.is_a_reshaped(), "Matrix A already reshaped is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.is_b_reshaped(), "Matrix B already reshaped is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.pretranspose_A(), "Matrix A already pretransposed is not supported");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.pretranspose_B(), "Matrix B already pretransposed is not supported");
    if (output->data_type() == DataType::F32) // int8_dequantize_f32_path (CpuGemmLowpMatrixMultiplyCore.cpp:387-391)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(a, 1, DataType::QASYMM8_SIGNED);
        ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(b, 1, DataType::QASYMM8_SIGNED);
        ARM_COMPUTE_RETURN_ERROR_ON_MSG(s.type != GEMMLowpOutputStageType::NONE, "an F32 output takes no output stage");
    }
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.accumulate() && s.type != GEMMLowpOutputStageType::NONE,
                                    "Accumulation is not supported for output QASYMM8/QASYMM8_SIGNED");

    MatrixView va, vo;
    ARM_COMPUTE_RETURN_ON_ERROR(matrix_view(a, gemm_info.reinterpret_input_as_3d(), "a", va));
    ARM_COMPUTE_RETURN_ON_ERROR(matrix_view(output, gemm_info.depth_output_gemm3d() != 0, "output", vo));
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(gemm_info.depth_output_gemm3d() != 0 &&
                                        output->dimension(2) != static_cast<size_t>(gemm_info.depth_output_gemm3d()),
                                    "depth_output_gemm3d differs from the output's third dimension");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(output->dimension(0) != b->dimension(0) || vo.rows != va.rows,
                                    "output shape must be [N, M]");
    const size_t batch_b = b->tensor_shape().total_size_upper(2);
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(vo.batch != va.batch, "output batch differs from a");
    ARM_COMPUTE_RETURN_ERROR_ON_MSG(batch_b != 1 && batch_b != va.batch, "b must be 2-D or have a's batch count");
    if (c != nullptr)
    {
        ARM_COMPUTE_RETURN_ERROR_ON_DATA_TYPE_CHANNEL_NOT_IN(c, 1, DataType::S32);
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
    d.M              = static_cast<int32_t>(va.rows);
    d.N              = static_cast<int32_t>(b->dimension(0));
    d.K              = static_cast<int32_t>(a->dimension(0));
    d.batch          = static_cast<int32_t>(va.batch);
    d.lda            = va.ld;
    d.ldb            = static_cast<int64_t>(b->strides_in_bytes()[1]);
    d.ldd            = vo.ld;
    d.a_batch_stride = va.batch_stride;
    d.b_batch_stride = batch_b > 1 ? static_cast<int64_t>(b->strides_in_bytes()[2]) : 0;
    d.d_batch_stride = vo.batch_stride;
    d.a_dtype        = cu::to_cugl_dtype(a->data_type());
    d.b_dtype        = cu::to_cugl_dtype(b->data_type());
    d.dst_dtype      = cu::to_cugl_dtype(output->data_type());
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
            return Status(ErrorCode::RUNTIME_ERROR,
                          "only output stages NONE, QUANTIZE_DOWN and QUANTIZE_DOWN_FIXEDPOINT are implemented");
    }
    d.is_quantized_per_channel    = s.is_quantized_per_channel ? 1 : 0;
    d.gemmlowp_multiplier         = s.gemmlowp_multiplier;
    d.gemmlowp_shift              = s.gemmlowp_shift;
    d.h_gemmlowp_multipliers      = s.gemmlowp_multipliers.data();
    d.h_gemmlowp_shifts           = s.gemmlowp_shifts.data();
    d.gemmlowp_offset             = s.gemmlowp_offset;
    d.gemmlowp_min_bound          = s.gemmlowp_min_bound;
    d.gemmlowp_max_bound          = s.gemmlowp_max_bound;
    d.has_bias                    = c != nullptr ? 1 : 0;
    d.reshape_b_only_on_first_run = gemm_info.reshape_b_only_on_first_run() ? 1 : 0;
    d.accumulate                  = gemm_info.accumulate() ? 1 : 0;
    // the s8 x s8 -> f32 path multiplies the int32 result by both operand scales (CpuGemmLowpMatrixMultiplyCore.cpp:305-320)
    d.dequantize_scale = output->data_type() == DataType::F32
                             ? a->quantization_info().uniform().scale * b->quantization_info().uniform().scale
                             : 0.f;
    return Status{};
}

bool same_geometry(const cugl_gemm_desc &x, const cugl_gemm_desc &y)
{
    return x.M == y.M && x.N == y.N && x.K == y.K && x.batch == y.batch && x.lda == y.lda && x.ldb == y.ldb &&
           x.ldd == y.ldd && x.a_batch_stride == y.a_batch_stride && x.b_batch_stride == y.b_batch_stride &&
           x.d_batch_stride == y.d_batch_stride;
}
} // namespace

struct CUGEMMLowpMatrixMultiplyCore::Impl
{
    explicit Impl(std::shared_ptr<IMemoryManager> mm) : memory_group(std::move(mm)) {}
    MemoryGroup             memory_group;
    CUOperand               a{}, b{}, c{}, output{};
    GEMMInfo                gemm_info{};
    GEMMLowpOutputStageInfo stage{};
    cugl_gemm_desc          desc{};
    cugl_gemm_plan         *plan{nullptr};
    cu::TemporaryWorkspace  workspace{};
    bool                    is_prepared{false};

    void destroy_plan()
    {
        if (plan != nullptr)
        {
            cugl_gemmlowp_plan_destroy(plan);
            plan = nullptr;
        }
    }

    // Tensors are allocated -- and, in the validation fixtures, padded -- after configure(): when the row pitches
    // seen at run time differ from the ones the plan was created for, the plan is created again for them.
    void refresh_plan()
    {
        cugl_gemm_desc now;
        CU_THROW_ON(make_desc(a.tensor()->info(), b.tensor()->info(), c.tensor() != nullptr ? c.tensor()->info() : nullptr,
                              output.tensor()->info(), gemm_info, stage, now));
        if (plan != nullptr && same_geometry(now, desc))
        {
            return;
        }
        destroy_plan();
        desc              = now;
        cugl_context *ctx = CUScheduler::get().context();
        CU_THROW_ON(cu_status(cugl_gemmlowp_plan_create(ctx, &desc, &plan), ctx, "CUGEMMLowpMatrixMultiplyCore"));
        is_prepared = false;
    }
};

CUGEMMLowpMatrixMultiplyCore::CUGEMMLowpMatrixMultiplyCore(std::shared_ptr<IMemoryManager> memory_manager,
                                                           IWeightsManager                *weights_manager)
    : _impl(std::make_unique<Impl>(std::move(memory_manager)))
{
    // B is re-laid out on the device inside the plan; a host-side weights manager has nothing to manage here
    ARM_COMPUTE_UNUSED(weights_manager);
}

CUGEMMLowpMatrixMultiplyCore::~CUGEMMLowpMatrixMultiplyCore()
{
    if (_impl)
    {
        _impl->destroy_plan();
    }
}

Status CUGEMMLowpMatrixMultiplyCore::validate(const ITensorInfo *a, const ITensorInfo *b, const ITensorInfo *c,
                                              const ITensorInfo *output, const GEMMInfo &gemm_info)
{
    cugl_gemm_desc                d;
    const GEMMLowpOutputStageInfo stage = gemm_info.gemmlowp_output_stage();
    ARM_COMPUTE_RETURN_ON_ERROR(make_desc(a, b, c, output, gemm_info, stage, d));
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
    CU_THROW_ON(validate(a->info(), b->info(), c != nullptr ? c->info() : nullptr, output->info(), gemm_info));
    _impl->destroy_plan();
    _impl->a.set(a);
    _impl->b.set(b);
    _impl->c.set(c);
    _impl->output.set(output);
    _impl->gemm_info   = gemm_info;
    _impl->stage       = gemm_info.gemmlowp_output_stage();
    _impl->is_prepared = false;
    _impl->refresh_plan();
    // Temporary-lifetime workspace (row sums, the 16-byte-pitch copy of an unaligned A): managed by the memory
    // group so that a memory manager can share the bytes with other functions (MemoryHelpers.h:56-105)
    _impl->workspace.configure(_impl->memory_group, cugl_gemmlowp_plan_temp_bytes(_impl->plan));
}

void CUGEMMLowpMatrixMultiplyCore::update_quantization_parameters(const GEMMLowpOutputStageInfo &output_stage)
{
    CU_ERROR_IF(_impl->plan == nullptr, "update_quantization_parameters before configure");
    _impl->stage = output_stage;
    GEMMLowpOutputStageInfo copy = output_stage; // the setter takes a non-const reference (GEMMInfo.h:230)
    _impl->gemm_info.set_gemmlowp_output_stage(copy);
    cugl_gemm_desc d;
    CU_THROW_ON(make_desc(_impl->a.tensor()->info(), _impl->b.tensor()->info(),
                          _impl->c.tensor() != nullptr ? _impl->c.tensor()->info() : nullptr, _impl->output.tensor()->info(),
                          _impl->gemm_info, _impl->stage, d));
    cugl_context *ctx = CUScheduler::get().context();
    if (!same_geometry(d, _impl->desc))
    {
        _impl->refresh_plan(); // new pitches: the new plan reads the new parameters anyway
        return;
    }
    CU_THROW_ON(cu_status(cugl_gemmlowp_update_quantization(_impl->plan, &d), ctx,
                          "CUGEMMLowpMatrixMultiplyCore::update_quantization_parameters"));
    _impl->desc = d;
}

void CUGEMMLowpMatrixMultiplyCore::update_quantization_parameters()
{
    CU_ERROR_IF(_impl->plan == nullptr, "update_quantization_parameters before configure");
    // NEGEMMLowpMatrixMultiplyCore.cpp:118-159: a per-tensor fixed-point stage from the three quantizations
    const ITensorInfo      *a  = _impl->a.tensor()->info();
    const ITensorInfo      *b  = _impl->b.tensor()->info();
    const ITensorInfo      *o  = _impl->output.tensor()->info();
    const DataType          dt = a->data_type();
    GEMMLowpOutputStageInfo s;
    s.type                     = GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT;
    s.gemmlowp_offset          = o->quantization_info().uniform().offset;
    s.gemmlowp_min_bound       = dt == DataType::QASYMM8 ? 0 : -128;
    s.gemmlowp_max_bound       = dt == DataType::QASYMM8 ? 255 : 127;
    s.is_quantized_per_channel = false;
    s.output_data_type         = o->data_type();
    CU_THROW_ON(quantization::calculate_quantized_multipliers(a->quantization_info(), b->quantization_info(),
                                                              o->quantization_info(), s));
    update_quantization_parameters(s);
}

void CUGEMMLowpMatrixMultiplyCore::prepare()
{
    CU_ERROR_IF(_impl->plan == nullptr, "prepare before configure");
    _impl->refresh_plan();
    if (_impl->is_prepared)
    {
        return;
    }
    cugl_context *ctx = CUScheduler::get().context();
    CU_THROW_ON(cu_status(cugl_gemmlowp_prepare(_impl->plan, _impl->b.device(true)), ctx, "CUGEMMLowpMatrixMultiplyCore::prepare"));
    if (_impl->gemm_info.reshape_b_only_on_first_run())
    {
        _impl->b.tensor()->mark_as_unused(); // as NEGEMMLowpMatrixMultiplyCore.cpp:180-183
    }
    _impl->is_prepared = true;
}

void CUGEMMLowpMatrixMultiplyCore::run()
{
    prepare();
    MemoryGroupResourceScope scope_mg(_impl->memory_group);
    cugl_context *ctx    = CUScheduler::get().context();
    const bool    need_b = !_impl->gemm_info.reshape_b_only_on_first_run();
    if (_impl->workspace.bytes() != 0 && cugl_gemmlowp_plan_temp_bytes(_impl->plan) <= _impl->workspace.bytes())
    {
        CU_THROW_ON(cu_status(cugl_gemmlowp_plan_bind_temp(_impl->plan, _impl->workspace.device_ptr(), _impl->workspace.bytes()),
                              ctx, "CUGEMMLowpMatrixMultiplyCore::run"));
    }
    // an accumulating run reads the output first: a staged host output has to travel in as well
    void *dst = _impl->output.device(_impl->gemm_info.accumulate());
    CU_THROW_ON(cu_status(cugl_gemmlowp_run(_impl->plan, _impl->a.device(true), need_b ? _impl->b.device(true) : nullptr,
                                            static_cast<const int32_t *>(_impl->c.device(true)), dst),
                          ctx, "CUGEMMLowpMatrixMultiplyCore::run"));
    _impl->output.download(); // host output tensors only; blocks
}
} // namespace arm_compute
