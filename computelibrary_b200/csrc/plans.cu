// Plan objects behind the cugl C ABI: the CUDA counterparts of CpuGemmLowpMatrixMultiplyCore
// (configure / prepare / run with its auxiliary tensors) and CpuGemmConv2d (im2col + GEMMLowp), plus
// the thin entry points of the stand-alone kernels.
#include "kernels.cuh"

#include <climits>
#include <cstring>
#include <vector>

using namespace cugl;

namespace
{
inline int64_t round_up(int64_t v, int64_t m)
{
    return (v + m - 1) / m * m;
}
inline bool is_q8(int32_t t)
{
    return t == CUGL_U8 || t == CUGL_S8;
}

// Device-side state one quantized GEMM needs besides its operands: the auxiliary tensors of
// CpuGemmLowpMatrixMultiplyCore.h:144-155 (VectorSumCol, VectorSumRow, TmpB) and the per-channel
// output-stage vectors.
struct GemmCore
{
    cugl_context *ctx = nullptr;
    int           M = 0, N = 0, K = 0;
    bool          a_signed = false, b_signed = false;
    int32_t       dst_dtype = CUGL_U8;
    int32_t       a_off = 0, b_off = 0;
    int32_t       stage = CUGL_STAGE_NONE;
    bool          per_channel = false;
    int32_t       mult = 0, shift = 0, result_offset = 0, min_bound = INT32_MIN, max_bound = INT32_MAX;
    bool          accumulate = false; // stage NONE: dst += result
    float         dq_scale   = 0.f;   // F32 destination: result * dq_scale
    uint8_t      *d_bt     = nullptr; // [N][ldbt], K-major, zero padded
    int64_t       ldbt     = 0;
    int32_t      *d_colsum = nullptr; // [N]
    int32_t      *d_rowsum = nullptr; // [M]; plan-owned, allocated when first needed unless a temporary workspace is bound
    int32_t      *d_rowsum_bound = nullptr; // row sums inside the caller's temporary workspace
    int           rowsum_len = 0;
    // A whose base or row pitch is not a multiple of 16 bytes cannot be described to the TMA engine.  A copy with
    // rows of round_up(K, 16) bytes in temporary memory keeps such products on the tensor cores (the role of the
    // TmpA slot of CpuGemmLowpMatrixMultiplyCore.h:144-155, there an interleaved copy of A).
    uint8_t      *d_tmp_a = nullptr;       // plan-owned copy, allocated on first use unless a workspace is bound
    size_t        tmp_a_capacity = 0;
    uint8_t      *d_tmp_a_bound = nullptr; // inside the caller's temporary workspace
    int64_t       lda_hint = 0;            // row pitch of A announced at configure time (sizes the workspace share)
    int           tmp_a_rows = 0;          // rows one launch copies at most
    int32_t      *d_mults  = nullptr; // [N]
    int32_t      *d_shifts = nullptr;
    bool          force_simt = false;
    bool          allow_pair = true; // SM-pair (cta_group::2) kernel permitted
    bool          generic_stage = false; // a left shift or an INT32_MIN multiplier is present
    bool          wide_stage    = false; // shifts in [2, 31], multipliers in [0, 2^31), no row-sum term
    int           max_shift     = 0;     // largest right shift of the stage
    int           pack_stage    = 0;     // < 0: keep off the saturating-pack encoding of the output stage
    int           epi_warps     = 0;     // 4 / 8 force that build of the tensor-core kernels, 0 = automatic
    int           channel_major = 0;     // > 0 / < 0 force / forbid the channel-major kernel, 0 = automatic
    int           split_tail    = 0;     // < 0: the SM-pair kernel keeps the tiles of a short last wave whole
    int           block_n       = 0;     // 64 / 128 / 256 force that tile width of the one-CTA kernels, 0 = automatic
    int           pair_drain    = 0;     // < 0: every accumulator buffer is drained on its own
    int           tma_store     = 0;     // < 0: no bulk tensor stores in the epilogue
    int           resident_b    = 0;     // < 0: the implicit convolution reloads the weights with every tile
    int           double_tile   = 0;     // < 0: the implicit convolution keeps 128-row units of work

    // bytes of the row-sum vector as a share of a temporary workspace (none without a B offset)
    size_t rowsum_bytes() const
    {
        return b_off != 0 ? static_cast<size_t>(round_up(sizeof(int32_t) * static_cast<int64_t>(rowsum_len), 256)) : 0;
    }

    size_t tmp_a_bytes() const
    {
        return (lda_hint & 15) != 0 ? static_cast<size_t>(round_up(round_up(K, 16) * static_cast<int64_t>(tmp_a_rows), 256)) : 0;
    }

    cugl_status tmp_a_buffer(size_t bytes, uint8_t **out)
    {
        if (d_tmp_a_bound != nullptr && bytes <= tmp_a_bytes())
        {
            *out = d_tmp_a_bound;
            return CUGL_SUCCESS;
        }
        if (d_tmp_a == nullptr || tmp_a_capacity < bytes)
        {
            if (d_tmp_a != nullptr)
            {
                CUGL_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
                cugl_free(ctx, d_tmp_a);
                d_tmp_a = nullptr;
            }
            CUGL_TRY(cugl_malloc(ctx, bytes, reinterpret_cast<void **>(&d_tmp_a)));
            tmp_a_capacity = bytes;
        }
        *out = d_tmp_a;
        return CUGL_SUCCESS;
    }

    // the row sums live in the bound workspace, else in plan-owned memory allocated on first use
    cugl_status rowsum_buffer(int32_t **out)
    {
        if (d_rowsum_bound != nullptr)
        {
            *out = d_rowsum_bound;
            return CUGL_SUCCESS;
        }
        if (d_rowsum == nullptr)
        {
            CUGL_TRY(cugl_malloc(ctx, sizeof(int32_t) * static_cast<size_t>(rowsum_len > 0 ? rowsum_len : 1),
                                 reinterpret_cast<void **>(&d_rowsum)));
        }
        *out = d_rowsum;
        return CUGL_SUCCESS;
    }

    cugl_status alloc(int n_b_copies, int rowsum_len)
    {
        ldbt = round_up(K, 128);
        CUGL_TRY(cugl_malloc(ctx, static_cast<size_t>(ldbt) * N * n_b_copies, reinterpret_cast<void **>(&d_bt)));
        CUGL_TRY(cugl_malloc(ctx, sizeof(int32_t) * N * n_b_copies, reinterpret_cast<void **>(&d_colsum)));
        this->rowsum_len = rowsum_len;
        CUGL_TRY(cugl_memset(ctx, d_bt, 0, static_cast<size_t>(ldbt) * N * n_b_copies));
        return CUGL_SUCCESS;
    }

    cugl_status upload_stage_vectors(const int32_t *h_mults, const int32_t *h_shifts)
    {
        // the integer-multiply stage runs on the generic encoding
        generic_stage = stage == CUGL_STAGE_QUANTIZE_DOWN || (!per_channel && (shift < 0 || mult == INT32_MIN));
        wide_stage    = stage == CUGL_STAGE_QUANTIZE_DOWN_FIXEDPOINT && b_off == 0 &&
                     (per_channel || (shift >= 2 && shift <= 31 && mult >= 0));
        max_shift = shift;
        if (!per_channel)
        {
            return CUGL_SUCCESS;
        }
        for (int i = 0; i < N; ++i)
        {
            max_shift     = h_shifts[i] > max_shift || i == 0 ? h_shifts[i] : max_shift;
            generic_stage = generic_stage || h_shifts[i] < 0 || h_mults[i] == INT32_MIN;
            wide_stage    = wide_stage && h_shifts[i] >= 2 && h_shifts[i] <= 31 && h_mults[i] >= 0;
        }
        if (d_mults == nullptr)
        {
            CUGL_TRY(cugl_malloc(ctx, sizeof(int32_t) * N, reinterpret_cast<void **>(&d_mults)));
            CUGL_TRY(cugl_malloc(ctx, sizeof(int32_t) * N, reinterpret_cast<void **>(&d_shifts)));
        }
        // pageable source: the copy is staged before the call returns, so the caller's vectors may die
        CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(d_mults, h_mults, sizeof(int32_t) * N, cudaMemcpyHostToDevice,
                                           ctx->stream));
        CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(d_shifts, h_shifts, sizeof(int32_t) * N, cudaMemcpyHostToDevice,
                                           ctx->stream));
        CUGL_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        return CUGL_SUCCESS;
    }

    void release()
    {
        if (ctx == nullptr)
        {
            return;
        }
        cugl_free(ctx, d_bt);
        cugl_free(ctx, d_colsum);
        cugl_free(ctx, d_rowsum);
        cugl_free(ctx, d_tmp_a);
        d_tmp_a = nullptr;
        cugl_free(ctx, d_mults);
        cugl_free(ctx, d_shifts);
        d_bt = nullptr;
        d_colsum = d_rowsum = d_mults = d_shifts = nullptr;
    }

    EpilogueParams epilogue(const int32_t *bias, int b_copy, const int32_t *rowsum = nullptr) const
    {
        EpilogueParams ep{};
        ep.colsum = a_off != 0 ? d_colsum + static_cast<size_t>(b_copy) * N : nullptr;
        ep.rowsum = b_off != 0 ? rowsum : nullptr;
        ep.bias   = bias;
        ep.mults  = per_channel ? d_mults : nullptr;
        ep.shifts = per_channel ? d_shifts : nullptr;
        ep.mult   = mult;
        ep.shift  = shift;
        ep.a_off  = a_off;
        ep.b_off  = b_off;
        ep.k_term = (a_off != 0 && b_off != 0)
                        ? static_cast<int32_t>(static_cast<uint32_t>(a_off) * static_cast<uint32_t>(b_off) *
                                               static_cast<uint32_t>(K))
                        : 0;
        ep.result_offset  = result_offset;
        const int32_t tlo = dst_dtype == CUGL_S8 ? -128 : 0;
        const int32_t thi = dst_dtype == CUGL_S8 ? 127 : 255;
        ep.lo             = min_bound > tlo ? min_bound : tlo;
        ep.hi             = max_bound < thi ? max_bound : thi;
        if (stage == CUGL_STAGE_QUANTIZE_DOWN && min_bound == max_bound)
        {
            // tests/validation/reference/GEMMLowp.cpp:93-97: equal bounds mean "no bounded ReLU", type range only
            ep.lo = tlo;
            ep.hi = thi;
        }
        ep.stage          = stage;
        ep.out_signed     = dst_dtype == CUGL_S8;
        ep.out_f32        = dst_dtype == CUGL_F32 ? 1 : 0;
        ep.accumulate     = accumulate ? 1 : 0;
        ep.dq_scale       = dq_scale;
        return ep;
    }

    bool uses_tcgen05(const GemmOperands &op) const
    {
        return !force_simt && gemmlowp_tcgen05_supported(op);
    }

    // rows x K product against B copy b_copy.
    cugl_status gemm(const void *d_a, int64_t lda, int rows, void *d_dst, int64_t ldd, const int32_t *d_bias,
                     int b_copy, int rowsum_off, void *const *extra_dst = nullptr, int n_extra = 0,
                     const void *d_residual = nullptr, int res_floor = 0, int res_cap = 255)
    {
        GemmOperands op{};
        op.a        = d_a;
        op.bt       = d_bt + static_cast<size_t>(b_copy) * ldbt * N;
        op.dst      = d_dst;
        op.lda      = lda;
        op.ldbt     = ldbt;
        op.ldd      = ldd;
        op.M        = rows;
        op.N        = N;
        op.K        = K;
        op.a_signed = a_signed;
        op.b_signed = b_signed;
        op.generic_stage = generic_stage;
        op.wide_stage    = wide_stage;
        op.max_shift     = max_shift;
        op.pack_stage    = pack_stage;
        op.epi_warps     = epi_warps;
        op.channel_major = channel_major;
        op.split_tail    = split_tail;
        op.block_n       = block_n;
        op.pair_drain    = pair_drain;
        op.tma_store     = tma_store;
        op.resident_b    = resident_b;
        op.double_tile   = double_tile;
        op.n_extra_dst   = n_extra;
        op.residual      = d_residual;
        op.res_floor     = res_floor;
        op.res_cap       = res_cap;
        for (int i = 0; i < n_extra; ++i)
        {
            op.extra_dst[i] = extra_dst[i];
        }
        if (!force_simt && ((reinterpret_cast<uintptr_t>(d_a) | static_cast<uint64_t>(lda)) & 15) != 0)
        {
            const int64_t kp  = round_up(K, 16);
            uint8_t      *tmp = nullptr;
            CUGL_TRY(tmp_a_buffer(static_cast<size_t>(kp) * rows, &tmp));
            CUGL_CUDA_TRY(ctx, cudaMemcpy2DAsync(tmp, kp, d_a, lda, K, rows, cudaMemcpyDeviceToDevice, ctx->stream));
            op.a   = tmp; // bytes K .. kp-1 of a row are never read: the tensor map ends at K
            op.lda = kp;
        }
        if ((n_extra > 0 || d_residual != nullptr) && !uses_tcgen05(op))
        {
            return fail(ctx, CUGL_UNSUPPORTED_CONFIG,
                        "several destinations or a fused residual need the tensor-core kernel (16-byte aligned A "
                        "with 16-byte row pitch)");
        }
        int32_t *rowsum = nullptr;
        if (b_off != 0)
        {
            CUGL_TRY(rowsum_buffer(&rowsum));
            rowsum += rowsum_off;
            CUGL_TRY(launch_reduce_rows(ctx, op.a, a_signed, rows, K, op.lda, 1, rowsum));
        }
        const EpilogueParams ep = epilogue(d_bias, b_copy, rowsum);
        return uses_tcgen05(op) ? launch_gemmlowp_tcgen05(ctx, op, ep, allow_pair) : launch_gemmlowp_simt(ctx, op, ep);
    }
};

} // namespace

// need_host_vectors = false: the per-channel multipliers and shifts live in device memory only (the
// allocation-free entry point), so their host copies are neither required nor read.
const char *cugl::validate_gemm_desc(const cugl_gemm_desc *d, cugl_status *code, bool need_host_vectors)
{
    *code = CUGL_INVALID_ARGUMENT;
    if (d == nullptr) return "descriptor is NULL";
    if (d->M < 1 || d->N < 1 || d->K < 1 || d->batch < 1) return "M, N, K and batch must be positive";
    if (!is_q8(d->a_dtype)) return "A must be QASYMM8 or QASYMM8_SIGNED";
    if (!is_q8(d->b_dtype)) return "B must be QASYMM8, QASYMM8_SIGNED, QSYMM8 or QSYMM8_PER_CHANNEL";
    if (d->stage != CUGL_STAGE_NONE && d->stage != CUGL_STAGE_QUANTIZE_DOWN_FIXEDPOINT &&
        d->stage != CUGL_STAGE_QUANTIZE_DOWN)
    {
        *code = CUGL_UNSUPPORTED_CONFIG;
        return "only output stages NONE, QUANTIZE_DOWN and QUANTIZE_DOWN_FIXEDPOINT are implemented";
    }
    if (d->stage == CUGL_STAGE_QUANTIZE_DOWN)
    {
        if (d->is_quantized_per_channel)
        {
            for (int i = 0; need_host_vectors && d->h_gemmlowp_shifts != nullptr && i < d->N; ++i)
            {
                if (d->h_gemmlowp_shifts[i] < 0 || d->h_gemmlowp_shifts[i] > 31) return "QUANTIZE_DOWN needs shifts in [0, 31]";
            }
        }
        else if (d->gemmlowp_shift < 0 || d->gemmlowp_shift > 31)
        {
            return "QUANTIZE_DOWN needs a shift in [0, 31]";
        }
    }
    if (d->stage == CUGL_STAGE_NONE)
    {
        if (d->dst_dtype != CUGL_S32 && d->dst_dtype != CUGL_F32) return "output stage NONE requires an S32 or F32 output";
        if (d->has_bias) return "Bias addition not supported in NEGEMMLowpMatrixMultiplyCore for output S32";
        if (d->dst_dtype == CUGL_F32 && !(d->dequantize_scale > 0.f)) return "an F32 output needs a positive dequantize_scale";
    }
    else
    {
        if (!is_q8(d->dst_dtype)) return "a quantize-down output stage requires a QASYMM8 / QASYMM8_SIGNED output";
        if (d->accumulate) return "Accumulation is not supported for output QASYMM8/QASYMM8_SIGNED";
        if (d->gemmlowp_min_bound > d->gemmlowp_max_bound) return "gemmlowp_min_bound > gemmlowp_max_bound";
        if (d->is_quantized_per_channel)
        {
            if (need_host_vectors && (d->h_gemmlowp_multipliers == nullptr || d->h_gemmlowp_shifts == nullptr))
                return "per-channel output stage needs N multipliers and shifts";
            if (d->dst_dtype != CUGL_U8 && d->N > 1 && d->b_offset != 0)
                return "per-channel requantisation with a non-zero B offset is only defined for QASYMM8 output";
        }
    }
    const int64_t dsz = (d->dst_dtype == CUGL_S32 || d->dst_dtype == CUGL_F32) ? 4 : 1;
    if (d->lda < d->K) return "lda is smaller than a row of A";
    if (d->ldb < d->N) return "ldb is smaller than a row of B";
    if (d->ldd < d->N * dsz) return "ldd is smaller than a row of the output";
    if (dsz == 4 && (d->ldd % 4) != 0) return "ldd of an S32 / F32 output must be a multiple of 4";
    if (d->batch > 1)
    {
        if (d->a_batch_stride < static_cast<int64_t>(d->M) * d->lda) return "a_batch_stride overlaps batches";
        if (d->d_batch_stride < static_cast<int64_t>(d->M) * d->ldd) return "d_batch_stride overlaps batches";
        if (d->b_batch_stride != 0 && d->b_batch_stride < static_cast<int64_t>(d->K) * d->ldb)
            return "b_batch_stride overlaps batches";
    }
    *code = CUGL_SUCCESS;
    return nullptr;
}

namespace
{
const char *validate_gemm(const cugl_gemm_desc *d, cugl_status *code)
{
    return cugl::validate_gemm_desc(d, code, true);
}
} // namespace

struct cugl_gemm_plan
{
    cugl_context        *ctx = nullptr;
    cugl_gemm_desc       desc{};
    std::vector<int32_t> h_mults, h_shifts;
    GemmCore             core;
    bool                 collapse_batch = false; // batch folded into M (shared B, dense strides)
    int                  b_copies       = 1;
    bool                 prepared       = false;
    // staging for the host-buffer entry point
    void    *d_a_stage = nullptr, *d_dst_stage = nullptr;
    int32_t *d_bias_stage = nullptr;
    // cugl_gemmlowp_run_host pipelines row blocks over three streams: copies in, GEMM (the context's stream),
    // copies out
    cudaStream_t             s_in = nullptr, s_out = nullptr;
    int                      host_blocks = 0; // row blocks of the host-buffer pipeline, 0 = default
    std::vector<cudaEvent_t> ev_in, ev_done;
};

namespace
{
constexpr int kHostPipelineBlocks    = 8;  // default number of row blocks of the host-buffer pipeline
constexpr int kMaxHostPipelineBlocks = 32;

void apply_quant_fields(cugl_gemm_plan *p, const cugl_gemm_desc *d)
{
    GemmCore &c     = p->core;
    c.a_off         = d->a_offset;
    c.b_off         = d->b_offset;
    c.stage         = d->stage;
    c.per_channel   = d->stage != CUGL_STAGE_NONE && d->is_quantized_per_channel != 0;
    c.mult          = d->gemmlowp_multiplier;
    c.shift         = d->gemmlowp_shift;
    c.result_offset = d->gemmlowp_offset;
    c.min_bound     = d->gemmlowp_min_bound;
    c.max_bound     = d->gemmlowp_max_bound;
    c.accumulate    = d->accumulate != 0;
    c.dq_scale      = d->dequantize_scale;
}

cugl_status relayout_b(cugl_gemm_plan *p, const void *d_b)
{
    const cugl_gemm_desc &d = p->desc;
    for (int i = 0; i < p->b_copies; ++i)
    {
        const uint8_t *src = static_cast<const uint8_t *>(d_b) + static_cast<int64_t>(i) * d.b_batch_stride;
        CUGL_TRY(launch_transpose_colsum(p->ctx, src, p->core.b_signed, d.K, d.N, d.ldb,
                                         p->core.d_bt + static_cast<size_t>(i) * p->core.ldbt * d.N, p->core.ldbt,
                                         p->core.d_colsum + static_cast<size_t>(i) * d.N));
    }
    return CUGL_SUCCESS;
}
} // namespace

extern "C"
{
    cugl_status cugl_gemmlowp_validate(const cugl_gemm_desc *desc, const char **reason)
    {
        cugl_status code;
        const char *why = validate_gemm(desc, &code);
        if (reason != nullptr)
        {
            *reason = why != nullptr ? why : "";
        }
        if (why != nullptr)
        {
            set_global_error(std::string("cugl_gemmlowp_validate: ") + why);
        }
        return code;
    }

    cugl_status cugl_gemmlowp_plan_create(cugl_context *ctx, const cugl_gemm_desc *desc, cugl_gemm_plan **out)
    {
        if (ctx == nullptr || out == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_create: NULL argument");
        }
        *out = nullptr;
        cugl_status code;
        const char *why = validate_gemm(desc, &code);
        if (why != nullptr)
        {
            return fail(ctx, code, std::string("cugl_gemmlowp_plan_create: ") + why);
        }
        auto *p = new cugl_gemm_plan();
        p->ctx  = ctx;
        p->desc = *desc;
        if (desc->stage != CUGL_STAGE_NONE && desc->is_quantized_per_channel)
        {
            p->h_mults.assign(desc->h_gemmlowp_multipliers, desc->h_gemmlowp_multipliers + desc->N);
            p->h_shifts.assign(desc->h_gemmlowp_shifts, desc->h_gemmlowp_shifts + desc->N);
        }
        p->desc.h_gemmlowp_multipliers = nullptr;
        p->desc.h_gemmlowp_shifts      = nullptr;
        p->collapse_batch = desc->batch > 1 && desc->b_batch_stride == 0 &&
                            desc->a_batch_stride == static_cast<int64_t>(desc->M) * desc->lda &&
                            desc->d_batch_stride == static_cast<int64_t>(desc->M) * desc->ldd;
        p->b_copies = (desc->batch > 1 && desc->b_batch_stride != 0) ? desc->batch : 1;
        GemmCore &c = p->core;
        c.ctx       = ctx;
        c.M         = desc->M;
        c.N         = desc->N;
        c.K         = desc->K;
        c.a_signed  = desc->a_dtype == CUGL_S8;
        c.b_signed  = desc->b_dtype == CUGL_S8;
        c.dst_dtype = desc->dst_dtype;
        apply_quant_fields(p, desc);
        c.lda_hint   = desc->lda;
        c.tmp_a_rows = p->collapse_batch ? desc->M * desc->batch : desc->M;
        cugl_status s = c.alloc(p->b_copies, desc->M * desc->batch);
        if (s == CUGL_SUCCESS)
        {
            s = c.upload_stage_vectors(p->h_mults.data(), p->h_shifts.data());
        }
        if (s != CUGL_SUCCESS)
        {
            cugl_gemmlowp_plan_destroy(p);
            return s;
        }
        *out = p;
        return CUGL_SUCCESS;
    }

    void cugl_gemmlowp_plan_destroy(cugl_gemm_plan *plan)
    {
        if (plan == nullptr)
        {
            return;
        }
        cudaStreamSynchronize(plan->ctx->stream);
        plan->core.release();
        cugl_free(plan->ctx, plan->d_a_stage);
        cugl_free(plan->ctx, plan->d_dst_stage);
        cugl_free(plan->ctx, plan->d_bias_stage);
        for (cudaEvent_t e : plan->ev_in) cudaEventDestroy(e);
        for (cudaEvent_t e : plan->ev_done) cudaEventDestroy(e);
        if (plan->s_in != nullptr) cudaStreamDestroy(plan->s_in);
        if (plan->s_out != nullptr) cudaStreamDestroy(plan->s_out);
        delete plan;
    }

    cugl_status cugl_gemmlowp_prepare(cugl_gemm_plan *plan, const void *d_b)
    {
        if (plan == nullptr || d_b == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_prepare: NULL argument");
        }
        CUGL_TRY(relayout_b(plan, d_b));
        plan->prepared = true;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_run(cugl_gemm_plan *plan, const void *d_a, const void *d_b, const int32_t *d_bias,
                                  void *d_dst)
    {
        if (plan == nullptr || d_a == nullptr || d_dst == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run: NULL argument");
        }
        const cugl_gemm_desc &d = plan->desc;
        if (d.has_bias && d_bias == nullptr)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run: plan was configured with a bias");
        }
        if (!plan->prepared || !d.reshape_b_only_on_first_run)
        {
            if (d_b == nullptr)
            {
                return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                            "cugl_gemmlowp_run: B is required (not prepared, or B is not constant)");
            }
            CUGL_TRY(relayout_b(plan, d_b));
            plan->prepared = true;
        }
        const int32_t *bias = d.has_bias ? d_bias : nullptr;
        if (plan->collapse_batch || d.batch == 1)
        {
            return plan->core.gemm(d_a, d.lda, d.M * d.batch, d_dst, d.ldd, bias, 0, 0);
        }
        for (int i = 0; i < d.batch; ++i)
        {
            CUGL_TRY(plan->core.gemm(static_cast<const uint8_t *>(d_a) + i * d.a_batch_stride, d.lda, d.M,
                                     static_cast<uint8_t *>(d_dst) + i * d.d_batch_stride, d.ldd, bias,
                                     plan->b_copies > 1 ? i : 0, i * d.M));
        }
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_run_multi(cugl_gemm_plan *plan, const void *d_a, const int32_t *d_bias,
                                        void *const *d_dsts, int32_t n_dsts)
    {
        if (plan == nullptr || d_a == nullptr || d_dsts == nullptr || n_dsts < 1 || n_dsts > 8)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_multi: bad argument");
        }
        const cugl_gemm_desc &d = plan->desc;
        if (!plan->prepared || d.batch != 1)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_multi: needs a prepared plan with batch 1");
        }
        for (int i = 0; i < n_dsts; ++i)
        {
            if (d_dsts[i] == nullptr)
            {
                return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_multi: NULL destination");
            }
        }
        if (d.has_bias && d_bias == nullptr)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_multi: plan was configured with a bias");
        }
        return plan->core.gemm(d_a, d.lda, d.M, d_dsts[0], d.ldd, d.has_bias ? d_bias : nullptr, 0, 0, d_dsts + 1,
                               n_dsts - 1);
    }

    cugl_status cugl_gemmlowp_run_host(cugl_gemm_plan *plan, const void *h_a, const int32_t *h_bias, void *h_dst)
    {
        if (plan == nullptr || h_a == nullptr || h_dst == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_host: NULL argument");
        }
        const cugl_gemm_desc &d   = plan->desc;
        cugl_context         *ctx = plan->ctx;
        if (!plan->prepared)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_host: call cugl_gemmlowp_prepare first");
        }
        const size_t a_bytes =
            d.batch > 1 ? static_cast<size_t>(d.a_batch_stride) * d.batch : static_cast<size_t>(d.lda) * d.M;
        const size_t d_bytes =
            d.batch > 1 ? static_cast<size_t>(d.d_batch_stride) * d.batch : static_cast<size_t>(d.ldd) * d.M;
        // each buffer on its own: a failed allocation must not leave the plan believing that all three exist
        if (plan->d_a_stage == nullptr) CUGL_TRY(cugl_malloc(ctx, a_bytes, &plan->d_a_stage));
        if (plan->d_dst_stage == nullptr) CUGL_TRY(cugl_malloc(ctx, d_bytes, &plan->d_dst_stage));
        if (plan->d_bias_stage == nullptr)
        {
            CUGL_TRY(cugl_malloc(ctx, sizeof(int32_t) * d.N, reinterpret_cast<void **>(&plan->d_bias_stage)));
        }
        if (d.has_bias && h_bias == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_host: plan was configured with a bias");
        }
        // Large single-batch products run as a pipeline over row blocks: block i+1 travels to the device while
        // block i is multiplied and block i-1 travels back (PCIe is full duplex), so the call costs about the
        // longer of the two copies instead of copy + GEMM + copy.  Pinned host buffers are needed for the overlap;
        // pageable ones still work, serialised by the driver.
        // Row blocks of the pipeline.  The call costs about (first block in) + (all blocks out) or (all blocks in) +
        // (last block out), whichever is longer, and large copies run nearer the link rate than small ones: so the
        // default schedule is tapered -- 1/16, 1/8, 1/4, 1/4, 1/8, 1/8, 1/16 of the rows -- small blocks at both ends,
        // large ones in the middle.  Measured on 4096 x 4096 x 4096 (16.8 MB each way, 55 GB/s per direction alone):
        // 0.68 ms unpipelined, 0.61 ms with eight equal blocks, 0.55 ms with three equal blocks or this schedule;
        // copies in both directions with no dependency between them take 0.39 ms.
        std::vector<int> block_rows;
        if (d.batch == 1 && d.M >= 2048)
        {
            if (plan->host_blocks > 0)
            {
                const int rows_per = static_cast<int>(round_up((d.M + plan->host_blocks - 1) / plan->host_blocks, 256));
                for (int r0 = 0; r0 < d.M; r0 += rows_per) block_rows.push_back(d.M - r0 < rows_per ? d.M - r0 : rows_per);
            }
            else
            {
                static const int sixteenths[] = {1, 2, 4, 4, 2, 2, 1};
                int              r0          = 0;
                for (int f : sixteenths)
                {
                    int rows = static_cast<int>(round_up(static_cast<int64_t>(d.M) * f / 16, 256));
                    rows     = d.M - r0 < rows ? d.M - r0 : rows;
                    if (rows > 0) block_rows.push_back(rows);
                    r0 += rows;
                }
                if (r0 < d.M) block_rows.push_back(d.M - r0);
            }
        }
        if (block_rows.size() > 1)
        {
            if (plan->s_in == nullptr)
            {
                CUGL_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&plan->s_in, cudaStreamNonBlocking));
                CUGL_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&plan->s_out, cudaStreamNonBlocking));
                plan->ev_in.resize(kMaxHostPipelineBlocks + 1);
                plan->ev_done.resize(kMaxHostPipelineBlocks + 1);
                for (cudaEvent_t &e : plan->ev_in) CUGL_CUDA_TRY(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
                for (cudaEvent_t &e : plan->ev_done) CUGL_CUDA_TRY(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            }
            const int      n_blocks = static_cast<int>(block_rows.size());
            const uint8_t *ha       = static_cast<const uint8_t *>(h_a);
            uint8_t       *da       = static_cast<uint8_t *>(plan->d_a_stage);
            uint8_t       *dd       = static_cast<uint8_t *>(plan->d_dst_stage);
            uint8_t       *hd       = static_cast<uint8_t *>(h_dst);
            // the staging buffers are free: every earlier call ended with a synchronisation of all three streams
            if (d.has_bias)
            {
                CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(plan->d_bias_stage, h_bias, sizeof(int32_t) * d.N, cudaMemcpyHostToDevice,
                                                   plan->s_in));
            }
            for (int i = 0, r0 = 0; i < n_blocks; r0 += block_rows[i], ++i)
            {
                const size_t rows = static_cast<size_t>(block_rows[i]);
                CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(da + static_cast<size_t>(r0) * d.lda, ha + static_cast<size_t>(r0) * d.lda,
                                                   rows * d.lda, cudaMemcpyHostToDevice, plan->s_in));
                CUGL_CUDA_TRY(ctx, cudaEventRecord(plan->ev_in[i], plan->s_in));
            }
            for (int i = 0, r0 = 0; i < n_blocks; r0 += block_rows[i], ++i)
            {
                const int rows = block_rows[i];
                CUGL_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, plan->ev_in[i], 0));
                CUGL_TRY(plan->core.gemm(da + static_cast<size_t>(r0) * d.lda, d.lda, rows, dd + static_cast<size_t>(r0) * d.ldd,
                                         d.ldd, d.has_bias ? plan->d_bias_stage : nullptr, 0, r0));
                CUGL_CUDA_TRY(ctx, cudaEventRecord(plan->ev_done[i], ctx->stream));
                CUGL_CUDA_TRY(ctx, cudaStreamWaitEvent(plan->s_out, plan->ev_done[i], 0));
                CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(hd + static_cast<size_t>(r0) * d.ldd, dd + static_cast<size_t>(r0) * d.ldd,
                                                   static_cast<size_t>(rows) * d.ldd, cudaMemcpyDeviceToHost, plan->s_out));
            }
            CUGL_CUDA_TRY(ctx, cudaStreamSynchronize(plan->s_out));
            CUGL_CUDA_TRY(ctx, cudaStreamSynchronize(plan->s_in));
            return cugl_sync(ctx);
        }
        CUGL_TRY(cugl_memcpy_h2d(ctx, plan->d_a_stage, h_a, a_bytes));
        if (d.has_bias)
        {
            CUGL_TRY(cugl_memcpy_h2d(ctx, plan->d_bias_stage, h_bias, sizeof(int32_t) * d.N));
        }
        CUGL_TRY(cugl_gemmlowp_run(plan, plan->d_a_stage, nullptr, plan->d_bias_stage, plan->d_dst_stage));
        CUGL_TRY(cugl_memcpy_d2h(ctx, h_dst, plan->d_dst_stage, d_bytes));
        return cugl_sync(ctx);
    }

    cugl_status cugl_gemmlowp_update_quantization(cugl_gemm_plan *plan, const cugl_gemm_desc *desc)
    {
        if (plan == nullptr || desc == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT,
                        "cugl_gemmlowp_update_quantization: NULL argument");
        }
        const cugl_gemm_desc &o = plan->desc;
        if (desc->M != o.M || desc->N != o.N || desc->K != o.K || desc->batch != o.batch ||
            desc->a_dtype != o.a_dtype || desc->b_dtype != o.b_dtype || desc->dst_dtype != o.dst_dtype ||
            desc->stage != o.stage || desc->is_quantized_per_channel != o.is_quantized_per_channel)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                        "cugl_gemmlowp_update_quantization: shapes, types and stage kind must not change");
        }
        cugl_status code;
        const char *why = validate_gemm(desc, &code);
        if (why != nullptr)
        {
            return fail(plan->ctx, code, std::string("cugl_gemmlowp_update_quantization: ") + why);
        }
        plan->desc.a_offset            = desc->a_offset;
        plan->desc.b_offset            = desc->b_offset;
        plan->desc.gemmlowp_multiplier = desc->gemmlowp_multiplier;
        plan->desc.gemmlowp_shift      = desc->gemmlowp_shift;
        plan->desc.gemmlowp_offset     = desc->gemmlowp_offset;
        plan->desc.gemmlowp_min_bound  = desc->gemmlowp_min_bound;
        plan->desc.gemmlowp_max_bound  = desc->gemmlowp_max_bound;
        plan->desc.dequantize_scale    = desc->dequantize_scale;
        apply_quant_fields(plan, &plan->desc);
        if (plan->core.per_channel)
        {
            plan->h_mults.assign(desc->h_gemmlowp_multipliers, desc->h_gemmlowp_multipliers + desc->N);
            plan->h_shifts.assign(desc->h_gemmlowp_shifts, desc->h_gemmlowp_shifts + desc->N);
        }
        CUGL_TRY(plan->core.upload_stage_vectors(plan->h_mults.data(), plan->h_shifts.data()));
        return CUGL_SUCCESS;
    }

    const char *cugl_gemmlowp_plan_kernel(const cugl_gemm_plan *plan)
    {
        if (plan == nullptr)
        {
            return "";
        }
        // the decision also depends on the alignment of A, only known at run(): assume an aligned base
        GemmOperands op{};
        op.a    = reinterpret_cast<const void *>(uintptr_t(256));
        op.bt   = plan->core.d_bt;
        op.lda  = round_up(plan->desc.lda, 16); // an unaligned pitch runs on a 16-byte-pitch copy of A
        op.ldbt = plan->core.ldbt;
        op.M    = plan->desc.M;
        op.N    = plan->desc.N;
        op.K    = plan->desc.K;
        if (!plan->core.uses_tcgen05(op))
        {
            return "simt";
        }
        op.M         = plan->collapse_batch ? plan->desc.M * plan->desc.batch : plan->desc.M;
        op.epi_warps = plan->core.epi_warps;
        op.block_n   = plan->core.block_n;
        return (plan->core.allow_pair && gemmlowp_tcgen05_uses_pair(plan->ctx, op)) ? "tcgen05_2cta" : "tcgen05";
    }

    cugl_status cugl_gemmlowp_plan_set_epilogue_warps(cugl_gemm_plan *plan, int warps)
    {
        if (plan == nullptr || (warps != 0 && warps != 4 && warps != 8 && warps != 16))
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT,
                        "cugl_gemmlowp_plan_set_epilogue_warps: plan is NULL or warps is not 0, 4, 8 or 16");
        }
        plan->core.epi_warps = warps;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_set_tile_columns(cugl_gemm_plan *plan, int columns)
    {
        if (plan == nullptr || (columns != 0 && columns != 64 && columns != 128 && columns != 256))
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT,
                        "cugl_gemmlowp_plan_set_tile_columns: plan is NULL or columns is not 0, 64, 128 or 256");
        }
        plan->core.block_n = columns;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_set_paired_drain(cugl_gemm_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_set_paired_drain: NULL plan");
        }
        plan->core.pair_drain = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_set_tma_store(cugl_gemm_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_set_tma_store: NULL plan");
        }
        plan->core.tma_store = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_force_simt(cugl_gemm_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_force_simt: NULL plan");
        }
        plan->core.force_simt = on != 0;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_allow_pair_kernel(cugl_gemm_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_allow_pair_kernel: NULL plan");
        }
        plan->core.allow_pair = on != 0;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_set_host_pipeline(cugl_gemm_plan *plan, int blocks)
    {
        if (plan == nullptr || blocks < 0 || blocks > kMaxHostPipelineBlocks)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT,
                        "cugl_gemmlowp_plan_set_host_pipeline: NULL plan or more than 32 blocks");
        }
        plan->host_blocks = blocks;
        return CUGL_SUCCESS;
    }

    int cugl_gemmlowp_plan_launches(const cugl_gemm_plan *plan)
    {
        if (plan == nullptr)
        {
            return 0;
        }
        const cugl_gemm_desc &d       = plan->desc;
        const int             n_gemms = (plan->collapse_batch || d.batch == 1) ? 1 : d.batch;
        int                   n       = n_gemms * (1 + (plan->core.b_off != 0 ? 1 : 0));
        if (!d.reshape_b_only_on_first_run)
        {
            n += plan->b_copies;
        }
        return n;
    }

    // ---- stand-alone kernels ---------------------------------------------------------------------
    cugl_status cugl_reduce_rows(cugl_context *ctx, const void *d_a, int32_t dtype, int32_t M, int32_t K, int64_t lda,
                                 int32_t scalar, int32_t *d_out)
    {
        if (ctx == nullptr || d_a == nullptr || d_out == nullptr || !is_q8(dtype) || M < 0 || K < 0 || lda < K)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_reduce_rows: bad argument");
        }
        return launch_reduce_rows(ctx, d_a, dtype == CUGL_S8, M, K, lda, scalar, d_out);
    }

    cugl_status cugl_reduce_cols(cugl_context *ctx, const void *d_b, int32_t dtype, int32_t K, int32_t N, int64_t ldb,
                                 int32_t scalar, int32_t *d_out)
    {
        if (ctx == nullptr || d_b == nullptr || d_out == nullptr || !is_q8(dtype) || N < 0 || K < 0 || ldb < N)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_reduce_cols: bad argument");
        }
        return launch_reduce_cols(ctx, d_b, dtype == CUGL_S8, K, N, ldb, scalar, d_out);
    }

    cugl_status cugl_offset_contribution(cugl_context *ctx, int32_t *d_mm, int32_t M, int32_t N, int32_t K,
                                         int64_t ld_bytes, const int32_t *d_colsum, const int32_t *d_rowsum,
                                         int32_t a_offset, int32_t b_offset)
    {
        if (ctx == nullptr || d_mm == nullptr || M < 0 || N < 0 || ld_bytes < 4ll * N || (ld_bytes & 3) != 0 ||
            (a_offset != 0 && d_colsum == nullptr) || (b_offset != 0 && d_rowsum == nullptr))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_offset_contribution: bad argument");
        }
        return launch_offset_contribution(ctx, d_mm, M, N, K, ld_bytes, d_colsum, d_rowsum, a_offset, b_offset);
    }

    cugl_status cugl_output_stage(cugl_context *ctx, const int32_t *d_in, int64_t ld_in_bytes, const int32_t *d_bias,
                                  void *d_out, int64_t ld_out_bytes, int32_t out_dtype, int32_t M, int32_t N,
                                  const int32_t *d_multipliers, const int32_t *d_shifts, int32_t multiplier,
                                  int32_t shift, int32_t n_mult, int32_t result_offset, int32_t min_bound,
                                  int32_t max_bound)
    {
        const bool out16 = out_dtype == CUGL_S16; // QSYMM16 (CpuGemmLowpQuantizeDownInt32ToInt16ScaleByFixedPointKernel)
        if (ctx == nullptr || d_in == nullptr || d_out == nullptr || !(is_q8(out_dtype) || out16) || M < 0 || N < 0 ||
            ld_in_bytes < 4ll * N || (ld_in_bytes & 3) != 0 || ld_out_bytes < (out16 ? 2ll : 1ll) * N ||
            (out16 && (((reinterpret_cast<uintptr_t>(d_out) | static_cast<uint64_t>(ld_out_bytes)) & 1) != 0)))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage: bad argument");
        }
        if (min_bound > max_bound)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage: min_bound > max_bound");
        }
        const bool pc = n_mult > 1;
        if (pc && (n_mult != N || d_multipliers == nullptr || d_shifts == nullptr))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage: per-channel needs N multipliers and shifts");
        }
        const int32_t tlo = out16 ? -32768 : (out_dtype == CUGL_S8 ? -128 : 0);
        const int32_t thi = out16 ? 32767 : (out_dtype == CUGL_S8 ? 127 : 255);
        return launch_output_stage(ctx, d_in, ld_in_bytes, d_bias, d_out, ld_out_bytes, M, N,
                                   pc ? d_multipliers : nullptr, pc ? d_shifts : nullptr, multiplier, shift,
                                   result_offset, min_bound > tlo ? min_bound : tlo, max_bound < thi ? max_bound : thi,
                                   false, out16);
    }

    cugl_status cugl_output_stage_quantize_down(cugl_context *ctx, const int32_t *d_in, int64_t ld_in_bytes, const int32_t *d_bias,
                                  void *d_out, int64_t ld_out_bytes, int32_t out_dtype, int32_t M, int32_t N,
                                  const int32_t *d_multipliers, const int32_t *d_shifts, int32_t multiplier,
                                  int32_t shift, int32_t n_mult, int32_t result_offset, int32_t min_bound,
                                  int32_t max_bound)
    {
        if (ctx == nullptr || d_in == nullptr || d_out == nullptr || !is_q8(out_dtype) || M < 0 || N < 0 ||
            ld_in_bytes < 4ll * N || (ld_in_bytes & 3) != 0 || ld_out_bytes < N)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage_quantize_down: bad argument");
        }
        if (min_bound > max_bound)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage_quantize_down: min_bound > max_bound");
        }
        const bool pc = n_mult > 1;
        if (pc && (n_mult != N || d_multipliers == nullptr || d_shifts == nullptr))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage_quantize_down: per-channel needs N multipliers and shifts");
        }
        const int32_t tlo = out_dtype == CUGL_S8 ? -128 : 0, thi = out_dtype == CUGL_S8 ? 127 : 255;
        if (!pc && (shift < 0 || shift > 31))
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_output_stage_quantize_down: shift must lie in [0, 31]");
        }
        const bool bounded = min_bound != max_bound; // equal bounds: type range only (GEMMLowp.cpp:93-97)
        return launch_output_stage(ctx, d_in, ld_in_bytes, d_bias, d_out, ld_out_bytes, M, N,
                                   pc ? d_multipliers : nullptr, pc ? d_shifts : nullptr, multiplier, shift,
                                   result_offset, bounded && min_bound > tlo ? min_bound : tlo,
                                   bounded && max_bound < thi ? max_bound : thi, true);
    }

    cugl_status cugl_im2col_nhwc(cugl_context *ctx, const void *d_src, void *d_dst, int32_t C, int32_t W, int32_t H,
                                 int32_t B, int32_t kw, int32_t kh, int32_t stride_x, int32_t stride_y,
                                 int32_t pad_left, int32_t pad_top, int32_t dil_x, int32_t dil_y, int32_t Wo,
                                 int32_t Ho, int32_t pad_value, int64_t row_stride)
    {
        if (ctx == nullptr || d_src == nullptr || d_dst == nullptr || C < 1 || W < 1 || H < 1 || B < 1 || kw < 1 ||
            kh < 1 || stride_x < 1 || stride_y < 1 || dil_x < 1 || dil_y < 1 || Wo < 1 || Ho < 1 ||
            row_stride < static_cast<int64_t>(kh) * kw * C)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_im2col_nhwc: bad argument");
        }
        return launch_im2col_nhwc(ctx, d_src, d_dst, C, W, H, B, kw, kh, stride_x, stride_y, pad_left, pad_top, dil_x,
                                  dil_y, Wo, Ho, pad_value, row_stride);
    }

    cugl_status cugl_weights_reshape_nhwc(cugl_context *ctx, const void *d_w, void *d_dst, int32_t K, int32_t OFM)
    {
        if (ctx == nullptr || d_w == nullptr || d_dst == nullptr || K < 1 || OFM < 1)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_weights_reshape_nhwc: bad argument");
        }
        return launch_transpose_bytes(ctx, d_w, OFM, K, d_dst);
    }
}

// ---------------------------------------------------------------------------------------------------
// Convolution plan
// ---------------------------------------------------------------------------------------------------
struct cugl_conv_plan
{
    cugl_context        *ctx = nullptr;
    cugl_conv_desc       desc{};
    std::vector<int32_t> h_mults, h_shifts;
    GemmCore             core;
    int                  Wo = 0, Ho = 0;
    int64_t              M = 0, K = 0, Kp = 0;
    bool                 skip_im2col = false;
    bool                 implicit    = false;   // gather the patches inside the GEMM kernel, no im2col matrix
    bool                 allow_implicit = true;
    int                  allow_tma_im2col = 1; // implicit lowering, im2col-mode TMA loads: 0 never, 1 where they are exact and
                                               // measured at least level with the gather (128-channel blocks), 2 wherever exact (64 channels too)
    uint8_t             *d_cols      = nullptr; // [M][Kp] im2col matrix (allocated on first explicit run)
    uint8_t             *d_pad       = nullptr; // kConvPadBytes of the input zero point: source of out-of-image taps
    // Geometry the lowerings work on: the descriptor's own, or -- stride 2 with at most four channels -- the
    // 2x2 space-to-depth form (16 channels, stride 1, zero weights where the original kernel has no tap).
    bool     fold = false;
    int      eC = 0, eW = 0, eH = 0, ekw = 0, ekh = 0, esx = 1, esy = 1, epl = 0, ept = 0;
    int      fold_oy = 0, fold_ox = 0;
    uint8_t *d_fold = nullptr; // [B][eH][eW][16]; plan-owned, allocated on first use unless a workspace is bound
    // temporary workspace handed in by the caller (cugl_conv2d_plan_bind_temp): row sums | folded input | im2col matrix
    uint8_t *d_temp = nullptr;
    size_t   temp_bound_bytes = 0;

    size_t fold_bytes() const
    {
        return fold ? static_cast<size_t>(round_up(static_cast<int64_t>(desc.B) * eH * eW * 16, 256)) : 0;
    }
    bool explicit_lowering() const
    {
        return !skip_im2col && !(implicit && allow_implicit && !core.force_simt);
    }
    size_t cols_bytes() const
    {
        return explicit_lowering() ? static_cast<size_t>(round_up(M * Kp, 256)) : 0;
    }
    size_t temp_bytes() const
    {
        return core.rowsum_bytes() + fold_bytes() + cols_bytes();
    }
    // fused residual addition (cugl_conv2d_plan_set_residual): clamp bounds of the saturating form
    bool residual_set = false;
    int  res_floor = 0, res_cap = 255;
    bool                 prepared    = false;
    void                *d_src_stage = nullptr, *d_dst_stage = nullptr;
    int32_t             *d_bias_stage = nullptr;
};

namespace
{
void conv_out_dims(const cugl_conv_desc *d, int *Wo, int *Ho)
{
    // scaled_dimensions with DimensionRoundingType::FLOOR (src/core/Utils.cpp)
    const int kw_eff = d->dil_x * (d->kw - 1) + 1;
    const int kh_eff = d->dil_y * (d->kh - 1) + 1;
    *Wo              = (d->W + d->pad_left + d->pad_right - kw_eff) / d->stride_x + 1;
    *Ho              = (d->H + d->pad_top + d->pad_bottom - kh_eff) / d->stride_y + 1;
}

const char *validate_conv(const cugl_conv_desc *d, cugl_status *code)
{
    *code = CUGL_INVALID_ARGUMENT;
    if (d == nullptr) return "descriptor is NULL";
    if (d->B < 1 || d->H < 1 || d->W < 1 || d->C < 1 || d->OFM < 1 || d->kh < 1 || d->kw < 1)
        return "tensor dimensions must be positive";
    if (d->stride_x < 1 || d->stride_y < 1 || d->dil_x < 1 || d->dil_y < 1) return "stride and dilation must be >= 1";
    if (d->pad_left < 0 || d->pad_right < 0 || d->pad_top < 0 || d->pad_bottom < 0) return "negative padding";
    if (!is_q8(d->src_dtype) || !is_q8(d->w_dtype)) return "input and weights must be 8-bit quantized";
    if (d->src_dtype == CUGL_S8 && d->w_dtype == CUGL_U8)
        return "QASYMM8 weights with a QASYMM8_SIGNED input are not supported";
    if (d->min_bound > d->max_bound) return "min_bound > max_bound";
    if (d->is_quantized_per_channel)
    {
        if (d->h_gemmlowp_multipliers == nullptr || d->h_gemmlowp_shifts == nullptr)
            return "per-channel weights need OFM multipliers and shifts";
        if (d->w_zero_point != 0) return "QSYMM8_PER_CHANNEL weights are symmetric: w_zero_point must be 0";
    }
    int Wo, Ho;
    conv_out_dims(d, &Wo, &Ho);
    if (Wo < 1 || Ho < 1) return "kernel larger than the padded input";
    if (static_cast<int64_t>(d->B) * Ho * Wo > INT32_MAX) return "too many output pixels";
    *code = CUGL_SUCCESS;
    return nullptr;
}
} // namespace

extern "C"
{
    void cugl_conv2d_out_dims(const cugl_conv_desc *desc, int32_t *Wo, int32_t *Ho)
    {
        int w = 0, h = 0;
        if (desc != nullptr)
        {
            conv_out_dims(desc, &w, &h);
        }
        if (Wo != nullptr) *Wo = w;
        if (Ho != nullptr) *Ho = h;
    }

    cugl_status cugl_conv2d_validate(const cugl_conv_desc *desc, const char **reason)
    {
        cugl_status code;
        const char *why = validate_conv(desc, &code);
        if (reason != nullptr)
        {
            *reason = why != nullptr ? why : "";
        }
        if (why != nullptr)
        {
            set_global_error(std::string("cugl_conv2d_validate: ") + why);
        }
        return code;
    }

    cugl_status cugl_conv2d_plan_create(cugl_context *ctx, const cugl_conv_desc *desc, cugl_conv_plan **out)
    {
        if (ctx == nullptr || out == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_create: NULL argument");
        }
        *out = nullptr;
        cugl_status code;
        const char *why = validate_conv(desc, &code);
        if (why != nullptr)
        {
            return fail(ctx, code, std::string("cugl_conv2d_plan_create: ") + why);
        }
        auto *p = new cugl_conv_plan();
        p->ctx  = ctx;
        p->desc = *desc;
        if (desc->is_quantized_per_channel)
        {
            p->h_mults.assign(desc->h_gemmlowp_multipliers, desc->h_gemmlowp_multipliers + desc->OFM);
            p->h_shifts.assign(desc->h_gemmlowp_shifts, desc->h_gemmlowp_shifts + desc->OFM);
        }
        p->desc.h_gemmlowp_multipliers = nullptr;
        p->desc.h_gemmlowp_shifts      = nullptr;
        conv_out_dims(desc, &p->Wo, &p->Ho);
        p->eC = desc->C, p->eW = desc->W, p->eH = desc->H, p->ekw = desc->kw, p->ekh = desc->kh;
        p->esx = desc->stride_x, p->esy = desc->stride_y, p->epl = desc->pad_left, p->ept = desc->pad_top;
        p->fold = desc->C <= 4 && desc->stride_x == 2 && desc->stride_y == 2 && desc->dil_x == 1 && desc->dil_y == 1 &&
                  desc->w_zero_point == 0 && desc->kw * desc->kh > 1;
        if (p->fold)
        {
            p->fold_ox = desc->pad_left & 1, p->fold_oy = desc->pad_top & 1;
            p->eC = 16, p->eW = (desc->W + 1) / 2, p->eH = (desc->H + 1) / 2;
            p->ekw = (p->fold_ox + desc->kw + 1) / 2, p->ekh = (p->fold_oy + desc->kh + 1) / 2;
            p->esx = p->esy = 1;
            p->epl = (desc->pad_left + p->fold_ox) / 2, p->ept = (desc->pad_top + p->fold_oy) / 2;
        }
        p->M  = static_cast<int64_t>(desc->B) * p->Ho * p->Wo;
        p->K  = static_cast<int64_t>(p->ekh) * p->ekw * p->eC;
        p->Kp = round_up(p->K, 16);
        // CpuGemmConv2d.cpp:189-191: a 1x1, stride-1, unpadded NHWC convolution is a plain GEMM on the
        // input tensor.  Kept only when the rows are already 16-byte multiples (TMA stride rule).
        p->skip_im2col = desc->kw == 1 && desc->kh == 1 && desc->stride_x == 1 && desc->stride_y == 1 &&
                         desc->pad_left == 0 && desc->pad_right == 0 && desc->pad_top == 0 &&
                         desc->pad_bottom == 0 && (desc->C % 16) == 0;
        GemmCore &c     = p->core;
        c.ctx           = ctx;
        c.M             = static_cast<int>(p->M);
        c.N             = desc->OFM;
        c.K             = static_cast<int>(p->K);
        c.a_signed      = desc->src_dtype == CUGL_S8;
        c.b_signed      = desc->w_dtype == CUGL_S8;
        c.dst_dtype     = desc->src_dtype;
        c.a_off         = -desc->src_zero_point; // CpuGemmConv2d.cpp:266-280: offsets are negated
        c.b_off         = -desc->w_zero_point;
        c.stage         = CUGL_STAGE_QUANTIZE_DOWN_FIXEDPOINT;
        c.per_channel   = desc->is_quantized_per_channel != 0;
        c.mult          = desc->gemmlowp_multiplier;
        c.shift         = desc->gemmlowp_shift;
        c.result_offset = desc->dst_zero_point;
        c.min_bound     = desc->min_bound;
        c.max_bound     = desc->max_bound;
        cugl_status s   = c.alloc(1, c.M);
        if (s == CUGL_SUCCESS)
        {
            s = c.upload_stage_vectors(p->h_mults.data(), p->h_shifts.data());
        }
        // Implicit GEMM whenever the gather kernel can address the tensors: channel count a multiple of 16 and
        // symmetric weights (no row-sum term).  Otherwise explicit im2col.
        p->implicit = !p->skip_im2col && (p->eC % 16) == 0 && desc->w_zero_point == 0;
        if (s == CUGL_SUCCESS && p->implicit)
        {
            s = cugl_malloc(ctx, kConvPadBytes, reinterpret_cast<void **>(&p->d_pad));
            if (s == CUGL_SUCCESS)
            {
                s = cugl_memset(ctx, p->d_pad, desc->src_zero_point & 0xff, kConvPadBytes);
            }
        }
        if (s != CUGL_SUCCESS)
        {
            cugl_conv2d_plan_destroy(p);
            return s;
        }
        *out = p;
        return CUGL_SUCCESS;
    }

    void cugl_conv2d_plan_destroy(cugl_conv_plan *plan)
    {
        if (plan == nullptr)
        {
            return;
        }
        cudaStreamSynchronize(plan->ctx->stream);
        plan->core.release();
        cugl_free(plan->ctx, plan->d_cols);
        cugl_free(plan->ctx, plan->d_pad);
        cugl_free(plan->ctx, plan->d_fold);
        cugl_free(plan->ctx, plan->d_src_stage);
        cugl_free(plan->ctx, plan->d_dst_stage);
        cugl_free(plan->ctx, plan->d_bias_stage);
        delete plan;
    }

    cugl_status cugl_conv2d_prepare(cugl_conv_plan *plan, const void *d_weights)
    {
        if (plan == nullptr || d_weights == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_prepare: NULL argument");
        }
        cugl_context *ctx = plan->ctx;
        GemmCore     &c   = plan->core;
        // NHWC weights [OFM][kh][kw][C] are already the K-major operand the tensor cores want: the
        // reshape of CpuWeightsReshapeKernel followed by the pretranspose of the assembly path cancel out.
        // Copy the rows into the zero-padded buffer and reduce each row (= column of the GEMM's B).
        if (plan->fold)
        {
            const cugl_conv_desc &d = plan->desc;
            CUGL_TRY(launch_fold_weights(ctx, d_weights, c.d_bt, c.ldbt, c.N, d.kh, d.kw, d.C, plan->ekh, plan->ekw,
                                         plan->fold_oy, plan->fold_ox));
        }
        else
        {
            CUGL_CUDA_TRY(ctx, cudaMemcpy2DAsync(c.d_bt, c.ldbt, d_weights, plan->K, plan->K, c.N,
                                                 cudaMemcpyDeviceToDevice, ctx->stream));
        }
        CUGL_TRY(launch_reduce_rows(ctx, c.d_bt, c.b_signed, c.N, c.K, c.ldbt, 1, c.d_colsum));
        plan->prepared = true;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_residual(cugl_conv_plan *plan, float conv_out_scale, float residual_scale,
                                              int32_t residual_zero_point, float dst_scale, int32_t dst_zero_point,
                                              int32_t activation, float act_a, float act_b)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_residual: NULL plan");
        }
        if (plan->desc.src_dtype != CUGL_U8)
        {
            return fail(plan->ctx, CUGL_UNSUPPORTED_CONFIG, "fused residual addition needs a QASYMM8 (uint8) output");
        }
        if (!(conv_out_scale > 0.f) || !(residual_scale > 0.f) || !(dst_scale > 0.f) || activation < CUGL_ACT_NONE ||
            activation > CUGL_ACT_LU_BOUNDED_RELU)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_residual: bad scale or activation");
        }
        int lo = 0, hi = 255;
        if (!classify_add(conv_out_scale, plan->desc.dst_zero_point, residual_scale, residual_zero_point, dst_scale,
                          dst_zero_point, activation, act_a, act_b, &lo, &hi))
        {
            return fail(plan->ctx, CUGL_UNSUPPORTED_CONFIG,
                        "this addition is not a saturating byte addition for every input pair: run cugl_add_qasymm8 "
                        "after the convolution instead");
        }
        plan->residual_set = true;
        plan->res_floor    = lo;
        plan->res_cap      = hi;
        return CUGL_SUCCESS;
    }

    static cugl_status conv2d_run_impl(cugl_conv_plan *plan, const void *d_src, const int32_t *d_bias,
                                       const void *d_residual, void *d_dst);

    cugl_status cugl_conv2d_run(cugl_conv_plan *plan, const void *d_src, const int32_t *d_bias, void *d_dst)
    {
        return conv2d_run_impl(plan, d_src, d_bias, nullptr, d_dst);
    }

    cugl_status cugl_conv2d_run_residual(cugl_conv_plan *plan, const void *d_src, const int32_t *d_bias,
                                         const void *d_residual, void *d_dst)
    {
        if (plan == nullptr || d_residual == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_run_residual: NULL argument");
        }
        if (!plan->residual_set)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                        "cugl_conv2d_run_residual: call cugl_conv2d_plan_set_residual first");
        }
        return conv2d_run_impl(plan, d_src, d_bias, d_residual, d_dst);
    }

    static cugl_status conv2d_run_impl(cugl_conv_plan *plan, const void *d_src, const int32_t *d_bias,
                                       const void *d_residual, void *d_dst)
    {
        if (plan == nullptr || d_src == nullptr || d_dst == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_run: NULL argument");
        }
        const cugl_conv_desc &d = plan->desc;
        if (!plan->prepared)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_conv2d_run: call cugl_conv2d_prepare first");
        }
        if (d.has_bias && d_bias == nullptr)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT, "cugl_conv2d_run: plan was configured with a bias");
        }
        const bool bound = plan->d_temp != nullptr;
        if (bound && plan->temp_bound_bytes < plan->temp_bytes())
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                        "cugl_conv2d_run: the bound temporary workspace is smaller than cugl_conv2d_plan_temp_bytes");
        }
        if (plan->fold)
        {
            uint8_t *fold_buf = bound ? plan->d_temp + plan->core.rowsum_bytes() : plan->d_fold;
            if (fold_buf == nullptr)
            {
                CUGL_TRY(cugl_malloc(plan->ctx, plan->fold_bytes(), reinterpret_cast<void **>(&plan->d_fold)));
                fold_buf = plan->d_fold;
            }
            CUGL_TRY(launch_fold_input(plan->ctx, d_src, fold_buf, d.B, d.H, d.W, d.C, plan->eH, plan->eW,
                                       d.src_zero_point));
            d_src = fold_buf;
        }
        if (plan->implicit && plan->allow_implicit && !plan->core.force_simt)
        {
            GemmCore    &c = plan->core;
            GemmOperands op{};
            op.a             = nullptr;
            op.bt            = c.d_bt;
            op.dst           = d_dst;
            op.lda           = 0;
            op.ldbt          = c.ldbt;
            op.ldd           = d.OFM;
            op.M             = static_cast<int>(plan->M);
            op.N             = c.N;
            op.K             = c.K;
            op.a_signed      = c.a_signed;
            op.b_signed      = c.b_signed;
            op.generic_stage = c.generic_stage;
            op.wide_stage    = c.wide_stage;
            op.max_shift     = c.max_shift;
            op.pack_stage    = c.pack_stage;
            op.epi_warps     = c.epi_warps;
            op.channel_major = c.channel_major;
            op.block_n       = c.block_n;
            op.pair_drain    = c.pair_drain;
            op.tma_store     = c.tma_store;
            op.resident_b    = c.resident_b;
            op.double_tile   = c.double_tile;
            op.n_extra_dst   = 0;
            op.residual      = d_residual;
            op.res_floor     = plan->res_floor;
            op.res_cap       = plan->res_cap;
            ConvOperands cv{};
            cv.src    = d_src;
            cv.pad    = plan->d_pad;
            cv.C      = plan->eC;
            cv.W      = plan->eW;
            cv.H      = plan->eH;
            cv.B      = d.B;
            cv.kw     = plan->ekw;
            cv.kh     = plan->ekh;
            cv.sx     = plan->esx;
            cv.sy     = plan->esy;
            cv.pad_l  = plan->epl;
            cv.pad_t  = plan->ept;
            cv.dil_x  = d.dil_x;
            cv.dil_y  = d.dil_y;
            cv.Wo     = plan->Wo;
            cv.Ho     = plan->Ho;
            // Input zero point 0 and whole 128-channel blocks: the TMA unit builds the patch tiles itself (im2col-mode
            // tensor map, out-of-image taps read as zero = the zero point) and the GEMM kernels run unchanged; else
            // the gather kernel, whose out-of-image taps copy any zero point from the pad buffer.
            if (plan->allow_tma_im2col != 0 && d.src_zero_point == 0 && (plan->eC != 64 || plan->allow_tma_im2col > 1))
            {
                GemmOperands ot  = op;
                ot.conv          = &cv;
                ot.channel_major = -1;
                if (gemmlowp_conv_tma_supported(ot))
                {
                    return launch_gemmlowp_tcgen05(plan->ctx, ot, c.epilogue(d.has_bias ? d_bias : nullptr, 0), c.allow_pair);
                }
            }
            if (gemmlowp_conv_tcgen05_supported(op, cv))
            {
                return launch_gemmlowp_conv_tcgen05(plan->ctx, op, c.epilogue(d.has_bias ? d_bias : nullptr, 0), cv);
            }
        }
        const void *a   = d_src;
        int64_t     lda = plan->eC;
        if (!plan->skip_im2col)
        {
            uint8_t *cols = bound ? plan->d_temp + plan->core.rowsum_bytes() + plan->fold_bytes() : plan->d_cols;
            if (cols == nullptr)
            {
                CUGL_TRY(cugl_malloc(plan->ctx, static_cast<size_t>(plan->M) * plan->Kp,
                                     reinterpret_cast<void **>(&plan->d_cols)));
                cols = plan->d_cols;
            }
            CUGL_TRY(launch_im2col_nhwc(plan->ctx, d_src, cols, plan->eC, plan->eW, plan->eH, d.B, plan->ekw,
                                        plan->ekh, plan->esx, plan->esy, plan->epl, plan->ept, d.dil_x, d.dil_y,
                                        plan->Wo, plan->Ho, d.src_zero_point, plan->Kp));
            a   = cols;
            lda = plan->Kp;
        }
        return plan->core.gemm(a, lda, static_cast<int>(plan->M), d_dst, d.OFM, d.has_bias ? d_bias : nullptr, 0, 0,
                               nullptr, 0, d_residual, plan->res_floor, plan->res_cap);
    }

    cugl_status cugl_conv2d_run_host(cugl_conv_plan *plan, const void *h_src, const int32_t *h_bias, void *h_dst)
    {
        if (plan == nullptr || h_src == nullptr || h_dst == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_run_host: NULL argument");
        }
        const cugl_conv_desc &d   = plan->desc;
        cugl_context         *ctx = plan->ctx;
        const size_t src_bytes    = static_cast<size_t>(d.B) * d.H * d.W * d.C;
        const size_t dst_bytes    = static_cast<size_t>(plan->M) * d.OFM;
        if (plan->d_src_stage == nullptr) CUGL_TRY(cugl_malloc(ctx, src_bytes, &plan->d_src_stage));
        if (plan->d_dst_stage == nullptr) CUGL_TRY(cugl_malloc(ctx, dst_bytes, &plan->d_dst_stage));
        if (plan->d_bias_stage == nullptr)
        {
            CUGL_TRY(cugl_malloc(ctx, sizeof(int32_t) * d.OFM, reinterpret_cast<void **>(&plan->d_bias_stage)));
        }
        CUGL_TRY(cugl_memcpy_h2d(ctx, plan->d_src_stage, h_src, src_bytes));
        if (d.has_bias)
        {
            if (h_bias == nullptr)
            {
                return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_conv2d_run_host: plan was configured with a bias");
            }
            CUGL_TRY(cugl_memcpy_h2d(ctx, plan->d_bias_stage, h_bias, sizeof(int32_t) * d.OFM));
        }
        CUGL_TRY(cugl_conv2d_run(plan, plan->d_src_stage, plan->d_bias_stage, plan->d_dst_stage));
        CUGL_TRY(cugl_memcpy_d2h(ctx, h_dst, plan->d_dst_stage, dst_bytes));
        return cugl_sync(ctx);
    }

    cugl_status cugl_conv2d_plan_allow_implicit(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_allow_implicit: NULL plan");
        }
        plan->allow_implicit = on != 0;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_set_tail_split(cugl_gemm_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_set_tail_split: NULL plan");
        }
        plan->core.split_tail = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_gemmlowp_plan_set_channel_major(cugl_gemm_plan *plan, int mode)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_set_channel_major: NULL plan");
        }
        plan->core.channel_major = mode;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_channel_major(cugl_conv_plan *plan, int mode)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_channel_major: NULL plan");
        }
        plan->core.channel_major = mode;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_epilogue_warps(cugl_conv_plan *plan, int warps)
    {
        if (plan == nullptr || (warps != 0 && warps != 4 && warps != 8 && warps != 16))
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT,
                        "cugl_conv2d_plan_set_epilogue_warps: plan is NULL or warps is not 0, 4, 8 or 16");
        }
        plan->core.epi_warps = warps;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_tile_columns(cugl_conv_plan *plan, int columns)
    {
        if (plan == nullptr || (columns != 0 && columns != 64 && columns != 128 && columns != 256))
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT,
                        "cugl_conv2d_plan_set_tile_columns: plan is NULL or columns is not 0, 64, 128 or 256");
        }
        plan->core.block_n = columns;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_paired_drain(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_paired_drain: NULL plan");
        }
        plan->core.pair_drain = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_tma_store(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_tma_store: NULL plan");
        }
        plan->core.tma_store = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_resident_weights(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_resident_weights: NULL plan");
        }
        plan->core.resident_b = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_double_tile(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_double_tile: NULL plan");
        }
        plan->core.double_tile = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_allow_tma_im2col(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_allow_tma_im2col: NULL plan");
        }
        plan->allow_tma_im2col = on < 0 ? 0 : (on > 2 ? 2 : on);
        return CUGL_SUCCESS;
    }

    int cugl_conv2d_plan_uses_tma_im2col(const cugl_conv_plan *plan)
    {
        // the conditions the plan can see; the run adds the alignment of the source pointer (16 bytes)
        return plan != nullptr && plan->implicit && plan->allow_implicit && !plan->core.force_simt && plan->allow_tma_im2col != 0 &&
                       plan->desc.src_zero_point == 0 && ((plan->eC % 128) == 0 || (plan->eC == 64 && plan->allow_tma_im2col > 1))
                   ? 1
                   : 0;
    }

    const char *cugl_conv2d_plan_kernel(const cugl_conv_plan *plan)
    {
        if (plan == nullptr)
        {
            return "";
        }
        if (plan->skip_im2col)
        {
            return "gemm";
        }
        return (plan->implicit && plan->allow_implicit) ? "implicit" : "im2col";
    }

    int cugl_conv2d_plan_launches(const cugl_conv_plan *plan)
    {
        if (plan == nullptr)
        {
            return 0;
        }
        const int fold = plan->fold ? 1 : 0;
        if (plan->implicit && plan->allow_implicit)
        {
            return fold + 1;
        }
        return fold + (plan->skip_im2col ? 0 : 1) + 1 + (plan->core.b_off != 0 ? 1 : 0);
    }
    cugl_status cugl_conv2d_update_quantization(cugl_conv_plan *plan, const cugl_conv_desc *desc)
    {
        if (plan == nullptr || desc == nullptr)
        {
            return fail(plan ? plan->ctx : nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_update_quantization: NULL argument");
        }
        const cugl_conv_desc &o = plan->desc;
        if (desc->B != o.B || desc->H != o.H || desc->W != o.W || desc->C != o.C || desc->OFM != o.OFM || desc->kh != o.kh ||
            desc->kw != o.kw || desc->stride_x != o.stride_x || desc->stride_y != o.stride_y ||
            desc->pad_left != o.pad_left || desc->pad_right != o.pad_right || desc->pad_top != o.pad_top ||
            desc->pad_bottom != o.pad_bottom || desc->dil_x != o.dil_x || desc->dil_y != o.dil_y ||
            desc->src_dtype != o.src_dtype || desc->w_dtype != o.w_dtype ||
            desc->is_quantized_per_channel != o.is_quantized_per_channel || desc->has_bias != o.has_bias)
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                        "cugl_conv2d_update_quantization: geometry, types and per-channel kind must not change");
        }
        cugl_status code;
        const char *why = validate_conv(desc, &code);
        if (why != nullptr)
        {
            return fail(plan->ctx, code, std::string("cugl_conv2d_update_quantization: ") + why);
        }
        // the lowering was chosen for symmetric or asymmetric weights; a weights zero point appearing later would
        // need the row sums the implicit kernel does not compute
        if ((desc->w_zero_point != 0) != (o.w_zero_point != 0))
        {
            return fail(plan->ctx, CUGL_UNSUPPORTED_CONFIG,
                        "cugl_conv2d_update_quantization: the weights zero point may not change between zero and non-zero");
        }
        const bool zp_changed = desc->src_zero_point != o.src_zero_point;
        plan->desc.src_zero_point      = desc->src_zero_point;
        plan->desc.w_zero_point        = desc->w_zero_point;
        plan->desc.gemmlowp_multiplier = desc->gemmlowp_multiplier;
        plan->desc.gemmlowp_shift      = desc->gemmlowp_shift;
        plan->desc.dst_zero_point      = desc->dst_zero_point;
        plan->desc.min_bound           = desc->min_bound;
        plan->desc.max_bound           = desc->max_bound;
        GemmCore &c     = plan->core;
        c.a_off         = -desc->src_zero_point;
        c.b_off         = -desc->w_zero_point;
        c.mult          = desc->gemmlowp_multiplier;
        c.shift         = desc->gemmlowp_shift;
        c.result_offset = desc->dst_zero_point;
        c.min_bound     = desc->min_bound;
        c.max_bound     = desc->max_bound;
        if (c.per_channel)
        {
            plan->h_mults.assign(desc->h_gemmlowp_multipliers, desc->h_gemmlowp_multipliers + desc->OFM);
            plan->h_shifts.assign(desc->h_gemmlowp_shifts, desc->h_gemmlowp_shifts + desc->OFM);
        }
        CUGL_TRY(c.upload_stage_vectors(plan->h_mults.data(), plan->h_shifts.data()));
        if (zp_changed && plan->d_pad != nullptr)
        {
            // out-of-image taps read the input zero point from the pad buffer
            CUGL_TRY(cugl_memset(plan->ctx, plan->d_pad, desc->src_zero_point & 0xff, kConvPadBytes));
        }
        return CUGL_SUCCESS;
    }

    cugl_status cugl_transpose_batched(cugl_context *ctx, const void *d_src, void *d_dst, int32_t rows, int32_t cols,
                                       int32_t batch)
    {
        if (ctx == nullptr || d_src == nullptr || d_dst == nullptr || rows < 1 || cols < 1 || batch < 1 || batch > 65535)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_transpose_batched: bad argument");
        }
        return launch_transpose_bytes(ctx, d_src, rows, cols, d_dst, batch);
    }

    cugl_status cugl_gemmlowp_plan_set_saturating_pack(cugl_gemm_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_set_saturating_pack: NULL plan");
        }
        plan->core.pack_stage = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_conv2d_plan_set_saturating_pack(cugl_conv_plan *plan, int on)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_set_saturating_pack: NULL plan");
        }
        plan->core.pack_stage = on != 0 ? 0 : -1;
        return CUGL_SUCCESS;
    }

    // ---- temporary workspaces (MemoryRequirements with lifetime Temporary, arm_compute/core/experimental/Types.h:89-125)
    size_t cugl_gemmlowp_plan_temp_bytes(const cugl_gemm_plan *plan)
    {
        return plan != nullptr ? plan->core.rowsum_bytes() + plan->core.tmp_a_bytes() : 0;
    }

    cugl_status cugl_gemmlowp_plan_bind_temp(cugl_gemm_plan *plan, void *d_ws, size_t bytes)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_plan_bind_temp: NULL plan");
        }
        if (d_ws != nullptr && ((reinterpret_cast<uintptr_t>(d_ws) & 255) != 0 ||
                                bytes < plan->core.rowsum_bytes() + plan->core.tmp_a_bytes()))
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                        "cugl_gemmlowp_plan_bind_temp: workspace must be 256-byte aligned and hold cugl_gemmlowp_plan_temp_bytes");
        }
        plan->core.d_rowsum_bound = (d_ws != nullptr && plan->core.rowsum_bytes() != 0) ? static_cast<int32_t *>(d_ws) : nullptr;
        plan->core.d_tmp_a_bound  = (d_ws != nullptr && plan->core.tmp_a_bytes() != 0)
                                        ? static_cast<uint8_t *>(d_ws) + plan->core.rowsum_bytes()
                                        : nullptr;
        return CUGL_SUCCESS;
    }

    size_t cugl_conv2d_plan_temp_bytes(const cugl_conv_plan *plan)
    {
        return plan != nullptr ? plan->temp_bytes() : 0;
    }

    cugl_status cugl_conv2d_plan_bind_temp(cugl_conv_plan *plan, void *d_ws, size_t bytes)
    {
        if (plan == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_conv2d_plan_bind_temp: NULL plan");
        }
        if (d_ws != nullptr && ((reinterpret_cast<uintptr_t>(d_ws) & 255) != 0 || bytes < plan->temp_bytes()))
        {
            return fail(plan->ctx, CUGL_INVALID_ARGUMENT,
                        "cugl_conv2d_plan_bind_temp: workspace must be 256-byte aligned and hold cugl_conv2d_plan_temp_bytes");
        }
        plan->d_temp              = static_cast<uint8_t *>(d_ws);
        plan->temp_bound_bytes    = d_ws != nullptr ? bytes : 0;
        plan->core.d_rowsum_bound = plan->core.b_off != 0 ? static_cast<int32_t *>(d_ws) : nullptr;
        return CUGL_SUCCESS;
    }
}
