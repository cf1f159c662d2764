/*
 * cugl -- C ABI of the B200 (sm_100a) backend for Compute Library's quantized GEMM path.
 *
 * This header is the drop-in boundary: host C++ that keeps the arm_compute API
 * (IFunction::configure/validate/run, ITensor/TensorInfo/QuantizationInfo, GEMMInfo,
 * GEMMLowpOutputStageInfo) reaches the GPU only through these entry points.  Plain C types only.
 * Every "d_" pointer is a device pointer on the context's device; every "h_" pointer is host memory.
 * Work is enqueued on the context's stream and is asynchronous unless the comment says otherwise.
 * There is no CPU fallback: a call that cannot run on the GPU returns an error.
 *
 * Reference citations are paths inside the Compute Library tree.
 *
 * Arithmetic contract (all two's-complement int32; identical to tests/validation/reference/GEMMLowp.cpp):
 *   acc[m,n] = sum_k A[m,k]*B[k,n] + a_offset*colsum_B[n] + b_offset*rowsum_A[m] + K*a_offset*b_offset
 *            ( == sum_k (A[m,k]+a_offset)*(B[k,n]+b_offset): offsets are ADDED as passed )
 *   acc     += bias[n]
 *   r        = shift < 0 ? sqdmulh(acc << -shift, mult) : (sqdmulh(acc, mult) + (1 << (shift-1))) >> shift
 *              sqdmulh(a,b) = (int64(a)*b*2) >> 32  (floor, saturating only for INT32_MIN*INT32_MIN)
 *   out      = clamp(r + result_offset, max(min_bound, type_min), min(max_bound, type_max))
 */
#ifndef CUGL_H
#define CUGL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define CUGL_API
#else
#define CUGL_API __attribute__((visibility("default")))
#endif

/* Status codes; the values mirror AclStatus (arm_compute/AclTypes.h:53-64) where a counterpart exists. */
typedef enum cugl_status
{
    CUGL_SUCCESS            = 0,
    CUGL_RUNTIME_ERROR      = 1, /* CUDA error or device-side time-out; see cugl_last_error_string */
    CUGL_OUT_OF_MEMORY      = 2,
    CUGL_UNIMPLEMENTED      = 3,
    CUGL_UNSUPPORTED_TARGET = 4, /* no sm_100 device */
    CUGL_INVALID_ARGUMENT   = 6,
    CUGL_UNSUPPORTED_CONFIG = 8
} cugl_status;

/* 8-bit operand / output element types.  QASYMM8 -> U8; QASYMM8_SIGNED, QSYMM8, QSYMM8_PER_CHANNEL -> S8
 * (arm_compute/core/CoreTypes.h DataType). */
typedef enum cugl_dtype
{
    CUGL_U8  = 0,
    CUGL_S8  = 1,
    CUGL_S32 = 2,
    CUGL_S16 = 3, /* QSYMM16: destination of the stand-alone fixed-point output stage only */
    CUGL_F32 = 4  /* destination of the GEMM with stage NONE: the int32 result times dequantize_scale */
} cugl_dtype;

/* GEMMLowpOutputStageType (arm_compute/function_info/GEMMInfo.h:40-46).  Only NONE and
 * QUANTIZE_DOWN_FIXEDPOINT are on the accelerated path. */
typedef enum cugl_stage
{
    CUGL_STAGE_NONE                     = 0,
    /* ((acc + gemmlowp_offset + bias) * gemmlowp_multiplier) >> gemmlowp_shift, integer multiply, shift >= 0;
     * clamp to [min, max] when they differ, saturate to the 8-bit type (GEMMLowpOutputStageType::QUANTIZE_DOWN,
     * tests/validation/reference/GEMMLowp.cpp:66-104) */
    CUGL_STAGE_QUANTIZE_DOWN            = 1,
    CUGL_STAGE_QUANTIZE_DOWN_FIXEDPOINT = 2
} cugl_stage;

typedef struct cugl_context   cugl_context;   /* one per device + stream; not thread-safe */
typedef struct cugl_gemm_plan cugl_gemm_plan; /* configured NEGEMMLowpMatrixMultiplyCore instance */
typedef struct cugl_conv_plan cugl_conv_plan; /* configured NEGEMMConvolutionLayer instance */

/* ------------------------------------------------------------------------------------------------
 * Context, memory, stream.  Replaces the host TensorAllocator / MemoryManagerOnDemand / NEScheduler
 * trio (src/runtime/TensorAllocator.cpp:133-146, arm_compute/runtime/IAllocator.h:39-61,
 * src/runtime/IScheduler.cpp:58-180) by cudaMalloc-backed regions and one CUDA stream.
 * ---------------------------------------------------------------------------------------------- */

/* stream: the cudaStream_t to enqueue on; NULL is the CUDA default stream.  Pass CUGL_STREAM_CREATE to let
 * the context create (and later destroy) a non-blocking stream of its own. */
#define CUGL_STREAM_CREATE ((void *)(intptr_t)-1)
CUGL_API cugl_status cugl_context_create(int device, void *stream, cugl_context **out);
CUGL_API void        cugl_context_destroy(cugl_context *ctx);
/* Text of the last error raised through this context (never NULL). ctx may be NULL: global last error. */
CUGL_API const char *cugl_last_error_string(const cugl_context *ctx);
CUGL_API void       *cugl_context_stream(const cugl_context *ctx);
CUGL_API int         cugl_context_device(const cugl_context *ctx);
CUGL_API int         cugl_context_sm_count(const cugl_context *ctx);

/* Profiling aid (the role of the reference's scheduler timer, tests/framework/instruments/SchedulerTimer.cpp):
 * when d_buffer is not NULL every tensor-core GEMM launch records %globaltimer timestamps (ns) of its pipeline
 * events into it: int64 [grid][8 tiles][8 events]; events 0 first copy issued, 1 accumulator acquired, 2 first
 * operands landed, 3 last MMA issued, 4 epilogue sees the accumulator, 5 tile stored.  The buffer must hold
 * 64 * 8 bytes per CTA of the launch (at most 2 * SM count CTAs).  NULL switches tracing off. */
CUGL_API cugl_status cugl_context_set_trace_buffer(cugl_context *ctx, void *d_buffer);

/* Every wait of a tensor-core kernel on a barrier (operands landed, stage free, accumulator complete / drained) is
 * bounded: when it has lasted longer than the limit the kernel stops issuing work, waits for the copies it has in
 * flight, frees its tensor memory, returns, and the next cugl_sync() reports CUGL_RUNTIME_ERROR; the context stays
 * usable.  The limit is two seconds unless set here, in microseconds (0 restores the default).  It is the
 * counterpart of the scheduler-side run-time checks of the reference (IScheduler::schedule errors); the reference
 * has no device waits. */
CUGL_API cugl_status cugl_context_set_wait_limit_us(cugl_context *ctx, uint64_t microseconds);
/* Test instrument of that path, no reference counterpart: in the NEXT tensor-core GEMM launch of this context the
 * producer of CTA 0 leaves out the operand copies of k-block ordinal `k_block` (counted over the CTA's tile
 * sequence), so that the wait for them runs out.  One shot: the launch after it is normal again. */
CUGL_API cugl_status cugl_context_withhold_copy_once(cugl_context *ctx, int k_block);
/* The tensor-core kernels are launched with programmatic stream serialization (on by default): a kernel lets the next
 * one in the stream start its prologue (barrier set-up, tensor-memory allocation) while its own last tiles finish, and
 * every kernel waits for its predecessor's completion (griddepcontrol.wait) before its first access to global memory.
 * A stream that is being captured into a CUDA graph gets plain launches (measured faster there).  0 restores plain
 * stream order everywhere.  No
 * reference counterpart (the NE scheduler runs its kernels back to back on the host threads). */
CUGL_API cugl_status cugl_context_set_dependent_launch(cugl_context *ctx, int on);

/* IAllocator::allocate / free (arm_compute/runtime/IAllocator.h:39-61): device regions, 256-byte aligned. */
CUGL_API cugl_status cugl_malloc(cugl_context *ctx, size_t bytes, void **d_ptr);
CUGL_API cugl_status cugl_free(cugl_context *ctx, void *d_ptr);
/* Pinned host staging memory for map()/unmap() style access (ICLTensor::map precedent,
 * arm_compute/core/CL/ICLTensor.h:45-111). */
CUGL_API cugl_status cugl_host_alloc(cugl_context *ctx, size_t bytes, void **h_ptr);
CUGL_API cugl_status cugl_host_free(cugl_context *ctx, void *h_ptr);
CUGL_API cugl_status cugl_memcpy_h2d(cugl_context *ctx, void *d_dst, const void *h_src, size_t bytes);
CUGL_API cugl_status cugl_memcpy_d2h(cugl_context *ctx, void *h_dst, const void *d_src, size_t bytes);
/* Device-to-device copy on the context's stream (the reshape-type layers that only re-label a dense tensor:
 * NEFlattenLayer / NEReshapeLayer, src/cpu/operators/CpuFlatten.cpp). */
CUGL_API cugl_status cugl_memcpy_d2d(cugl_context *ctx, void *d_dst, const void *d_src, size_t bytes);
/* Strided 2-D copies for host tensors with padding (ITensorInfo strides_in_bytes /
 * offset_first_element_in_bytes, arm_compute/core/ITensorInfo.h:197-211). */
CUGL_API cugl_status cugl_memcpy2d_h2d(cugl_context *ctx, void *d_dst, size_t d_pitch, const void *h_src,
                                       size_t h_pitch, size_t width_bytes, size_t rows);
CUGL_API cugl_status cugl_memcpy2d_d2h(cugl_context *ctx, void *h_dst, size_t h_pitch, const void *d_src,
                                       size_t d_pitch, size_t width_bytes, size_t rows);
/* CUDA IPC: export a cugl_malloc'ed buffer to the other single-GPU processes of the node (64-byte handle) and
 * map a peer's buffer into this process. */
CUGL_API cugl_status cugl_ipc_get_handle(cugl_context *ctx, void *d_ptr, void *handle64);
CUGL_API cugl_status cugl_ipc_open_handle(cugl_context *ctx, const void *handle64, void **d_ptr);
CUGL_API cugl_status cugl_ipc_close_handle(cugl_context *ctx, void *d_ptr);
CUGL_API cugl_status cugl_memset(cugl_context *ctx, void *d_ptr, int value, size_t bytes);
/* Blocks until the stream is idle; reports any asynchronous CUDA error or device-side time-out.
 * (CLScheduler::sync precedent; IFunction::run of a device backend does not block,
 * arm_compute/runtime/IFunction.h:46-51.) */
CUGL_API cugl_status cugl_sync(cugl_context *ctx);

/* ------------------------------------------------------------------------------------------------
 * Host-side quantisation helpers (no GPU work).
 * ---------------------------------------------------------------------------------------------- */

/* quantization::calculate_quantized_multiplier (src/core/utils/quantization/AsymmHelpers.cpp:43-115).
 * shift > 0: right shift; shift < 0: left shift. */
CUGL_API cugl_status cugl_calculate_quantized_multiplier(float multiplier, int32_t *quant_multiplier,
                                                         int32_t *shift);
/* quantization::calculate_quantized_multipliers (AsymmHelpers.cpp:117-152): multiplier[i] =
 * i_scale * w_scales[i] / o_scale in float32. */
CUGL_API cugl_status cugl_calculate_quantized_multipliers(float i_scale, const float *w_scales, int n,
                                                          float o_scale, int32_t *multipliers, int32_t *shifts);

/* ------------------------------------------------------------------------------------------------
 * NEGEMMLowpMatrixMultiplyCore (+ fused NEGEMMLowpOutputStage)
 *   arm_compute/runtime/NEON/functions/NEGEMMLowpMatrixMultiplyCore.h:54-128
 *   src/cpu/operators/CpuGemmLowpMatrixMultiplyCore.cpp:116-360 (configure), 362-645 (validate),
 *   647-811 (run), 813-850 (prepare)
 * ---------------------------------------------------------------------------------------------- */
typedef struct cugl_gemm_desc
{
    int32_t M, N, K;     /* dst is M x N; A is M x K (K contiguous); B is K x N (N contiguous) */
    int32_t batch;       /* >= 1; A and dst slide along the batch, B only if b_batch_stride != 0 */
    int64_t lda;         /* bytes between rows of A  (TensorInfo::strides_in_bytes()[1]) */
    int64_t ldb;         /* bytes between rows of B */
    int64_t ldd;         /* bytes between rows of dst */
    int64_t a_batch_stride, b_batch_stride, d_batch_stride; /* bytes; b_batch_stride 0 = shared B */
    int32_t a_dtype;     /* CUGL_U8 | CUGL_S8 */
    int32_t b_dtype;     /* CUGL_U8 | CUGL_S8 */
    int32_t dst_dtype;   /* CUGL_U8 | CUGL_S8 with a quantize-down stage; CUGL_S32 or CUGL_F32 with stage NONE */
    int32_t a_offset;    /* a->quantization_info().uniform().offset AS PASSED to the core (it is added);
                            library callers pass the negated zero point (CpuGemmConv2d.cpp:266-280) */
    int32_t b_offset;    /* likewise; must be 0 for per-channel B with a signed dst
                            (CpuGemmLowpOffsetContributionOutputStageKernel.cpp:832-836) */
    int32_t stage;       /* cugl_stage */
    int32_t is_quantized_per_channel; /* GEMMLowpOutputStageInfo::is_quantized_per_channel */
    int32_t gemmlowp_multiplier;      /* per-tensor multiplier / shift / offset / bounds: */
    int32_t gemmlowp_shift;           /*   GEMMLowpOutputStageInfo, GEMMInfo.h:49-82 */
    const int32_t *h_gemmlowp_multipliers; /* per-channel: N host values (read during plan_create / update) */
    const int32_t *h_gemmlowp_shifts;
    int32_t gemmlowp_offset;
    int32_t gemmlowp_min_bound;
    int32_t gemmlowp_max_bound;
    int32_t has_bias;                 /* c != nullptr: S32 [N], only with an output stage */
    int32_t reshape_b_only_on_first_run; /* GEMMInfo flag: B (and its column sums) are constant after prepare */
    int32_t accumulate;  /* GEMMInfo::accumulate(): stage NONE only, dst += result instead of dst = result
                            (CpuGemmLowpMatrixMultiplyCore.cpp:393-401) */
    float   dequantize_scale; /* dst_dtype CUGL_F32: dst = float(int32 result) * dequantize_scale, the product of the
                            two operand scales (the s8 -> f32 rows of NEGEMMLowpMatrixMultiplyCore.h:72-90;
                            CpuGemmLowpMatrixMultiplyCore.cpp:305-320); float(x) rounds to nearest, one float multiply */
} cugl_gemm_desc;

/* static Status validate(a, b, c, output, gemm_info): pure host check, no GPU needed.
 * Rules: CpuGemmLowpMatrixMultiplyCore.cpp:370-401 and
 * CpuGemmLowpOffsetContributionOutputStageKernel.cpp:820-906.  reason (optional) receives a pointer to a
 * static string. */
CUGL_API cugl_status cugl_gemmlowp_validate(const cugl_gemm_desc *desc, const char **reason);
/* configure(): validates, sizes the workspace (transposed B, column / row sums, per-channel vectors)
 * and uploads the output-stage vectors.  Allocates device memory; no kernel is launched. */
CUGL_API cugl_status cugl_gemmlowp_plan_create(cugl_context *ctx, const cugl_gemm_desc *desc,
                                               cugl_gemm_plan **out);
CUGL_API void        cugl_gemmlowp_plan_destroy(cugl_gemm_plan *plan);
/* prepare(): re-lays B out K-major for the tensor cores and reduces its columns
 * (CpuGemmLowpMatrixMultiplyCore.cpp:813-846).  After it, d_b may be freed when
 * reshape_b_only_on_first_run is set. */
CUGL_API cugl_status cugl_gemmlowp_prepare(cugl_gemm_plan *plan, const void *d_b);
/* run(): d_b is only read when reshape_b_only_on_first_run == 0 (or prepare has not been called);
 * d_bias may be NULL when has_bias == 0. */
CUGL_API cugl_status cugl_gemmlowp_run(cugl_gemm_plan *plan, const void *d_a, const void *d_b,
                                       const int32_t *d_bias, void *d_dst);
/* Fused GEMMLowp + push all-gather step for the column-sharded linear layer: the epilogue stores every
 * finished 8-bit tile into ALL n_dsts (1..8) destination matrices, which share the descriptor's ldd.  Pass this
 * GPU's own buffer and the peers' buffers (opened with cugl_ipc_open_handle), each already advanced to this
 * GPU's first column: the output block then crosses NVLink while later tiles are still being computed, and no
 * separate all-gather runs.  Plain peer stores, no multicast.  Completion on the peers is established by the
 * caller (stream sync + a host barrier).  Needs the tensor-core kernel; no counterpart in the reference, which
 * is single-device. */
CUGL_API cugl_status cugl_gemmlowp_run_multi(cugl_gemm_plan *plan, const void *d_a, const int32_t *d_bias,
                                             void *const *d_dsts, int32_t n_dsts);
/* Same function driven from host buffers: copies A (and bias) in, runs, copies dst out, and blocks
 * until dst is valid.  h_a / h_dst follow lda / ldd of the descriptor. */
CUGL_API cugl_status cugl_gemmlowp_run_host(cugl_gemm_plan *plan, const void *h_a, const int32_t *h_bias,
                                            void *h_dst);
/* update_quantization_parameters() (NEGEMMLowpMatrixMultiplyCore.cpp:118-159): re-reads offsets and the
 * output-stage fields of desc; shapes and types must be unchanged. */
CUGL_API cugl_status cugl_gemmlowp_update_quantization(cugl_gemm_plan *plan, const cugl_gemm_desc *desc);
/* Which kernel the plan will launch: "tcgen05_2cta" (TMA + tcgen05.mma.cta_group::2.kind::i8 on SM pairs,
 * 256 x 256 tiles), "tcgen05" (one CTA per 128 x N tile) or "simt" (shape / stride not expressible as a TMA
 * tensor map). */
CUGL_API const char *cugl_gemmlowp_plan_kernel(const cugl_gemm_plan *plan);
/* Force the generic kernel (testing aid: both kernels must agree bit for bit). */
CUGL_API cugl_status cugl_gemmlowp_plan_force_simt(cugl_gemm_plan *plan, int on);
/* on = 0 keeps the plan to the one-CTA tensor-core kernels (testing aid). */
CUGL_API cugl_status cugl_gemmlowp_plan_allow_pair_kernel(cugl_gemm_plan *plan, int on);
/* cugl_gemmlowp_run_host splits a large product into row blocks that travel in, are multiplied and travel out as a
 * pipeline; blocks = how many (1: no pipeline, 0: the default, at most 32).  Tuning aid; results do not depend on it. */
CUGL_API cugl_status cugl_gemmlowp_plan_set_host_pipeline(cugl_gemm_plan *plan, int blocks);
/* Number of kernels one cugl_gemmlowp_run of this plan launches. */
CUGL_API int cugl_gemmlowp_plan_launches(const cugl_gemm_plan *plan);
/* The tensor-core kernels exist with four, eight and (256-column one-CTA tiles only) sixteen epilogue warps; the
 * library picks by K and N (long K: four; short K: eight, sixteen for more than 128 output columns).
 * warps = 4, 8 or 16 forces one build where it exists, 0 restores the automatic choice (testing / measurement
 * aid: the results are identical). */
CUGL_API cugl_status cugl_gemmlowp_plan_set_epilogue_warps(cugl_gemm_plan *plan, int warps);
/* The tensor-core GEMM can also run with the operand roles exchanged, which makes an accumulator lane an output
 * channel (output-stage terms in registers, byte-wise transposed stores; never with a row-sum term or several
 * destinations).  mode > 0 requests it, < 0 forbids it, 0 lets the library choose (K from 256 to 1024 with at
 * least 256 output channels).  Testing / measurement aid: the results are identical. */
CUGL_API cugl_status cugl_gemmlowp_plan_set_channel_major(cugl_gemm_plan *plan, int mode);
/* SM-pair kernel: when the last wave of 256 x 256 tiles fills at most half of the SM pairs, its tiles are
 * processed as two 256 x 128 halves each (on by default).  on = 0 keeps them whole.  Testing / measurement aid:
 * the results are identical. */
CUGL_API cugl_status cugl_gemmlowp_plan_set_tail_split(cugl_gemm_plan *plan, int on);
/* Tile width of the one-CTA tensor-core kernels, in output columns.  By default (0) the widest tile N calls for
 * (256 above 128 columns, 128 above 64, else 64) unless the output then has fewer tiles than the device has
 * SMs: a small output gets narrower tiles so that more SMs share its K loop (and is kept off the SM-pair and
 * sixteen-warp kernels, which exist for 256 columns only).  columns = 64, 128 or 256 forces a width (capped at
 * the widest N calls for).  Testing / measurement aid: the results are identical. */
CUGL_API cugl_status cugl_gemmlowp_plan_set_tile_columns(cugl_gemm_plan *plan, int columns);
/* One-CTA kernel, 256-column tiles, 8-bit output with shifts >= 2 and non-negative multipliers: two consecutive
 * tiles of one column block are drained from their two accumulator buffers together, so that each per-column
 * output-stage term is read from shared memory once for two elements (on by default).  on = 0 drains every
 * tile on its own.  Testing / measurement aid: the results are identical. */
CUGL_API cugl_status cugl_gemmlowp_plan_set_paired_drain(cugl_gemm_plan *plan, int on);
/* The one-CTA kernels with four or eight epilogue warps send a warp's 32 output rows off as one bulk tensor store from
 * shared memory where the destination allows it (8-bit output, one destination, 16-byte aligned base and pitch);
 * on = 0 keeps them on per-lane global stores (testing aid: results do not depend on it). */
CUGL_API cugl_status cugl_gemmlowp_plan_set_tma_store(cugl_gemm_plan *plan, int on);

/* Output stages whose clamp bounds are the whole range of the 8-bit output type (every shift in [2, 31], or [2, 22]
 * with a non-zero output offset; non-negative multipliers; no B offset) fold the offset into the per-column constant
 * and clamp by the saturation of the byte-packing instruction: fewer instructions per output (on by default).
 * on = 0 keeps the explicit add / min / max form.  Testing / measurement aid: the results are identical. */
CUGL_API cugl_status cugl_gemmlowp_plan_set_saturating_pack(cugl_gemm_plan *plan, int on);

/* MemoryRequirements of the operator with lifetime Temporary (arm_compute/core/experimental/Types.h:89-125; the
 * VectorSumRow slot of src/cpu/operators/CpuGemmLowpMatrixMultiplyCore.h:144-155): bytes of device memory a run of the
 * plan needs that hold nothing between runs (the row sums of A, only with a non-zero B offset).  By default the plan
 * allocates them itself on first use.  cugl_gemmlowp_plan_bind_temp makes later runs use [d_ws, d_ws + bytes)
 * instead (256-byte aligned, at least _temp_bytes), so that a host-side memory manager (MemoryGroup /
 * MemoryManagerOnDemand) can hand the same bytes to other functions between runs; d_ws = NULL unbinds. */
CUGL_API size_t      cugl_gemmlowp_plan_temp_bytes(const cugl_gemm_plan *plan);
CUGL_API cugl_status cugl_gemmlowp_plan_bind_temp(cugl_gemm_plan *plan, void *d_ws, size_t bytes);

/* Fused GEMMLowp that allocates nothing.  No counterpart in the reference: Compute Library always lets the
 * function object own its workspace.  For callers that cannot call cudaMalloc -- a serving loop whose device
 * memory is fully committed to its own arena, a plugin that may not touch the host's allocator, code inside
 * a stream capture.  The workspace (K-major copy of B, column sums, row sums) is a fixed array inside the
 * library image, about 4.3 MB held by every GPU that loads the library until the process exits.
 *   - Limits: batch == 1, M <= 65536, N <= 8192, N * round_up(K, 128) <= 4 MiB; larger problems are rejected
 *     with CUGL_INVALID_ARGUMENT (use the planned entry points).
 *   - Per-channel multipliers / shifts are read from DEVICE vectors (the h_ pointers of desc are ignored).
 *   - stream is the cudaStream_t to enqueue on (NULL = default stream); the device must be current.
 *   - The first call on a device resolves the array's device address and clears a status word; make that
 *     first call outside any stream capture.
 *   - All calls share the one array, which keeps the previous call's contents (the column sums are cleared
 *     by the call itself): calls that overlap on the GPU -- different streams, or graph branches -- race.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine; B is re-laid out on every call.
 *   - The call is asynchronous.  A device-side time-out (every wait of the kernels is bounded) cannot be reported
 *     by the call itself: ask cugl_gemmlowp_noalloc_status afterwards. */
CUGL_API cugl_status cugl_gemmlowp_run_noalloc(void *stream, const cugl_gemm_desc *desc, const void *d_a,
                                               const void *d_b, const int32_t *d_bias,
                                               const int32_t *d_multipliers, const int32_t *d_shifts, void *d_dst);
/* Companion of cugl_gemmlowp_run_noalloc (no counterpart in the reference either): waits for `stream`, then
 * returns CUGL_RUNTIME_ERROR if a kernel of an earlier allocation-free call on the current device gave up a bounded
 * wait (and clears that record), else CUGL_SUCCESS.  Allocates nothing; the role of cugl_sync for this path. */
CUGL_API cugl_status cugl_gemmlowp_noalloc_status(void *stream);

/* ------------------------------------------------------------------------------------------------
 * Stand-alone kernels of the path.
 * ---------------------------------------------------------------------------------------------- */

/* CpuGemmLowpMatrixAReductionKernel (src/cpu/kernels/CpuGemmLowpMatrixReductionKernel.cpp:133-204):
 * d_out[m] = scalar * sum_k A[m,k]  (scalar 1 when GEMMLowpReductionKernelInfo::mul_by_scalar is false). */
CUGL_API cugl_status cugl_reduce_rows(cugl_context *ctx, const void *d_a, int32_t dtype, int32_t M, int32_t K,
                                      int64_t lda, int32_t scalar, int32_t *d_out);
/* CpuGemmLowpMatrixBReductionKernel (…ReductionKernel.cpp:273-446): d_out[n] = scalar * sum_k B[k,n]. */
CUGL_API cugl_status cugl_reduce_cols(cugl_context *ctx, const void *d_b, int32_t dtype, int32_t K, int32_t N,
                                      int64_t ldb, int32_t scalar, int32_t *d_out);
/* CpuGemmLowpOffsetContributionKernel (src/cpu/kernels/CpuGemmLowpOffsetContributionKernel.cpp:116-229):
 * in place on an S32 [M,N] product.  d_colsum may be NULL when a_offset == 0, d_rowsum when b_offset == 0. */
CUGL_API cugl_status cugl_offset_contribution(cugl_context *ctx, int32_t *d_mm, int32_t M, int32_t N, int32_t K,
                                              int64_t ld_bytes, const int32_t *d_colsum, const int32_t *d_rowsum,
                                              int32_t a_offset, int32_t b_offset);
/* NEGEMMLowpOutputStage, QUANTIZE_DOWN_FIXEDPOINT (src/cpu/operators/CpuGemmLowpOutputStage.cpp:41-167,
 * CpuGemmLowpQuantizeDownInt32ToUint8ScaleByFixedPointKernel.cpp:78-186): S32 [M,N] (+ S32 bias [N])
 * -> U8 / S8 [M,N].  n_mult == 1: per-tensor (the NE function), n_mult == N: per-column device vectors.
 * out_dtype CUGL_S16 is the QSYMM16 variant (CpuGemmLowpOutputStage.cpp:73-80,
 * CpuGemmLowpQuantizeDownInt32ToInt16ScaleByFixedPointKernel): the same arithmetic saturated to int16, rows of
 * ld_out_bytes >= 2 N bytes, 2-byte aligned; the NE kernel has no offset, pass result_offset = 0 for it. */
CUGL_API cugl_status cugl_output_stage(cugl_context *ctx, const int32_t *d_in, int64_t ld_in_bytes,
                                       const int32_t *d_bias, void *d_out, int64_t ld_out_bytes, int32_t out_dtype,
                                       int32_t M, int32_t N, const int32_t *d_multipliers, const int32_t *d_shifts,
                                       int32_t multiplier, int32_t shift, int32_t n_mult, int32_t result_offset,
                                       int32_t min_bound, int32_t max_bound);
/* The same entry point for the QUANTIZE_DOWN (integer multiply) stage: NEGEMMLowpOutputStage with
 * GEMMLowpOutputStageType::QUANTIZE_DOWN (src/cpu/operators/CpuGemmLowpOutputStage.cpp:41-167). */
CUGL_API cugl_status cugl_output_stage_quantize_down(cugl_context *ctx, const int32_t *d_in, int64_t ld_in_bytes,
                                       const int32_t *d_bias, void *d_out, int64_t ld_out_bytes, int32_t out_dtype,
                                       int32_t M, int32_t N, const int32_t *d_multipliers, const int32_t *d_shifts,
                                       int32_t multiplier, int32_t shift, int32_t n_mult, int32_t result_offset,
                                       int32_t min_bound, int32_t max_bound);
/* CpuIm2ColKernel, NHWC, 8-bit (src/cpu/kernels/CpuIm2ColKernel.cpp:296-420,
 * src/cpu/kernels/directconv2d/impl.h:148-220,307-388): src [B][H][W][C] -> dst [B*Ho*Wo][row_stride]
 * with K = kh*kw*C bytes per row in (ky,kx,c) order; out-of-image taps = pad_value (the input zero
 * point); bytes K..row_stride-1 are zeroed. */
CUGL_API cugl_status cugl_im2col_nhwc(cugl_context *ctx, const void *d_src, void *d_dst, int32_t C, int32_t W,
                                      int32_t H, int32_t B, int32_t kw, int32_t kh, int32_t stride_x,
                                      int32_t stride_y, int32_t pad_left, int32_t pad_top, int32_t dil_x,
                                      int32_t dil_y, int32_t Wo, int32_t Ho, int32_t pad_value,
                                      int64_t row_stride);
/* CpuWeightsReshapeKernel (src/cpu/kernels/CpuWeightsReshapeKernel.cpp:121-183) for NHWC weights
 * [OFM][kh][kw][C] -> [K][OFM] (row = (ky*kw+kx)*C+c). */
CUGL_API cugl_status cugl_weights_reshape_nhwc(cugl_context *ctx, const void *d_w, void *d_dst, int32_t K,
                                               int32_t OFM);

/* batch dense matrices of rows x cols bytes, back to back, each transposed into cols x rows (blockwise through shared
 * memory).  With rows = C, cols = H*W this is the NCHW -> NHWC permute of 8-bit images (NEPermute with
 * PermutationVector(2, 0, 1), as CpuGemmConv2d's callers use it), with rows = H*W, cols = C the way back. */
CUGL_API cugl_status cugl_transpose_batched(cugl_context *ctx, const void *d_src, void *d_dst, int32_t rows,
                                            int32_t cols, int32_t batch);

/* ------------------------------------------------------------------------------------------------
 * NEGEMMConvolutionLayer for 8-bit NHWC tensors
 *   src/runtime/NEON/functions/NEGEMMConvolutionLayer.cpp:60-145
 *   src/cpu/operators/CpuGemmConv2d.cpp:243-332 (configure_mm), 461-651 (configure), 910-1009 (run),
 *   1011-1101 (prepare)
 * ---------------------------------------------------------------------------------------------- */
typedef struct cugl_conv_desc
{
    int32_t B, H, W, C;     /* src  TensorShape(C, W, H, B), NHWC */
    int32_t OFM, kh, kw;    /* weights TensorShape(C, kw, kh, OFM) */
    int32_t stride_x, stride_y;
    int32_t pad_left, pad_right, pad_top, pad_bottom; /* PadStrideInfo, FLOOR rounding */
    int32_t dil_x, dil_y;
    int32_t src_dtype;      /* CUGL_U8 | CUGL_S8; dst has the same type */
    int32_t w_dtype;        /* CUGL_U8 | CUGL_S8 */
    int32_t src_zero_point; /* TRUE zero points: the layer negates them itself (CpuGemmConv2d.cpp:266-280) */
    int32_t w_zero_point;   /* 0 for QSYMM8_PER_CHANNEL */
    int32_t is_quantized_per_channel;
    int32_t gemmlowp_multiplier, gemmlowp_shift;
    const int32_t *h_gemmlowp_multipliers; /* OFM host values when per-channel */
    const int32_t *h_gemmlowp_shifts;
    int32_t dst_zero_point; /* gemmlowp_offset */
    int32_t min_bound, max_bound; /* from get_quantized_activation_min_max (src/core/Utils.cpp:442-460) */
    int32_t has_bias;
} cugl_conv_desc;

CUGL_API cugl_status cugl_conv2d_validate(const cugl_conv_desc *desc, const char **reason);
CUGL_API cugl_status cugl_conv2d_plan_create(cugl_context *ctx, const cugl_conv_desc *desc, cugl_conv_plan **out);
CUGL_API void        cugl_conv2d_plan_destroy(cugl_conv_plan *plan);
/* prepare(): weights -> K-major GEMM operand + column sums (weights may be freed afterwards). */
CUGL_API cugl_status cugl_conv2d_prepare(cugl_conv_plan *plan, const void *d_weights);
/* run(): im2col (skipped for 1x1 / stride 1 / no pad, CpuGemmConv2d.cpp:189-191) + fused GEMMLowp.
 * dst is [B][Ho][Wo][OFM]. */
CUGL_API cugl_status cugl_conv2d_run(cugl_conv_plan *plan, const void *d_src, const int32_t *d_bias, void *d_dst);
CUGL_API cugl_status cugl_conv2d_run_host(cugl_conv_plan *plan, const void *h_src, const int32_t *h_bias,
                                          void *h_dst);
CUGL_API void cugl_conv2d_out_dims(const cugl_conv_desc *desc, int32_t *Wo, int32_t *Ho);
CUGL_API int  cugl_conv2d_plan_launches(const cugl_conv_plan *plan);
/* How the plan lowers the convolution: "implicit" (patches gathered inside the tensor-core kernel, no im2col
 * matrix: channel count a multiple of 16, symmetric weights), "im2col" (explicit CpuIm2ColKernel-style matrix +
 * GEMMLowp) or "gemm" (1x1 / stride 1 / no padding: the input tensor is the A matrix). */
CUGL_API const char *cugl_conv2d_plan_kernel(const cugl_conv_plan *plan);
/* on = 0 forces the explicit im2col lowering (testing aid: both lowerings must agree bit for bit). */
CUGL_API cugl_status cugl_conv2d_plan_allow_implicit(cugl_conv_plan *plan, int on);
/* The implicit lowering has two ways of forming the patch tiles: im2col-mode TMA loads (the copy engine walks the
 * window origins itself; exact when the input zero point is 0 -- the value out-of-image taps read as) and a gather by
 * eight warps of 16-byte asynchronous copies (any zero point, channels a multiple of 16).  on = 1 (default): TMA loads
 * for channel counts that are multiples of 128, where they measured level with the gather; on = 2: also for exactly
 * 64 channels (one filter tap per 64-byte-swizzle tile; correct, but measured slower than the gather); on = 0: never
 * (testing aid: the routes must agree bit for bit).  cugl_conv2d_plan_uses_tma_im2col tells which one the plan's next
 * run takes (1 / 0). */
CUGL_API cugl_status cugl_conv2d_plan_allow_tma_im2col(cugl_conv_plan *plan, int on);
CUGL_API int         cugl_conv2d_plan_uses_tma_im2col(const cugl_conv_plan *plan);
/* as cugl_gemmlowp_plan_set_epilogue_warps / cugl_gemmlowp_plan_set_channel_major (the latter acts on the
 * lowerings that run the plain GEMM kernel: 1x1 convolutions and the explicit im2col path) */
CUGL_API cugl_status cugl_conv2d_plan_set_epilogue_warps(cugl_conv_plan *plan, int warps);
CUGL_API cugl_status cugl_conv2d_plan_set_channel_major(cugl_conv_plan *plan, int mode);
/* as cugl_gemmlowp_plan_set_tile_columns, for every lowering of the convolution */
CUGL_API cugl_status cugl_conv2d_plan_set_tile_columns(cugl_conv_plan *plan, int columns);
/* as cugl_gemmlowp_plan_set_paired_drain, for the lowerings that run the plain GEMM kernel */
CUGL_API cugl_status cugl_conv2d_plan_set_paired_drain(cugl_conv_plan *plan, int on);
/* as cugl_gemmlowp_plan_set_tma_store */
CUGL_API cugl_status cugl_conv2d_plan_set_tma_store(cugl_conv_plan *plan, int on);
/* Implicit lowering with at most 64 output channels and K = kh * kw * C <= 640: the weight operand is loaded into shared
 * memory once per thread block and stays there (on by default); 0 reloads it with every tile as for larger filters.
 * For tests and measurements; results do not depend on it. */
CUGL_API cugl_status cugl_conv2d_plan_set_resident_weights(cugl_conv_plan *plan, int on);
/* The same layers (resident weights) with more than 256 output pixels per SM: a thread block works on units of 256
 * output pixels, two 128-row tiles that share every barrier hand-over (on by default); 0 keeps 128-row units.  For tests
 * and measurements; results do not depend on it. */
CUGL_API cugl_status cugl_conv2d_plan_set_double_tile(cugl_conv_plan *plan, int on);
/* NEGEMMConvolutionLayer::update_quantization_parameters (src/runtime/NEON/functions/NEGEMMConvolutionLayer.cpp:129-131,
 * src/cpu/operators/CpuGemmConv2d.cpp:858-908): re-reads the zero points, the multipliers / shifts, the output zero
 * point and the clamp bounds of desc; geometry and types must be unchanged.  The prepared weights stay valid. */
CUGL_API cugl_status cugl_conv2d_update_quantization(cugl_conv_plan *plan, const cugl_conv_desc *desc);
/* As cugl_gemmlowp_plan_temp_bytes / _bind_temp for the convolution: row sums, the folded stem input and -- explicit
 * lowering only -- the im2col matrix (the Im2ColOutput slot of CpuGemmConv2d, src/cpu/operators/CpuGemmConv2d.h). */
CUGL_API size_t      cugl_conv2d_plan_temp_bytes(const cugl_conv_plan *plan);
CUGL_API cugl_status cugl_conv2d_plan_bind_temp(cugl_conv_plan *plan, void *d_ws, size_t bytes);
/* as cugl_gemmlowp_plan_set_saturating_pack, for every lowering of the convolution */
CUGL_API cugl_status cugl_conv2d_plan_set_saturating_pack(cugl_conv_plan *plan, int on);
/* Fused residual addition: dst = act(quantize(dequantize(conv) + dequantize(residual))) computed in the epilogue
 * of the convolution, i.e. NEGEMMConvolutionLayer followed by NEArithmeticAddition (ConvertPolicy::SATURATE)
 * and NEActivationLayer (arm_compute/runtime/NEON/functions/NEArithmeticAddition.h:43-109) without the
 * intermediate tensors.  conv_out_scale with the plan's dst_zero_point is the quantization the convolution
 * requantizes to; dst_scale / dst_zero_point that of the sum.  QASYMM8 only.  The library enumerates all 65536
 * input pairs with the reference arithmetic and accepts the configuration when the addition is a saturating
 * byte addition followed by a clamp (always so when the three quantizations are equal); otherwise
 * CUGL_UNSUPPORTED_CONFIG is returned and the caller runs cugl_add_qasymm8 after cugl_conv2d_run. */
CUGL_API cugl_status cugl_conv2d_plan_set_residual(cugl_conv_plan *plan, float conv_out_scale, float residual_scale,
                                                   int32_t residual_zero_point, float dst_scale,
                                                   int32_t dst_zero_point, int32_t activation, float act_a,
                                                   float act_b);
/* residual and dst are [B][Ho][Wo][OFM]; they may be the same buffer. */
CUGL_API cugl_status cugl_conv2d_run_residual(cugl_conv_plan *plan, const void *d_src, const int32_t *d_bias,
                                              const void *d_residual, void *d_dst);

/* ------------------------------------------------------------------------------------------------
 * QASYMM8 layers between the convolutions of a quantized network (uint8, NHWC).  Each one computes what
 * Compute Library's scalar oracle computes: dequantize ((q - zero_point) * scale), float operator,
 * quantize (lround(v / scale) + zero_point, clamped to [0, 255]); results are identical to it bit for bit
 * except softmax (expf: within +-1, the tolerance of the reference's own tests).
 *   pooling     NEPoolingLayer          arm_compute/runtime/NEON/functions/NEPoolingLayer.h:48-109;
 *                                       oracle tests/validation/reference/PoolingLayer.cpp:40-196, 218-230
 *   addition    NEArithmeticAddition    arm_compute/runtime/NEON/functions/NEArithmeticAddition.h:43-109;
 *                                       oracle tests/validation/reference/ArithmeticOperations.cpp:124-151
 *   activation  NEActivationLayer       arm_compute/runtime/NEON/functions/NEActivationLayer.h:48-107;
 *                                       oracle tests/validation/reference/ActivationLayer.cpp:61-71
 *   softmax     NESoftmaxLayer          arm_compute/runtime/NEON/functions/NESoftmaxLayer.h:44-99;
 *                                       oracle tests/validation/reference/SoftmaxLayer.cpp:39-107, 201-213
 * ---------------------------------------------------------------------------------------------- */
typedef enum cugl_pool_type
{
    CUGL_POOL_MAX = 0,
    CUGL_POOL_AVG = 1
} cugl_pool_type;

typedef enum cugl_activation
{
    CUGL_ACT_NONE            = -1,
    CUGL_ACT_RELU            = 0, /* max(0, x)           */
    CUGL_ACT_BOUNDED_RELU    = 1, /* min(a, max(0, x))   */
    CUGL_ACT_LU_BOUNDED_RELU = 2  /* min(a, max(b, x))   */
} cugl_activation;

typedef struct cugl_pool_desc
{
    int32_t B, H, W, C;               /* src [B][H][W][C] */
    int32_t pool_type;                /* cugl_pool_type */
    int32_t pool_w, pool_h;
    int32_t stride_x, stride_y;
    int32_t pad_left, pad_right, pad_top, pad_bottom;
    int32_t exclude_padding;          /* AVG: divide by the in-image window area only */
    int32_t is_global;                /* window = whole image; pool_*, stride_*, pad_* ignored */
    float   src_scale;
    int32_t src_zero_point;
    float   dst_scale;
    int32_t dst_zero_point;
} cugl_pool_desc;

/* FLOOR rounding of the output size, as arm_compute::scaled_dimensions. */
CUGL_API void cugl_pool2d_out_dims(const cugl_pool_desc *desc, int32_t *Wo, int32_t *Ho);
CUGL_API cugl_status cugl_pool2d_validate(const cugl_pool_desc *desc);
/* dst is [B][Ho][Wo][C]. */
CUGL_API cugl_status cugl_pool2d_nhwc(cugl_context *ctx, const cugl_pool_desc *desc, const void *d_src, void *d_dst);

/* dst[i] = act(quantize(dequantize(a[i]) + dequantize(b[i]))) over n elements (ConvertPolicy::SATURATE).  The
 * activation (CUGL_ACT_NONE for none) acts on the quantized sum exactly as a separate NEActivationLayer with
 * equal input and output quantization would.  a_scale / b_scale must lie within 2^-20 .. 2^20. */
CUGL_API cugl_status cugl_add_qasymm8(cugl_context *ctx, const void *d_a, const void *d_b, void *d_dst, int64_t n,
                                      float a_scale, int32_t a_zero_point, float b_scale, int32_t b_zero_point,
                                      float dst_scale, int32_t dst_zero_point, int32_t activation, float act_a,
                                      float act_b);
CUGL_API cugl_status cugl_activation_qasymm8(cugl_context *ctx, const void *d_src, void *d_dst, int64_t n,
                                             int32_t activation, float act_a, float act_b, float src_scale,
                                             int32_t src_zero_point, float dst_scale, int32_t dst_zero_point);
/* rows x cols, contiguous rows; softmax along a row; output quantization is fixed at (1/256, 0). */
CUGL_API cugl_status cugl_softmax_qasymm8(cugl_context *ctx, const void *d_src, void *d_dst, int32_t rows, int32_t cols,
                                          float beta, float src_scale, int32_t src_zero_point);

#ifdef __cplusplus
}
#endif
#endif /* CUGL_H */
