// Fused GEMMLowp for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a real-time inference loop that has
// already handed all device memory to its own arena, a plugin loaded into a process whose allocator the
// plugin does not own, or code running between the begin and end of a stream capture, where an
// allocation is an error.  The planned entry points (cugl_gemmlowp_plan_create / prepare / run) allocate
// their workspace -- the K-major copy of B, its column sums, the row sums of A -- with cudaMalloc.  The
// entry point in this file takes that workspace from a fixed array that is part of the loaded library
// image instead, so nothing is allocated by the call, at the price of a size limit.
#include "kernels.cuh"

#include <climits>
#include <mutex>

namespace
{
// Limits of the fixed workspace.  Every GPU that loads the library holds kScratchBytes (about 4.3 MB)
// until the process exits.
constexpr int64_t kMaxBtBytes = 4ll << 20; // N * round_up(K, 128) <= 4 MiB
constexpr int     kMaxN       = 8192;
constexpr int     kMaxM       = 65536;
constexpr int64_t kOffColsum  = kMaxBtBytes;
constexpr int64_t kOffRowsum  = kOffColsum + 4ll * kMaxN;
constexpr int64_t kOffStatus  = kOffRowsum + 4ll * kMaxM;
constexpr int64_t kScratchBytes = kOffStatus + 256;

// In host code this name is only a handle for the runtime, not an address a kernel could use:
// the device address is looked up once per device with cudaGetSymbolAddress (below).
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

struct DeviceSetup
{
    bool           ready    = false;
    unsigned char *scratch  = nullptr; // device address of g_scratch on this device
    int            sm_count = 0;
};
DeviceSetup g_setup[64];
std::mutex  g_setup_mutex;

inline int64_t round_up128(int64_t v)
{
    return (v + 127) / 128 * 128;
}
} // namespace

extern "C" cugl_status cugl_gemmlowp_run_noalloc(void *stream, const cugl_gemm_desc *desc, const void *d_a,
                                                 const void *d_b, const int32_t *d_bias,
                                                 const int32_t *d_multipliers, const int32_t *d_shifts,
                                                 void *d_dst)
{
    using namespace cugl;
    // the per-channel vectors are device memory here: the h_ pointers of desc are neither needed nor read
    cugl_status code = CUGL_SUCCESS;
    const char *why  = validate_gemm_desc(desc, &code, false);
    if (why != nullptr)
    {
        return fail(nullptr, code, std::string("cugl_gemmlowp_run_noalloc: ") + why);
    }
    if (d_a == nullptr || d_b == nullptr || d_dst == nullptr)
    {
        return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_noalloc: NULL operand");
    }
    if (desc->batch != 1)
    {
        return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_noalloc: batch must be 1");
    }
    const bool per_channel = desc->stage != CUGL_STAGE_NONE && desc->is_quantized_per_channel != 0;
    if (per_channel && (d_multipliers == nullptr || d_shifts == nullptr))
    {
        return fail(nullptr, CUGL_INVALID_ARGUMENT,
                    "cugl_gemmlowp_run_noalloc: per-channel stage needs DEVICE vectors of N multipliers and shifts");
    }
    if (desc->has_bias && d_bias == nullptr)
    {
        return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_gemmlowp_run_noalloc: descriptor announces a bias");
    }
    const int64_t ldbt = round_up128(desc->K);
    if (desc->N > kMaxN || desc->M > kMaxM || ldbt * desc->N > kMaxBtBytes)
    {
        return fail(nullptr, CUGL_INVALID_ARGUMENT,
                    "cugl_gemmlowp_run_noalloc: problem exceeds the fixed workspace (limits: M <= 65536, N <= 8192, "
                    "N * round_up(K, 128) <= 4 MiB); use the planned entry points instead");
    }

    int device = 0;
    CUGL_CUDA_TRY(nullptr, cudaGetDevice(&device));
    if (device < 0 || device >= 64)
    {
        return fail(nullptr, CUGL_UNSUPPORTED_CONFIG, "cugl_gemmlowp_run_noalloc: device index above 63");
    }
    {
        // One-time set-up per device, with that device current: resolve the device address of the array.
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        DeviceSetup                &su = g_setup[device];
        if (!su.ready)
        {
            void *p = nullptr;
            CUGL_CUDA_TRY(nullptr, cudaGetSymbolAddress(&p, g_scratch));
            CUGL_CUDA_TRY(nullptr, cudaDeviceGetAttribute(&su.sm_count, cudaDevAttrMultiProcessorCount, device));
            su.scratch = static_cast<unsigned char *>(p);
            // the status word the kernels may write must start at zero; blocking, so that it is clear for every
            // stream and not only for the one this first call happens to use
            CUGL_CUDA_TRY(nullptr, cudaMemset(su.scratch + kOffStatus, 0, 256));
            su.ready = true;
        }
    }
    const DeviceSetup &su = g_setup[device];

    // A context object on the stack gives the kernel launchers their stream; nothing in it is allocated.
    cugl_context ctx;
    ctx.device   = device;
    ctx.sm_count = su.sm_count;
    ctx.stream   = static_cast<cudaStream_t>(stream);
    ctx.d_status = reinterpret_cast<int32_t *>(su.scratch + kOffStatus);

    uint8_t *d_bt     = su.scratch;
    int32_t *d_colsum = reinterpret_cast<int32_t *>(su.scratch + kOffColsum);
    int32_t *d_rowsum = reinterpret_cast<int32_t *>(su.scratch + kOffRowsum);
    const bool a_signed = desc->a_dtype == CUGL_S8, b_signed = desc->b_dtype == CUGL_S8;

    // B -> K-major copy + column sums (the launcher zeroes the sums first: they accumulate with atomics and
    // the array still holds the previous call's values)
    CUGL_TRY(launch_transpose_colsum(&ctx, d_b, b_signed, desc->K, desc->N, desc->ldb, d_bt, ldbt, d_colsum));
    if (desc->b_offset != 0)
    {
        CUGL_TRY(launch_reduce_rows(&ctx, d_a, a_signed, desc->M, desc->K, desc->lda, 1, d_rowsum));
    }

    EpilogueParams ep{};
    ep.colsum = desc->a_offset != 0 ? d_colsum : nullptr;
    ep.rowsum = desc->b_offset != 0 ? d_rowsum : nullptr;
    ep.bias   = desc->has_bias ? d_bias : nullptr;
    ep.mults  = per_channel ? d_multipliers : nullptr;
    ep.shifts = per_channel ? d_shifts : nullptr;
    ep.mult   = desc->gemmlowp_multiplier;
    ep.shift  = desc->gemmlowp_shift;
    ep.a_off  = desc->a_offset;
    ep.b_off  = desc->b_offset;
    ep.k_term = (desc->a_offset != 0 && desc->b_offset != 0)
                    ? static_cast<int32_t>(static_cast<uint32_t>(desc->a_offset) *
                                           static_cast<uint32_t>(desc->b_offset) * static_cast<uint32_t>(desc->K))
                    : 0;
    ep.result_offset  = desc->gemmlowp_offset;
    const int32_t tlo = desc->dst_dtype == CUGL_S8 ? -128 : 0, thi = desc->dst_dtype == CUGL_S8 ? 127 : 255;
    ep.lo             = desc->gemmlowp_min_bound > tlo ? desc->gemmlowp_min_bound : tlo;
    ep.hi             = desc->gemmlowp_max_bound < thi ? desc->gemmlowp_max_bound : thi;
    if (desc->stage == CUGL_STAGE_QUANTIZE_DOWN && desc->gemmlowp_min_bound == desc->gemmlowp_max_bound)
    {
        ep.lo = tlo; // equal bounds: no bounded ReLU, type range only
        ep.hi = thi;
    }
    ep.stage          = desc->stage;
    ep.out_signed     = desc->dst_dtype == CUGL_S8;
    ep.out_f32        = desc->dst_dtype == CUGL_F32 ? 1 : 0;
    ep.accumulate     = desc->accumulate != 0 ? 1 : 0;
    ep.dq_scale       = desc->dequantize_scale;

    GemmOperands op{};
    op.a        = d_a;
    op.bt       = d_bt;
    op.dst      = d_dst;
    op.lda      = desc->lda;
    op.ldbt     = ldbt;
    op.ldd      = desc->ldd;
    op.M        = desc->M;
    op.N        = desc->N;
    op.K        = desc->K;
    op.a_signed = a_signed;
    op.b_signed = b_signed;
    // the per-channel vectors live on the device only, so their signs cannot be inspected here:
    // take the fully general output-stage path for them
    op.generic_stage = per_channel || desc->gemmlowp_shift < 0 || desc->gemmlowp_multiplier == INT32_MIN ||
                       desc->stage == CUGL_STAGE_QUANTIZE_DOWN;
    return gemmlowp_tcgen05_supported(op) ? launch_gemmlowp_tcgen05(&ctx, op, ep, true)
                                          : launch_gemmlowp_simt(&ctx, op, ep);
}

// The tensor-core kernels bound every wait; when one runs out they record which role gave up in a status word
// inside the fixed array and return.  The planned entry points report that word through cugl_sync; this path
// has no context, so the word is read here: waits for `stream`, copies the word to the host, clears it for
// the next call and answers CUGL_RUNTIME_ERROR when it was set (dst of the affected call is then invalid).
// Allocates nothing.
extern "C" cugl_status cugl_gemmlowp_noalloc_status(void *stream)
{
    using namespace cugl;
    int device = 0;
    CUGL_CUDA_TRY(nullptr, cudaGetDevice(&device));
    unsigned char *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (device < 0 || device >= 64 || !g_setup[device].ready)
        {
            return CUGL_SUCCESS; // nothing has run on this device yet
        }
        scratch = g_setup[device].scratch;
    }
    cudaStream_t st   = static_cast<cudaStream_t>(stream);
    int32_t      word = 0;
    CUGL_CUDA_TRY(nullptr, cudaMemcpyAsync(&word, scratch + kOffStatus, sizeof(word), cudaMemcpyDeviceToHost, st));
    CUGL_CUDA_TRY(nullptr, cudaStreamSynchronize(st));
    if (word == 0)
    {
        return CUGL_SUCCESS;
    }
    CUGL_CUDA_TRY(nullptr, cudaMemsetAsync(scratch + kOffStatus, 0, sizeof(word), st));
    CUGL_CUDA_TRY(nullptr, cudaStreamSynchronize(st));
    return fail(nullptr, CUGL_RUNTIME_ERROR,
                "cugl_gemmlowp_run_noalloc: a bounded device wait ran out (role code " + std::to_string(word) +
                    ": 1 producer, 2 MMA issuer, 3 epilogue, 4 drain); the output of that call is invalid");
}
