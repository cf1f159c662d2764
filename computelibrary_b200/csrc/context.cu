// Context, device memory and stream entry points of the cugl C ABI: the CUDA counterpart of the host
// TensorAllocator / IAllocator / scheduler trio the NE functions sit on.
#include "common.cuh"

#include <cmath>
#include <cstring>
#include <mutex>

namespace
{
std::mutex  g_err_mutex;
std::string g_last_error = "";
} // namespace

namespace cugl
{
void set_global_error(const std::string &msg)
{
    std::lock_guard<std::mutex> lock(g_err_mutex);
    g_last_error = msg;
}

cugl_status fail(cugl_context *ctx, cugl_status code, const std::string &msg)
{
    if (ctx != nullptr)
    {
        ctx->last_error = msg;
    }
    set_global_error(msg);
    return code;
}

cugl_status check_cuda(cugl_context *ctx, cudaError_t e, const char *what)
{
    if (e == cudaSuccess)
    {
        return CUGL_SUCCESS;
    }
    const cugl_status code = (e == cudaErrorMemoryAllocation) ? CUGL_OUT_OF_MEMORY : CUGL_RUNTIME_ERROR;
    return fail(ctx, code, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}
} // namespace cugl

using cugl::check_cuda;
using cugl::fail;

extern "C"
{
    cugl_status cugl_context_create(int device, void *stream, cugl_context **out)
    {
        if (out == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_context_create: out is NULL");
        }
        *out      = nullptr;
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
        {
            (void)cudaGetLastError();
            return fail(nullptr, CUGL_UNSUPPORTED_TARGET,
                        "cugl_context_create: no CUDA device is visible; this backend has no CPU fallback");
        }
        if (device < 0 || device >= count)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_context_create: device index out of range");
        }
        cudaDeviceProp prop{};
        CUGL_CUDA_TRY(nullptr, cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
        {
            return fail(nullptr, CUGL_UNSUPPORTED_TARGET,
                        std::string("cugl_context_create: device '") + prop.name +
                            "' is not an sm_100 part; the kernels are built for sm_100a only");
        }
        CUGL_CUDA_TRY(nullptr, cudaSetDevice(device));
        auto *ctx     = new cugl_context();
        ctx->device   = device;
        ctx->sm_count = prop.multiProcessorCount;
        if (stream != CUGL_STREAM_CREATE)
        {
            ctx->stream = static_cast<cudaStream_t>(stream);
        }
        else
        {
            cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
            if (e != cudaSuccess)
            {
                delete ctx;
                return check_cuda(nullptr, e, "cudaStreamCreateWithFlags");
            }
            ctx->owns_stream = true;
        }
        cudaError_t e = cudaMalloc(&ctx->d_status, sizeof(int32_t));
        if (e == cudaSuccess)
        {
            e = cudaMemset(ctx->d_status, 0, sizeof(int32_t));
        }
        if (e == cudaSuccess)
        {
            e = cudaMallocHost(&ctx->h_status, sizeof(int32_t));
        }
        if (e != cudaSuccess)
        {
            cugl_context_destroy(ctx);
            return check_cuda(nullptr, e, "context status word");
        }
        *ctx->h_status = 0;
        *out           = ctx;
        return CUGL_SUCCESS;
    }

    void cugl_context_destroy(cugl_context *ctx)
    {
        if (ctx == nullptr)
        {
            return;
        }
        cudaSetDevice(ctx->device);
        if (ctx->d_status != nullptr)
        {
            cudaFree(ctx->d_status);
        }
        if (ctx->h_status != nullptr)
        {
            cudaFreeHost(ctx->h_status);
        }
        if (ctx->owns_stream && ctx->stream != nullptr)
        {
            cudaStreamDestroy(ctx->stream);
        }
        delete ctx;
    }

    const char *cugl_last_error_string(const cugl_context *ctx)
    {
        if (ctx != nullptr)
        {
            return ctx->last_error.c_str();
        }
        std::lock_guard<std::mutex> lock(g_err_mutex);
        static thread_local std::string copy;
        copy = g_last_error;
        return copy.c_str();
    }

    void *cugl_context_stream(const cugl_context *ctx)
    {
        return ctx != nullptr ? static_cast<void *>(ctx->stream) : nullptr;
    }
    int cugl_context_device(const cugl_context *ctx)
    {
        return ctx != nullptr ? ctx->device : -1;
    }
    int cugl_context_sm_count(const cugl_context *ctx)
    {
        return ctx != nullptr ? ctx->sm_count : 0;
    }

#define CUGL_NEED_CTX(ctx)                                                        \
    if ((ctx) == nullptr)                                                         \
    {                                                                             \
        return fail(nullptr, CUGL_INVALID_ARGUMENT, "context is NULL");           \
    }

    cugl_status cugl_malloc(cugl_context *ctx, size_t bytes, void **d_ptr)
    {
        CUGL_NEED_CTX(ctx);
        if (d_ptr == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_malloc: d_ptr is NULL");
        }
        *d_ptr = nullptr;
        if (bytes == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        CUGL_CUDA_TRY(ctx, cudaMalloc(d_ptr, bytes));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_free(cugl_context *ctx, void *d_ptr)
    {
        CUGL_NEED_CTX(ctx);
        if (d_ptr != nullptr)
        {
            CUGL_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
            CUGL_CUDA_TRY(ctx, cudaFree(d_ptr));
        }
        return CUGL_SUCCESS;
    }

    cugl_status cugl_host_alloc(cugl_context *ctx, size_t bytes, void **h_ptr)
    {
        CUGL_NEED_CTX(ctx);
        if (h_ptr == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_host_alloc: h_ptr is NULL");
        }
        *h_ptr = nullptr;
        if (bytes == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMallocHost(h_ptr, bytes));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_host_free(cugl_context *ctx, void *h_ptr)
    {
        CUGL_NEED_CTX(ctx);
        if (h_ptr != nullptr)
        {
            CUGL_CUDA_TRY(ctx, cudaFreeHost(h_ptr));
        }
        return CUGL_SUCCESS;
    }

    cugl_status cugl_memcpy_h2d(cugl_context *ctx, void *d_dst, const void *h_src, size_t bytes)
    {
        CUGL_NEED_CTX(ctx);
        if (bytes == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_memcpy_d2h(cugl_context *ctx, void *h_dst, const void *d_src, size_t bytes)
    {
        CUGL_NEED_CTX(ctx);
        if (bytes == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_memcpy_d2d(cugl_context *ctx, void *d_dst, const void *d_src, size_t bytes)
    {
        CUGL_NEED_CTX(ctx);
        if (bytes == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_memcpy2d_h2d(cugl_context *ctx, void *d_dst, size_t d_pitch, const void *h_src, size_t h_pitch,
                                  size_t width_bytes, size_t rows)
    {
        CUGL_NEED_CTX(ctx);
        if (width_bytes == 0 || rows == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMemcpy2DAsync(d_dst, d_pitch, h_src, h_pitch, width_bytes, rows,
                                             cudaMemcpyHostToDevice, ctx->stream));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_memcpy2d_d2h(cugl_context *ctx, void *h_dst, size_t h_pitch, const void *d_src, size_t d_pitch,
                                  size_t width_bytes, size_t rows)
    {
        CUGL_NEED_CTX(ctx);
        if (width_bytes == 0 || rows == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMemcpy2DAsync(h_dst, h_pitch, d_src, d_pitch, width_bytes, rows,
                                             cudaMemcpyDeviceToHost, ctx->stream));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_memset(cugl_context *ctx, void *d_ptr, int value, size_t bytes)
    {
        CUGL_NEED_CTX(ctx);
        if (bytes == 0)
        {
            return CUGL_SUCCESS;
        }
        CUGL_CUDA_TRY(ctx, cudaMemsetAsync(d_ptr, value, bytes, ctx->stream));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_context_set_trace_buffer(cugl_context *ctx, void *d_buffer)
    {
        CUGL_NEED_CTX(ctx);
        ctx->d_trace = static_cast<long long *>(d_buffer);
        return CUGL_SUCCESS;
    }

    cugl_status cugl_context_set_wait_limit_us(cugl_context *ctx, uint64_t microseconds)
    {
        CUGL_NEED_CTX(ctx);
        if (microseconds == 0)
        {
            ctx->spin_limit = cugl_context{}.spin_limit;
            return CUGL_SUCCESS;
        }
        int khz = 0; // clock64 counts SM clocks: convert at the device's peak rate, the limit is an upper bound
        CUGL_CUDA_TRY(ctx, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
        ctx->spin_limit = static_cast<long long>(microseconds) * khz / 1000;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_context_withhold_copy_once(cugl_context *ctx, int k_block)
    {
        CUGL_NEED_CTX(ctx);
        if (k_block < 0)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_context_withhold_copy_once: k_block must be >= 0");
        }
        ctx->withhold_kb = k_block;
        return CUGL_SUCCESS;
    }

    cugl_status cugl_context_set_dependent_launch(cugl_context *ctx, int on)
    {
        if (ctx == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "cugl_context_set_dependent_launch: NULL context");
        }
        ctx->dependent_launch = on != 0 ? 1 : 0;
        return CUGL_SUCCESS;
    }

    // ---- peer access to another process's device buffer (CUDA IPC) --------------------------------
    cugl_status cugl_ipc_get_handle(cugl_context *ctx, void *d_ptr, void *handle64)
    {
        CUGL_NEED_CTX(ctx);
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
        if (d_ptr == nullptr || handle64 == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_ipc_get_handle: NULL argument");
        }
        cudaIpcMemHandle_t h;
        CUGL_CUDA_TRY(ctx, cudaIpcGetMemHandle(&h, d_ptr));
        std::memcpy(handle64, &h, sizeof(h));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_ipc_open_handle(cugl_context *ctx, const void *handle64, void **d_ptr)
    {
        CUGL_NEED_CTX(ctx);
        if (handle64 == nullptr || d_ptr == nullptr)
        {
            return fail(ctx, CUGL_INVALID_ARGUMENT, "cugl_ipc_open_handle: NULL argument");
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handle64, sizeof(h));
        CUGL_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        CUGL_CUDA_TRY(ctx, cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
        return CUGL_SUCCESS;
    }

    cugl_status cugl_ipc_close_handle(cugl_context *ctx, void *d_ptr)
    {
        CUGL_NEED_CTX(ctx);
        if (d_ptr != nullptr)
        {
            CUGL_CUDA_TRY(ctx, cudaIpcCloseMemHandle(d_ptr));
        }
        return CUGL_SUCCESS;
    }

    cugl_status cugl_sync(cugl_context *ctx)
    {
        CUGL_NEED_CTX(ctx);
        CUGL_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                           ctx->stream));
        CUGL_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        if (*ctx->h_status != 0)
        {
            const int32_t code = *ctx->h_status;
            *ctx->h_status     = 0;
            cudaMemsetAsync(ctx->d_status, 0, sizeof(int32_t), ctx->stream);
            cudaStreamSynchronize(ctx->stream);
            return fail(ctx, CUGL_RUNTIME_ERROR,
                        "device-side bounded wait ran out (code " + std::to_string(code) +
                            ": 1 = TMA producer, 2 = MMA issuer, 3 = epilogue, 4 = drain); results are invalid");
        }
        return CUGL_SUCCESS;
    }

    // ---- host-side quantisation helpers ---------------------------------------------------------
    // quantization::calculate_quantized_multiplier (AsymmHelpers.cpp:43-115): frexp on the promoted
    // double, round to Q0.31, renormalise when the mantissa rounds up to 1.0.
    cugl_status cugl_calculate_quantized_multiplier(float multiplier, int32_t *quant_multiplier, int32_t *shift)
    {
        if (quant_multiplier == nullptr || shift == nullptr)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "calculate_quantized_multiplier: NULL output");
        }
        constexpr int64_t one_q31 = 1ll << 31;
        constexpr float   eps     = 0.00001f;
        int               exp     = 0;
        const double      q       = std::frexp(static_cast<double>(multiplier), &exp);
        int64_t           q_fixed = static_cast<int64_t>(std::llround(q * static_cast<double>(one_q31)));
        if (q_fixed > one_q31)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "calculate_quantized_multiplier: mantissa out of range");
        }
        int sh;
        if (multiplier >= 1.f)
        {
            sh = exp; // left shift
            if (q_fixed == one_q31)
            {
                q_fixed /= 2;
                ++sh;
            }
            if (sh < 0 || q_fixed > INT32_MAX)
            {
                return fail(nullptr, CUGL_INVALID_ARGUMENT, "calculate_quantized_multiplier: cannot represent");
            }
            *shift = -sh;
        }
        else
        {
            if (multiplier < -eps || multiplier > 1.0f + eps)
            {
                return fail(nullptr, CUGL_INVALID_ARGUMENT, "calculate_quantized_multiplier: multiplier < 0");
            }
            sh = -exp; // right shift
            if (q_fixed == one_q31)
            {
                q_fixed /= 2;
                --sh;
            }
            if (sh < 0 || q_fixed > INT32_MAX)
            {
                return fail(nullptr, CUGL_INVALID_ARGUMENT, "calculate_quantized_multiplier: cannot represent");
            }
            *shift = sh;
        }
        *quant_multiplier = static_cast<int32_t>(q_fixed);
        return CUGL_SUCCESS;
    }

    cugl_status cugl_calculate_quantized_multipliers(float i_scale, const float *w_scales, int n, float o_scale,
                                                     int32_t *multipliers, int32_t *shifts)
    {
        if (w_scales == nullptr || multipliers == nullptr || shifts == nullptr || n <= 0)
        {
            return fail(nullptr, CUGL_INVALID_ARGUMENT, "calculate_quantized_multipliers: bad argument");
        }
        for (int i = 0; i < n; ++i)
        {
            const float m = i_scale * w_scales[i] / o_scale; // float32, in this order (AsymmHelpers.cpp:139)
            CUGL_TRY(cugl_calculate_quantized_multiplier(m, &multipliers[i], &shifts[i]));
        }
        return CUGL_SUCCESS;
    }
}
