#include "arm_compute/runtime/CUDA/CUScheduler.h"

#include <string>

namespace arm_compute
{
Status cu_status(cugl_status s, cugl_context *ctx, const char *where)
{
    if (s == CUGL_SUCCESS)
    {
        return Status{};
    }
    const char *msg = cugl_last_error_string(ctx);
    return Status(ErrorCode::RUNTIME_ERROR, std::string(where) + ": " + (msg != nullptr ? msg : "") + " (cugl status " +
                                                std::to_string(static_cast<int>(s)) + ")");
}

CUScheduler &CUScheduler::get()
{
    static CUScheduler instance;
    return instance;
}

void CUScheduler::default_init(int device, void *stream)
{
    if (_ctx != nullptr)
    {
        return;
    }
    cugl_context *ctx = nullptr;
    const cugl_status s = cugl_context_create(device, stream != nullptr ? stream : CUGL_STREAM_CREATE, &ctx);
    CU_THROW_ON(cu_status(s, nullptr, "CUScheduler::default_init"));
    _ctx = ctx;
}

cugl_context *CUScheduler::context()
{
    if (_ctx == nullptr)
    {
        default_init();
    }
    return _ctx;
}

void CUScheduler::sync()
{
    CU_THROW_ON(cu_status(cugl_sync(context()), _ctx, "CUScheduler::sync"));
}

CUScheduler::~CUScheduler()
{
    if (_ctx != nullptr)
    {
        cugl_context_destroy(_ctx);
        _ctx = nullptr;
    }
}
} // namespace arm_compute
