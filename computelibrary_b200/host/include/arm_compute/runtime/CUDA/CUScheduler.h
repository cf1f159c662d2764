// One device + one stream: the role NEScheduler / CLScheduler play for their backends
// (arm_compute/runtime/IScheduler.h:144-211, CLScheduler::sync).  Work is enqueued, sync() blocks.
#pragma once
#include "arm_compute/core/Error.h"
#include "cugl.h"

namespace arm_compute
{
class CUScheduler
{
public:
    static CUScheduler &get();
    // device: CUDA ordinal; stream: cudaStream_t to share with the caller, or nullptr for a stream of its own.
    void          default_init(int device = 0, void *stream = nullptr);
    bool          is_initialised() const { return _ctx != nullptr; }
    cugl_context *context();
    void          sync();
    ~CUScheduler();

private:
    CUScheduler() = default;
    cugl_context *_ctx{nullptr};
};

// cugl status -> arm_compute::Status (text from cugl_last_error_string)
Status cu_status(cugl_status s, cugl_context *ctx, const char *where);

// ARM_COMPUTE_ERROR_THROW_ON / ARM_COMPUTE_ERROR_ON_MSG are compiled out of builds without asserts
// (arm_compute/core/Error.h:407-460) together with their argument.  Calls into the C ABI have side effects and CUDA
// errors must surface in every build, so the CUDA functions use these always-active forms.
#define CU_THROW_ON(status) (status).throw_if_error()
#define CU_ERROR_IF(cond, msg)      \
    do                              \
    {                               \
        if (cond)                   \
        {                           \
            ARM_COMPUTE_ERROR(msg); \
        }                           \
    } while (0)
} // namespace arm_compute
