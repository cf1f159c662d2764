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
} // namespace arm_compute
