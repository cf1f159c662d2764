// Private helpers shared by the CUDA function family.
#pragma once
#include "arm_compute/core/ITensorInfo.h"
#include "arm_compute/core/Types.h"
#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"
#include "arm_compute/runtime/MemoryGroup.h"

namespace arm_compute
{
namespace cu
{
inline int32_t to_cugl_dtype(DataType dt)
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
        case DataType::QSYMM16:
            return CUGL_S16;
        case DataType::F32:
            return CUGL_F32;
        default:
            return -1;
    }
}

// every dimension follows the one below it without gaps (padding in x or y breaks this)
inline bool is_dense(const ITensorInfo &ti)
{
    size_t expect = ti.element_size();
    for (size_t i = 0; i < ti.num_dimensions(); ++i)
    {
        if (ti.strides_in_bytes()[i] != expect)
        {
            return false;
        }
        expect *= ti.dimension(i);
    }
    return true;
}

// A U8 device tensor of `bytes` bytes whose lifetime the function's memory group manages: the protocol of
// manage_workspace (src/core/helpers/MemoryHelpers.h:56-105) for one slot of lifetime Temporary.  With a memory
// manager the bytes come from the manager's pool between acquire() and release(); without one they are the
// tensor's own.
class TemporaryWorkspace
{
public:
    void configure(MemoryGroup &group, size_t bytes)
    {
        if (_bytes != 0 || bytes == 0)
        {
            return; // nothing to hold, or configured before (a function configured twice keeps its first workspace)
        }
        _bytes = bytes;
        _tensor.allocator()->init(TensorInfo(TensorShape(bytes), 1, DataType::U8), 256);
        group.manage(&_tensor);
        _tensor.allocator()->allocate(); // ends the lifetime: a managed tensor only records its size here
    }
    size_t bytes() const { return _bytes; }
    void  *device_ptr() const { return _bytes != 0 ? _tensor.device_ptr() : nullptr; }

private:
    CUTensor _tensor{};
    size_t   _bytes{0};
};
} // namespace cu
} // namespace arm_compute
