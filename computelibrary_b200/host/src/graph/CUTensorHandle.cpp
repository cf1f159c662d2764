#include "arm_compute/graph/backends/CUDA/CUTensorHandle.h"

#include "arm_compute/graph/backends/CUDA/CUDeviceBackend.h"
#include "arm_compute/runtime/IMemoryGroup.h"

namespace arm_compute
{
namespace graph
{
namespace backends
{
CUTensorHandle::CUTensorHandle(const ITensorInfo &info) : _tensor()
{
    _tensor.allocator()->init(info);
}

void CUTensorHandle::allocate()
{
    _tensor.allocator()->allocate();
}

void CUTensorHandle::free()
{
    _tensor.allocator()->free();
}

void CUTensorHandle::manage(IMemoryGroup *mg)
{
    if (mg != nullptr)
    {
        mg->manage(&_tensor);
    }
}

void CUTensorHandle::map(bool blocking)
{
    _tensor.map(blocking);
}

void CUTensorHandle::unmap()
{
    _tensor.unmap();
}

void CUTensorHandle::release_if_unused()
{
    if (!_tensor.is_used())
    {
        _tensor.allocator()->free();
    }
}

arm_compute::ITensor &CUTensorHandle::tensor()
{
    return _tensor;
}

const arm_compute::ITensor &CUTensorHandle::tensor() const
{
    return _tensor;
}

ITensorHandle *CUTensorHandle::parent_handle()
{
    return this;
}

bool CUTensorHandle::is_subtensor() const
{
    return false;
}

Target CUTensorHandle::target() const
{
    return CUDATarget;
}
} // namespace backends
} // namespace graph
} // namespace arm_compute
