#include "arm_compute/runtime/CUDA/CUTensor.h"

#include "arm_compute/runtime/CUDA/CUScheduler.h"

namespace arm_compute
{
CUTensorAllocator::~CUTensorAllocator()
{
    try
    {
        free();
    }
    catch (...)
    {
    }
}

void CUTensorAllocator::init(const TensorInfo &input, size_t alignment)
{
    ARM_COMPUTE_UNUSED(alignment); // cudaMalloc regions are 256-byte aligned
    _info = input;
}

void CUTensorAllocator::allocate()
{
    ARM_COMPUTE_ERROR_ON_MSG(_device != nullptr, "CUTensorAllocator: already allocated");
    cugl_context *ctx = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_malloc(ctx, _info.total_size(), &_device), ctx, "CUTensorAllocator::allocate"));
    _owns = true;
}

void CUTensorAllocator::import_memory(void *device_ptr)
{
    ARM_COMPUTE_ERROR_ON_MSG(_device != nullptr, "CUTensorAllocator: already allocated");
    _device = device_ptr;
    _owns   = false;
}

void CUTensorAllocator::free()
{
    cugl_context *ctx = CUScheduler::get().is_initialised() ? CUScheduler::get().context() : nullptr;
    if (ctx != nullptr)
    {
        if (_host != nullptr)
        {
            cugl_sync(ctx);
            cugl_host_free(ctx, _host);
        }
        if (_device != nullptr && _owns)
        {
            cugl_sync(ctx);
            cugl_free(ctx, _device);
        }
    }
    _host   = nullptr;
    _device = nullptr;
    _owns = _mapped = false;
}

uint8_t *CUTensorAllocator::map(bool blocking)
{
    ARM_COMPUTE_ERROR_ON_MSG(_device == nullptr, "CUTensor::map: tensor is not allocated");
    cugl_context *ctx = CUScheduler::get().context();
    if (_host == nullptr)
    {
        void *p = nullptr;
        ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_host_alloc(ctx, _info.total_size(), &p), ctx, "CUTensor::map"));
        _host = static_cast<uint8_t *>(p);
    }
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_memcpy_d2h(ctx, _host, _device, _info.total_size()), ctx, "CUTensor::map"));
    if (blocking)
    {
        ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUTensor::map"));
    }
    _mapped = true;
    return _host;
}

void CUTensorAllocator::unmap()
{
    ARM_COMPUTE_ERROR_ON_MSG(!_mapped, "CUTensor::unmap: tensor is not mapped");
    cugl_context *ctx = CUScheduler::get().context();
    ARM_COMPUTE_ERROR_THROW_ON(cu_status(cugl_memcpy_h2d(ctx, _device, _host, _info.total_size()), ctx, "CUTensor::unmap"));
    _mapped = false;
}

void *cu_device_ptr(const ITensor *t)
{
    if (t == nullptr)
    {
        return nullptr;
    }
    const auto *cu = dynamic_cast<const CUTensor *>(t);
    ARM_COMPUTE_ERROR_ON_MSG(cu == nullptr, "CUDA functions take CUTensor operands (device memory)");
    ARM_COMPUTE_ERROR_ON_MSG(cu->device_ptr() == nullptr, "CUTensor operand is not allocated");
    return cu->device_ptr();
}
} // namespace arm_compute
