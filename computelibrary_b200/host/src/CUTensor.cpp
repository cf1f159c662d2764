#include "arm_compute/runtime/CUDA/CUTensor.h"

#include "arm_compute/core/Error.h"
#include "arm_compute/runtime/CUDA/CUAllocator.h"
#include "arm_compute/runtime/CUDA/CUScheduler.h"

#include <utility>

namespace arm_compute
{
// ---------------------------------------------------------------------------------------------- allocator
CUTensorAllocator::CUTensorAllocator(IMemoryManageable *owner) : _owner(owner)
{
}

CUTensorAllocator::~CUTensorAllocator()
{
    release_host();
    info().set_is_resizable(true);
}

CUTensorAllocator::CUTensorAllocator(CUTensorAllocator &&o) noexcept
    : ITensorAllocator(std::move(o)),
      _owner(o._owner),
      _associated_memory_group(o._associated_memory_group),
      _memory(std::move(o._memory)),
      _host(o._host),
      _host_bytes(o._host_bytes),
      _mapped(o._mapped)
{
    o._owner                   = nullptr;
    o._associated_memory_group = nullptr;
    o._memory                  = Memory();
    o._host                    = nullptr;
    o._host_bytes              = 0;
    o._mapped                  = false;
}

CUTensorAllocator &CUTensorAllocator::operator=(CUTensorAllocator &&o) noexcept
{
    if (&o != this)
    {
        release_host();
        _owner                     = o._owner;
        _associated_memory_group   = o._associated_memory_group;
        _memory                    = std::move(o._memory);
        _host                      = o._host;
        _host_bytes                = o._host_bytes;
        _mapped                    = o._mapped;
        o._owner                   = nullptr;
        o._associated_memory_group = nullptr;
        o._memory                  = Memory();
        o._host                    = nullptr;
        o._host_bytes              = 0;
        o._mapped                  = false;
        ITensorAllocator::operator=(std::move(o));
    }
    return *this;
}

void *CUTensorAllocator::device_ptr() const
{
    return _memory.region() == nullptr ? nullptr : _memory.region()->buffer();
}

void CUTensorAllocator::allocate()
{
    // cudaMalloc blocks are 256-byte aligned; a managed tensor gets its bytes from the group's pool at acquire()
    const size_t alignment_to_use = alignment() != 0 ? alignment() : 256;
    if (_associated_memory_group == nullptr)
    {
        CU_ERROR_IF(_memory.region() != nullptr && _memory.region()->buffer() != nullptr,
                                 "CUTensorAllocator: already allocated");
        _memory.set_owned_region(std::make_unique<CUMemoryRegion>(info().total_size(), alignment_to_use));
    }
    else
    {
        _associated_memory_group->finalize_memory(_owner, _memory, info().total_size(), alignment_to_use);
    }
    info().set_is_resizable(false);
}

void CUTensorAllocator::free()
{
    release_host();
    _memory.set_region(nullptr);
    info().set_is_resizable(true);
}

bool CUTensorAllocator::is_allocated() const
{
    return _memory.region() != nullptr;
}

Status CUTensorAllocator::import_memory(void *device_ptr)
{
    ARM_COMPUTE_RETURN_ERROR_ON(device_ptr == nullptr);
    ARM_COMPUTE_RETURN_ERROR_ON(_associated_memory_group != nullptr);
    _memory.set_owned_region(std::make_unique<CUMemoryRegion>(device_ptr, info().total_size()));
    info().set_is_resizable(false);
    return Status{};
}

void CUTensorAllocator::set_associated_memory_group(IMemoryGroup *associated_memory_group)
{
    ARM_COMPUTE_ERROR_ON(associated_memory_group == nullptr);
    ARM_COMPUTE_ERROR_ON(_associated_memory_group != nullptr && _associated_memory_group != associated_memory_group);
    ARM_COMPUTE_ERROR_ON(_memory.region() != nullptr && _memory.region()->buffer() != nullptr);
    _associated_memory_group = associated_memory_group;
}

uint8_t *CUTensorAllocator::map(bool blocking)
{
    void *dev = device_ptr();
    CU_ERROR_IF(dev == nullptr, "CUTensor::map: tensor is not allocated");
    cugl_context *ctx   = CUScheduler::get().context();
    const size_t  bytes = info().total_size();
    if (_host == nullptr || _host_bytes < bytes)
    {
        release_host();
        void *p = nullptr;
        CU_THROW_ON(cu_status(cugl_host_alloc(ctx, bytes > 0 ? bytes : 1, &p), ctx, "CUTensor::map"));
        _host       = static_cast<uint8_t *>(p);
        _host_bytes = bytes;
    }
    CU_THROW_ON(cu_status(cugl_memcpy_d2h(ctx, _host, dev, bytes), ctx, "CUTensor::map"));
    if (blocking)
    {
        CU_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUTensor::map"));
    }
    _mapped = true;
    return _host;
}

void CUTensorAllocator::unmap()
{
    CU_ERROR_IF(!_mapped, "CUTensor::unmap: tensor is not mapped");
    cugl_context *ctx = CUScheduler::get().context();
    CU_THROW_ON(cu_status(cugl_memcpy_h2d(ctx, device_ptr(), _host, info().total_size()), ctx, "CUTensor::unmap"));
    // the pinned mirror may be reused or released right away: wait for the copy
    CU_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUTensor::unmap"));
    _mapped = false;
}

uint8_t *CUTensorAllocator::lock()
{
    return map(true);
}

void CUTensorAllocator::unlock()
{
    unmap();
}

void CUTensorAllocator::release_host()
{
    if (_host != nullptr && CUScheduler::get().is_initialised())
    {
        cugl_context *ctx = CUScheduler::get().context();
        cugl_sync(ctx);
        cugl_host_free(ctx, _host);
    }
    _host       = nullptr;
    _host_bytes = 0;
    _mapped     = false;
}

// ------------------------------------------------------------------------------------------------- tensor
CUTensor::CUTensor(IRuntimeContext *ctx) : _allocator(this)
{
    ARM_COMPUTE_UNUSED(ctx);
}

CUTensor::CUTensor(CUTensor &&o) noexcept : ITensor(std::move(o)), _allocator(std::move(o._allocator))
{
    _allocator.set_owner(this);
}

CUTensor &CUTensor::operator=(CUTensor &&o) noexcept
{
    if (&o != this)
    {
        ITensor::operator=(std::move(o));
        _allocator = std::move(o._allocator);
        _allocator.set_owner(this);
    }
    return *this;
}

ITensorInfo *CUTensor::info() const
{
    return &_allocator.info();
}

ITensorInfo *CUTensor::info()
{
    return &_allocator.info();
}

uint8_t *CUTensor::buffer() const
{
    return _allocator.mapping();
}

void *CUTensor::device_ptr() const
{
    void *base = _allocator.device_ptr();
    return base == nullptr ? nullptr : static_cast<uint8_t *>(base) + _allocator.info().offset_first_element_in_bytes();
}

void CUTensor::map(bool blocking)
{
    _allocator.map(blocking);
}

void CUTensor::unmap()
{
    _allocator.unmap();
}

void CUTensor::associate_memory_group(IMemoryGroup *memory_group)
{
    _allocator.set_associated_memory_group(memory_group);
}

void *cu_device_ptr(const ITensor *t)
{
    if (t == nullptr)
    {
        return nullptr;
    }
    const auto *cu = dynamic_cast<const CUTensor *>(t);
    CU_ERROR_IF(cu == nullptr, "this CUDA function takes CUTensor operands (device memory)");
    CU_ERROR_IF(cu->device_ptr() == nullptr, "CUTensor operand is not allocated");
    return cu->device_ptr();
}

// ------------------------------------------------------------------------------------------------ operand
CUOperand::~CUOperand()
{
    if (_stage != nullptr && CUScheduler::get().is_initialised())
    {
        cugl_context *ctx = CUScheduler::get().context();
        cugl_sync(ctx);
        cugl_free(ctx, _stage);
    }
}

bool CUOperand::is_device() const
{
    return dynamic_cast<const CUTensor *>(_tensor) != nullptr;
}

void *CUOperand::device(bool upload)
{
    if (_tensor == nullptr)
    {
        return nullptr;
    }
    if (const auto *cu = dynamic_cast<const CUTensor *>(_tensor))
    {
        void *p = cu->device_ptr();
        CU_ERROR_IF(p == nullptr, "CUTensor operand is not allocated");
        return p;
    }
    // a host tensor: mirror its buffer, padding and all, so that strides and offsets carry over unchanged
    const ITensorInfo *ti    = _tensor->info();
    const size_t       bytes = ti->total_size();
    cugl_context      *ctx   = CUScheduler::get().context();
    CU_ERROR_IF(_tensor->buffer() == nullptr, "host tensor operand is not allocated");
    if (_stage == nullptr || _stage_bytes < bytes)
    {
        if (_stage != nullptr)
        {
            cugl_sync(ctx);
            cugl_free(ctx, _stage);
            _stage = nullptr;
        }
        CU_THROW_ON(cu_status(cugl_malloc(ctx, bytes > 0 ? bytes : 1, &_stage), ctx, "CUOperand"));
        _stage_bytes = bytes;
    }
    if (upload)
    {
        // pageable source: the driver stages the bytes before the call returns
        CU_THROW_ON(cu_status(cugl_memcpy_h2d(ctx, _stage, _tensor->buffer(), bytes), ctx, "CUOperand"));
    }
    return static_cast<uint8_t *>(_stage) + ti->offset_first_element_in_bytes();
}

void CUOperand::download()
{
    if (_tensor == nullptr || is_device() || _stage == nullptr)
    {
        return;
    }
    const ITensorInfo *ti  = _tensor->info();
    cugl_context      *ctx = CUScheduler::get().context();
    // valid elements only, plane by plane, so that the host tensor's padding bytes are left as they are
    const size_t   width  = ti->dimension(0) * ti->element_size();
    const size_t   rows   = ti->num_dimensions() > 1 ? ti->dimension(1) : 1;
    const size_t   pitch  = ti->num_dimensions() > 1 ? ti->strides_in_bytes()[1] : width;
    const size_t   planes = ti->tensor_shape().total_size_upper(2);
    const size_t   off0   = ti->offset_first_element_in_bytes();
    const uint8_t *dev    = static_cast<const uint8_t *>(_stage);
    for (size_t p = 0; p < planes; ++p)
    {
        // planes above dimension 2 follow each other at stride_z when the tensor has no z padding (the only
        // padding TensorInfo::extend_padding creates is in x and y, inside a plane)
        const size_t off = off0 + p * (ti->num_dimensions() > 2 ? ti->strides_in_bytes()[2] : 0);
        CU_THROW_ON(cu_status(cugl_memcpy2d_d2h(ctx, _tensor->buffer() + off, pitch, dev + off, pitch, width, rows),
                                             ctx, "CUOperand::download"));
    }
    CU_THROW_ON(cu_status(cugl_sync(ctx), ctx, "CUOperand::download"));
}
} // namespace arm_compute
