// Tensor allocator of the CUDA backend: ITensorAllocator (arm_compute/runtime/ITensorAllocator.h:60-111) over device
// memory, with the memory-group protocol of the host TensorAllocator (src/runtime/TensorAllocator.cpp:133-146: a
// managed tensor defers to IMemoryGroup::finalize_memory instead of allocating) and the map / unmap access of
// CLTensorAllocator (src/runtime/CL/CLTensorAllocator.cpp:131-239).
#pragma once
#include "arm_compute/runtime/IMemoryGroup.h"
#include "arm_compute/runtime/ITensorAllocator.h"
#include "arm_compute/runtime/Memory.h"

#include <cstdint>

namespace arm_compute
{
class CUTensorAllocator : public ITensorAllocator
{
public:
    explicit CUTensorAllocator(IMemoryManageable *owner = nullptr);
    ~CUTensorAllocator() override;
    CUTensorAllocator(const CUTensorAllocator &)            = delete;
    CUTensorAllocator &operator=(const CUTensorAllocator &) = delete;
    CUTensorAllocator(CUTensorAllocator &&) noexcept;
    CUTensorAllocator &operator=(CUTensorAllocator &&) noexcept;

    // Device address of byte 0 of the tensor's buffer (NOT of its first element: add
    // info().offset_first_element_in_bytes()); nullptr while unallocated or while a managed tensor's group is released.
    void *device_ptr() const;
    // Adopt device memory owned by the caller (a framework tensor, a peer buffer); never freed here.
    Status import_memory(void *device_ptr);
    void   set_associated_memory_group(IMemoryGroup *associated_memory_group);
    void   set_owner(IMemoryManageable *owner) { _owner = owner; }

    // Host access in the style of ICLTensor::map (arm_compute/core/CL/ICLTensor.h:45-111): map copies the buffer into
    // a pinned host mirror (blocking = wait for the copy), unmap writes the mirror back.
    uint8_t *map(bool blocking);
    void     unmap();
    uint8_t *mapping() const { return _mapped ? _host : nullptr; }

    // Inherited methods overridden:
    void allocate() override;
    void free() override;
    bool is_allocated() const override;

protected:
    uint8_t *lock() override;
    void     unlock() override;

private:
    void release_host();
    IMemoryManageable *_owner{nullptr};
    IMemoryGroup      *_associated_memory_group{nullptr};
    Memory             _memory{};
    uint8_t           *_host{nullptr};
    size_t             _host_bytes{0};
    bool               _mapped{false};
};
} // namespace arm_compute
