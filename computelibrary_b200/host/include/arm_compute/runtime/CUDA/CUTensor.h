// Device tensor of the CUDA backend: an ITensor whose bytes live in HBM.  Modelled on ICLTensor / CLTensor
// (arm_compute/core/CL/ICLTensor.h:45-111, arm_compute/runtime/CL/CLTensor.h:44-101): buffer() is only valid
// between map() and unmap(); the allocator follows ITensorAllocator (arm_compute/runtime/ITensorAllocator.h:60-111).
#pragma once
#include "arm_compute/core/TensorInfo.h"

namespace arm_compute
{
class CUTensorAllocator
{
public:
    CUTensorAllocator() = default;
    ~CUTensorAllocator();
    CUTensorAllocator(const CUTensorAllocator &)            = delete;
    CUTensorAllocator &operator=(const CUTensorAllocator &) = delete;
    void        init(const TensorInfo &input, size_t alignment = 0);
    TensorInfo &info() { return _info; }
    const TensorInfo &info() const { return _info; }
    void        allocate();            // cudaMalloc-backed region of info().total_size() bytes
    void        free();
    bool        is_allocated() const { return _device != nullptr; }
    // Adopt device memory owned by the caller (e.g. a framework tensor); never freed here.
    void        import_memory(void *device_ptr);
    void       *device_ptr() const { return _device; }
    uint8_t    *map(bool blocking);    // pinned host mirror filled from the device
    void        unmap();               // host mirror written back to the device
    uint8_t    *mapping() const { return _host; }

private:
    TensorInfo _info{};
    void      *_device{nullptr};
    uint8_t   *_host{nullptr};
    bool       _owns{false};
    bool       _mapped{false};
};

class CUTensor : public ITensor
{
public:
    CUTensor() = default;
    ITensorInfo       *info() const override { return const_cast<TensorInfo *>(&_allocator.info()); }
    ITensorInfo       *info() override { return &_allocator.info(); }
    uint8_t           *buffer() const override { return _allocator.mapping(); }
    CUTensorAllocator *allocator() { return &_allocator; }
    void              *device_ptr() const { return _allocator.device_ptr(); }
    void               map(bool blocking = true) { _allocator.map(blocking); }
    void               unmap() { _allocator.unmap(); }

private:
    mutable CUTensorAllocator _allocator{};
};

// Device pointer of any ITensor handed to a CUDA function: it must be a CUTensor.
void *cu_device_ptr(const ITensor *t);
} // namespace arm_compute
