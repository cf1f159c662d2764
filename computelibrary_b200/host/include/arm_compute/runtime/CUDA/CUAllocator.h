// Device memory for the CUDA backend behind Compute Library's own allocator interfaces, so that the library's
// memory management (MemoryManagerOnDemand + BlobLifetimeManager / OffsetLifetimeManager + PoolManager, MemoryGroup)
// works on HBM unchanged: a region is one cudaMalloc block, handed out by CUAllocator.
//   IAllocator      arm_compute/runtime/IAllocator.h:39-61
//   IMemoryRegion   arm_compute/runtime/IMemoryRegion.h:37-71
//   precedent       CLBufferAllocator (arm_compute/runtime/CL/CLBufferAllocator.h), CLBufferMemoryRegion
#pragma once
#include "arm_compute/runtime/IAllocator.h"
#include "arm_compute/runtime/IMemoryManager.h"
#include "arm_compute/runtime/IMemoryRegion.h"

#include <atomic>
#include <cstddef>
#include <memory>

namespace arm_compute
{
// A block of device memory.  buffer() is a DEVICE address: host code must not dereference it.
class CUMemoryRegion final : public IMemoryRegion
{
public:
    CUMemoryRegion(size_t size, size_t alignment); // owning: cudaMalloc'ed (256-byte aligned) through the scheduler's context
    CUMemoryRegion(void *device_ptr, size_t size); // wrapping: memory owned by the caller (or by a parent region)
    ~CUMemoryRegion() override;
    CUMemoryRegion(const CUMemoryRegion &)            = delete;
    CUMemoryRegion &operator=(const CUMemoryRegion &) = delete;

    void                          *buffer() override { return _ptr; }
    const void                    *buffer() const override { return _ptr; }
    std::unique_ptr<IMemoryRegion> extract_subregion(size_t offset, size_t size) override;

private:
    void *_ptr{nullptr};
    bool  _owned{false};
};

class CUAllocator final : public IAllocator
{
public:
    void                          *allocate(size_t size, size_t alignment) override;
    void                           free(void *ptr) override;
    std::unique_ptr<IMemoryRegion> make_region(size_t size, size_t alignment) override;

    // Bytes currently / at most held by owning CUMemoryRegions and CUAllocator::allocate blocks of this process.
    static size_t bytes_in_use();
    static size_t peak_bytes();
    static void   reset_peak();
};

// MemoryManagerOnDemand(BlobLifetimeManager, PoolManager): the manager the NEON examples create
// (examples/graph_*.cpp through the graph backend, src/graph/backends/NEON/NEDeviceBackend.cpp:118-135).  Populate it
// with a CUAllocator once every function has been configured:  mm->populate(allocator, num_pools).
std::shared_ptr<IMemoryManager> cu_create_memory_manager();
} // namespace arm_compute
