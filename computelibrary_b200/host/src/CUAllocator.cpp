#include "arm_compute/runtime/CUDA/CUAllocator.h"

#include "arm_compute/core/Error.h"
#include "arm_compute/runtime/BlobLifetimeManager.h"
#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/MemoryManagerOnDemand.h"
#include "arm_compute/runtime/PoolManager.h"

#include <mutex>
#include <unordered_map>

namespace arm_compute
{
namespace
{
std::atomic<size_t> g_in_use{0}, g_peak{0};
std::mutex          g_sizes_mutex;
std::unordered_map<void *, size_t> g_sizes; // blocks handed out by CUAllocator::allocate

void account(size_t bytes)
{
    const size_t now  = g_in_use.fetch_add(bytes) + bytes;
    size_t       peak = g_peak.load();
    while (now > peak && !g_peak.compare_exchange_weak(peak, now))
    {
    }
}

void *device_alloc(size_t size)
{
    cugl_context *ctx = CUScheduler::get().context();
    void         *p   = nullptr;
    CU_THROW_ON(cu_status(cugl_malloc(ctx, size > 0 ? size : 1, &p), ctx, "CUAllocator"));
    account(size);
    return p;
}

void device_free(void *p, size_t size)
{
    if (p == nullptr)
    {
        return;
    }
    if (CUScheduler::get().is_initialised())
    {
        // kernels that still use the block may be in flight on the scheduler's stream
        cugl_context *ctx = CUScheduler::get().context();
        cugl_sync(ctx);
        cugl_free(ctx, p);
    }
    g_in_use.fetch_sub(size);
}
} // namespace

CUMemoryRegion::CUMemoryRegion(size_t size, size_t alignment) : IMemoryRegion(size), _ptr(nullptr), _owned(true)
{
    CU_ERROR_IF(alignment > 256, "CUMemoryRegion: device blocks are 256-byte aligned");
    _ptr = device_alloc(size);
}

CUMemoryRegion::CUMemoryRegion(void *device_ptr, size_t size) : IMemoryRegion(size), _ptr(device_ptr), _owned(false)
{
}

CUMemoryRegion::~CUMemoryRegion()
{
    if (_owned)
    {
        device_free(_ptr, _size);
    }
}

std::unique_ptr<IMemoryRegion> CUMemoryRegion::extract_subregion(size_t offset, size_t size)
{
    if (_ptr != nullptr && offset + size <= _size)
    {
        return std::make_unique<CUMemoryRegion>(static_cast<uint8_t *>(_ptr) + offset, size);
    }
    return nullptr;
}

void *CUAllocator::allocate(size_t size, size_t alignment)
{
    CU_ERROR_IF(alignment > 256, "CUAllocator: device blocks are 256-byte aligned");
    void *p = device_alloc(size);
    std::lock_guard<std::mutex> lock(g_sizes_mutex);
    g_sizes[p] = size;
    return p;
}

void CUAllocator::free(void *ptr)
{
    size_t size = 0;
    {
        std::lock_guard<std::mutex> lock(g_sizes_mutex);
        auto                        it = g_sizes.find(ptr);
        if (it != g_sizes.end())
        {
            size = it->second;
            g_sizes.erase(it);
        }
    }
    device_free(ptr, size);
}

std::unique_ptr<IMemoryRegion> CUAllocator::make_region(size_t size, size_t alignment)
{
    return std::make_unique<CUMemoryRegion>(size, alignment);
}

size_t CUAllocator::bytes_in_use()
{
    return g_in_use.load();
}
size_t CUAllocator::peak_bytes()
{
    return g_peak.load();
}
void CUAllocator::reset_peak()
{
    g_peak.store(g_in_use.load());
}

std::shared_ptr<IMemoryManager> cu_create_memory_manager()
{
    auto lifetime_mgr = std::make_shared<BlobLifetimeManager>();
    auto pool_mgr     = std::make_shared<PoolManager>();
    return std::make_shared<MemoryManagerOnDemand>(lifetime_mgr, pool_mgr);
}
} // namespace arm_compute
