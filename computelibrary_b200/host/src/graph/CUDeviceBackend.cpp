#include "arm_compute/graph/backends/CUDA/CUDeviceBackend.h"

#include "arm_compute/graph/backends/BackendRegistrar.h"
#include "arm_compute/graph/backends/CUDA/CUFunctionFactory.h"
#include "arm_compute/graph/backends/CUDA/CUTensorHandle.h"
#include "arm_compute/graph/Graph.h"
#include "arm_compute/graph/GraphContext.h"
#include "arm_compute/graph/INode.h"
#include "arm_compute/graph/Logger.h"
#include "arm_compute/graph/Tensor.h"
#include "arm_compute/runtime/BlobLifetimeManager.h"
#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/IWeightsManager.h"
#include "arm_compute/runtime/MemoryGroup.h"
#include "arm_compute/runtime/MemoryManagerOnDemand.h"
#include "arm_compute/runtime/OffsetLifetimeManager.h"
#include "arm_compute/runtime/PoolManager.h"

#include <cstdio>
#include <cstdlib>

namespace arm_compute
{
namespace graph
{
namespace backends
{
// registered when the library is loaded, as the NEON and CL backends register themselves
static detail::BackendRegistrar<CUDeviceBackend> CUDeviceBackend_registrar(CUDATarget);

void CUDeviceBackend::initialize_backend()
{
    CUScheduler::get().default_init();
    _initialized = true;
}

namespace
{
// CU_GRAPH_MEMORY_MANAGER=0 leaves every tensor and workspace with an allocation of its own (to measure what the
// lifetime managers save); CU_GRAPH_REPORT_MEMORY=1 prints the peak of device bytes held when a graph is released.
bool env_flag(const char *name, bool otherwise)
{
    const char *v = std::getenv(name);
    return v == nullptr ? otherwise : (v[0] != '0' && v[0] != '\0');
}
} // namespace

void CUDeviceBackend::release_backend_context(GraphContext &ctx)
{
    ARM_COMPUTE_UNUSED(ctx);
    if (env_flag("CU_GRAPH_REPORT_MEMORY", false))
    {
        std::printf("CUDA graph backend: peak device bytes held by tensors and workspaces: %zu\n", CUAllocator::peak_bytes());
    }
}

void CUDeviceBackend::setup_backend_context(GraphContext &ctx)
{
    if (!_initialized)
    {
        initialize_backend();
    }
    // function-level (intra) and tensor-level (cross) memory managers over device memory
    if (ctx.memory_management_ctx(CUDATarget) == nullptr)
    {
        MemoryManagerContext mm_ctx;
        mm_ctx.target      = CUDATarget;
        const bool managed = env_flag("CU_GRAPH_MEMORY_MANAGER", true);
        mm_ctx.intra_mm    = managed ? create_memory_manager(MemoryManagerAffinity::Buffer) : nullptr;
        mm_ctx.cross_mm    = managed ? create_memory_manager(MemoryManagerAffinity::Buffer) : nullptr;
        mm_ctx.cross_group = std::make_shared<MemoryGroup>(mm_ctx.cross_mm);
        mm_ctx.allocator   = &_allocator;
        ctx.insert_memory_management_ctx(std::move(mm_ctx));
    }
    if (ctx.weights_management_ctx(CUDATarget) == nullptr)
    {
        WeightsManagerContext wm_ctx;
        wm_ctx.target = CUDATarget;
        wm_ctx.wm     = create_weights_manager();
        ctx.insert_weights_management_ctx(std::move(wm_ctx));
    }
}

bool CUDeviceBackend::is_backend_supported()
{
    // cugl_context_create answers CUGL_UNSUPPORTED_TARGET without an sm_100 device; probing that here would create
    // a context just to ask, so the question is deferred to initialize_backend(), which throws with that message
    return true;
}

IAllocator *CUDeviceBackend::backend_allocator()
{
    return &_allocator;
}

std::unique_ptr<ITensorHandle> CUDeviceBackend::create_tensor(const Tensor &tensor)
{
    const TensorDescriptor &tensor_desc = tensor.desc();
    ARM_COMPUTE_ERROR_ON(tensor_desc.target != CUDATarget);
    TensorInfo info(tensor_desc.shape, 1, tensor_desc.data_type, tensor_desc.quant_info);
    info.set_data_layout(tensor_desc.layout);
    return std::make_unique<CUTensorHandle>(info);
}

std::unique_ptr<ITensorHandle>
CUDeviceBackend::create_subtensor(ITensorHandle *parent, TensorShape shape, Coordinates coords, bool extend_parent)
{
    // sub-tensor views (depth-concatenate / split mutators) are not implemented: the mutators then keep the copies
    ARM_COMPUTE_UNUSED(parent, shape, coords, extend_parent);
    return nullptr;
}

std::unique_ptr<arm_compute::IFunction> CUDeviceBackend::configure_node(INode &node, GraphContext &ctx)
{
    ARM_COMPUTE_LOG_GRAPH_VERBOSE("Configuring CUDA node with ID : " << node.id() << std::endl);
    ARM_COMPUTE_ERROR_ON(node.assigned_target() != CUDATarget);
    return CUFunctionFactory::create(&node, ctx);
}

Status CUDeviceBackend::validate_node(INode &node)
{
    ARM_COMPUTE_LOG_GRAPH_VERBOSE("Validating CUDA node with ID : " << node.id() << std::endl);
    ARM_COMPUTE_ERROR_ON(node.assigned_target() != CUDATarget);
    return CUNodeValidator::validate(&node);
}

std::shared_ptr<arm_compute::IMemoryManager> CUDeviceBackend::create_memory_manager(MemoryManagerAffinity affinity)
{
    std::shared_ptr<ILifetimeManager> lifetime_mgr = nullptr;
    if (affinity == MemoryManagerAffinity::Buffer)
    {
        lifetime_mgr = std::make_shared<BlobLifetimeManager>();
    }
    else
    {
        lifetime_mgr = std::make_shared<OffsetLifetimeManager>();
    }
    auto pool_mgr = std::make_shared<PoolManager>();
    return std::make_shared<MemoryManagerOnDemand>(lifetime_mgr, pool_mgr);
}

std::shared_ptr<arm_compute::IWeightsManager> CUDeviceBackend::create_weights_manager()
{
    // the plans re-lay the weights out on the device themselves; nothing for a host-side manager to share
    return nullptr;
}

void CUDeviceBackend::sync()
{
    CUScheduler::get().sync();
}
} // namespace backends
} // namespace graph
} // namespace arm_compute
