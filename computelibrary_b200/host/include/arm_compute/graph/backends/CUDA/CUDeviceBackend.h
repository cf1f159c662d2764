// Graph backend of the CUDA function family: what NEDeviceBackend / CLDeviceBackend are for their targets
// (arm_compute/graph/IDeviceBackend.h:51-125; precedent src/graph/backends/NEON/NEDeviceBackend.cpp).  With it the
// graph frontend -- examples/graph_resnet50.cpp unchanged, its --type=QASYMM8 synthetic mode included -- builds its
// workload out of CU* functions: tensors are CUTensors, the cross- and intra-function memory managers are the
// library's own MemoryManagerOnDemand over a CUAllocator, sync() drains the scheduler's stream.
//
// Target: arm_compute::graph::Target (arm_compute/graph/Types.h:108-114) has no CUDA entry.  Inside Compute Library
// the integration adds one enumerator (and its name to TypeLoader.cpp / TypePrinter.h) and registers this backend
// under it.  Built against an unmodified tree -- as here -- the backend registers under Target::CL, whose slot is
// free in a build without OpenCL (the registry holds one backend per target): `--target=CL` then means this backend.
#pragma once
#include "arm_compute/graph/IDeviceBackend.h"
#include "arm_compute/runtime/CUDA/CUAllocator.h"

namespace arm_compute
{
namespace graph
{
namespace backends
{
constexpr Target CUDATarget = Target::CL; // see the note above

class CUDeviceBackend final : public IDeviceBackend
{
public:
    CUDeviceBackend() = default;

    // Inherited overridden methods
    void                                            initialize_backend() override;
    void                                            setup_backend_context(GraphContext &ctx) override;
    void                                            release_backend_context(GraphContext &ctx) override;
    bool                                            is_backend_supported() override;
    IAllocator                                     *backend_allocator() override;
    std::unique_ptr<ITensorHandle>                  create_tensor(const Tensor &tensor) override;
    std::unique_ptr<ITensorHandle>
    create_subtensor(ITensorHandle *parent, TensorShape shape, Coordinates coords, bool extend_parent) override;
    std::unique_ptr<arm_compute::IFunction>         configure_node(INode &node, GraphContext &ctx) override;
    Status                                          validate_node(INode &node) override;
    std::shared_ptr<arm_compute::IMemoryManager>    create_memory_manager(MemoryManagerAffinity affinity) override;
    std::shared_ptr<arm_compute::IWeightsManager>   create_weights_manager() override;
    void                                            sync() override;

private:
    bool        _initialized{false};
    CUAllocator _allocator{};
};
} // namespace backends
} // namespace graph
} // namespace arm_compute
