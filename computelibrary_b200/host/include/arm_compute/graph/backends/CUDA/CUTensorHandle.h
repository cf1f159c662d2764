// ITensorHandle over a CUTensor (arm_compute/graph/ITensorHandle.h:41-105; precedent CLTensorHandle): map() brings the
// bytes into the pinned host mirror for the graph's accessors, unmap() writes them back.
#pragma once
#include "arm_compute/graph/ITensorHandle.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"

namespace arm_compute
{
namespace graph
{
namespace backends
{
class CUTensorHandle final : public ITensorHandle
{
public:
    explicit CUTensorHandle(const ITensorInfo &info);
    CUTensorHandle(CUTensorHandle &&)            = default;
    CUTensorHandle &operator=(CUTensorHandle &&) = default;

    // Inherited overridden methods
    void                        allocate() override;
    void                        free() override;
    void                        manage(IMemoryGroup *mg) override;
    void                        map(bool blocking) override;
    void                        unmap() override;
    void                        release_if_unused() override;
    arm_compute::ITensor       &tensor() override;
    const arm_compute::ITensor &tensor() const override;
    ITensorHandle              *parent_handle() override;
    bool                        is_subtensor() const override;
    Target                      target() const override;

private:
    arm_compute::CUTensor _tensor;
};
} // namespace backends
} // namespace graph
} // namespace arm_compute
