// Device tensor of the CUDA backend: an ITensor whose bytes live in HBM.  Modelled on ICLTensor / CLTensor
// (arm_compute/core/CL/ICLTensor.h:45-111, arm_compute/runtime/CL/CLTensor.h:44-101): buffer() is only valid
// between map() and unmap().  The device buffer has the geometry of the TensorInfo (strides, padding,
// offset_first_element_in_bytes: arm_compute/core/ITensorInfo.h:197-211), so a tensor that was padded after
// configure() -- as the validation fixtures do -- is laid out on the device exactly as on the host.
#pragma once
#include "arm_compute/core/ITensor.h"
#include "arm_compute/runtime/CUDA/CUTensorAllocator.h"

namespace arm_compute
{
class IRuntimeContext;

class CUTensor : public ITensor, public IMemoryManageable
{
public:
    // ctx: accepted for signature parity with Tensor / CLTensor (arm_compute/runtime/Tensor.h:48, CLTensor.h:53); unused
    CUTensor(IRuntimeContext *ctx = nullptr);
    ~CUTensor() override             = default;
    CUTensor(const CUTensor &)            = delete;
    CUTensor &operator=(const CUTensor &) = delete;
    CUTensor(CUTensor &&) noexcept;
    CUTensor &operator=(CUTensor &&) noexcept;

    CUTensorAllocator *allocator() { return &_allocator; }
    // device address of the first element (buffer base + offset_first_element_in_bytes)
    void *device_ptr() const;
    void  map(bool blocking = true);
    void  unmap();

    // Inherited methods overridden:
    ITensorInfo *info() const override;
    ITensorInfo *info() override;
    uint8_t     *buffer() const override; // host mirror while mapped, else nullptr
    void         associate_memory_group(IMemoryGroup *memory_group) override;

private:
    mutable CUTensorAllocator _allocator;
};

// Device address of the first element of an operand that must be a CUTensor (the byte-wise layer functions).
void *cu_device_ptr(const ITensor *t);

// How a CUDA function reaches an operand.  A CUTensor is used where it lies.  Any other ITensor (a host Tensor) is
// staged: its whole buffer, padding included, is copied to a device buffer of the same geometry before the run
// (inputs) or copied back after it, row by row so that the host padding stays untouched (outputs; this blocks).
class CUOperand
{
public:
    CUOperand() = default;
    ~CUOperand();
    CUOperand(const CUOperand &)            = delete;
    CUOperand &operator=(const CUOperand &) = delete;
    void        set(const ITensor *t) { _tensor = t; }
    const ITensor *tensor() const { return _tensor; }
    bool        is_device() const;
    // device address of the first element; copies a host tensor in first when upload is set
    void *device(bool upload);
    // copy a staged output back to its host tensor (no-op for a CUTensor); blocks until the data is there
    void  download();

private:
    const ITensor *_tensor{nullptr};
    void          *_stage{nullptr};
    size_t         _stage_bytes{0};
};
} // namespace arm_compute
