// Accessor of the validation framework for CUTensor: the counterpart of tests/CL/CLAccessor.h:37-160.  The tensor is
// mapped (device -> pinned host mirror) while the accessor lives and written back when it goes away.
#pragma once
#include "arm_compute/runtime/CUDA/CUTensor.h"
#include "tests/IAccessor.h"

namespace arm_compute
{
namespace test
{
class CUAccessor : public IAccessor
{
public:
    explicit CUAccessor(CUTensor &tensor) : _tensor{tensor} { _tensor.map(true); }
    CUAccessor(const CUAccessor &)            = delete;
    CUAccessor &operator=(const CUAccessor &) = delete;
    CUAccessor(CUAccessor &&)                 = default;
    ~CUAccessor() override { _tensor.unmap(); }

    TensorShape      shape() const override { return _tensor.info()->tensor_shape(); }
    size_t           element_size() const override { return _tensor.info()->element_size(); }
    size_t           size() const override { return _tensor.info()->total_size(); }
    Format           format() const override { return _tensor.info()->format(); }
    DataLayout       data_layout() const override { return _tensor.info()->data_layout(); }
    DataType         data_type() const override { return _tensor.info()->data_type(); }
    int              num_channels() const override { return _tensor.info()->num_channels(); }
    int              num_elements() const override { return _tensor.info()->tensor_shape().total_size(); }
    PaddingSize      padding() const override { return _tensor.info()->padding(); }
    QuantizationInfo quantization_info() const override { return _tensor.info()->quantization_info(); }
    const void      *operator()(const Coordinates &coord) const override { return _tensor.ptr_to_element(coord); }
    void            *operator()(const Coordinates &coord) override { return _tensor.ptr_to_element(coord); }

private:
    CUTensor &_tensor;
};
} // namespace test
} // namespace arm_compute
