// Minimal stand-ins for ITensorInfo / TensorInfo / ITensor: shape, type, byte strides (dense, no padding
// unless set explicitly), quantisation info and layout.
#pragma once
#include "arm_compute/core/Error.h"
#include "arm_compute/core/QuantizationInfo.h"
#include "arm_compute/core/Types.h"

#include <memory>

namespace arm_compute
{
class ITensorInfo
{
public:
    virtual ~ITensorInfo()                                                         = default;
    virtual std::unique_ptr<ITensorInfo> clone() const                             = 0;
    virtual const TensorShape           &tensor_shape() const                      = 0;
    virtual ITensorInfo                 &set_tensor_shape(const TensorShape &s)    = 0;
    virtual DataType                     data_type() const                         = 0;
    virtual ITensorInfo                 &set_data_type(DataType dt)                = 0;
    virtual size_t                       element_size() const                      = 0;
    virtual size_t                       dimension(size_t i) const                 = 0;
    virtual size_t                       num_dimensions() const                    = 0;
    virtual const Strides               &strides_in_bytes() const                  = 0;
    virtual size_t                       offset_first_element_in_bytes() const     = 0;
    virtual size_t                       total_size() const                        = 0;
    virtual QuantizationInfo             quantization_info() const                 = 0;
    virtual ITensorInfo                 &set_quantization_info(const QuantizationInfo &q) = 0;
    virtual DataLayout                   data_layout() const                       = 0;
    virtual ITensorInfo                 &set_data_layout(const DataLayout &l)      = 0;
    virtual bool                         are_values_constant() const               = 0;
    virtual ITensorInfo                 &set_are_values_constant(bool c)           = 0;
};

class TensorInfo final : public ITensorInfo
{
public:
    TensorInfo() = default;
    TensorInfo(const TensorShape &shape, size_t num_channels, DataType dt) { init(shape, num_channels, dt); }
    TensorInfo(const TensorShape &shape, size_t num_channels, DataType dt, QuantizationInfo q)
    {
        init(shape, num_channels, dt);
        _qinfo = std::move(q);
    }
    TensorInfo(const ITensorInfo &o)
        : _shape(o.tensor_shape()), _dt(o.data_type()), _strides(o.strides_in_bytes()),
          _offset(o.offset_first_element_in_bytes()), _total(o.total_size()), _qinfo(o.quantization_info()),
          _layout(o.data_layout()), _const(o.are_values_constant())
    {
    }
    void init(const TensorShape &shape, size_t num_channels, DataType dt)
    {
        (void)num_channels;
        _shape = shape;
        _dt    = dt;
        recompute();
    }
    // Row pitch in bytes larger than the dense one (the library expresses this as right padding).
    void set_row_pitch(size_t bytes)
    {
        _pitch = bytes;
        recompute();
    }
    std::unique_ptr<ITensorInfo> clone() const override { return std::make_unique<TensorInfo>(*this); }
    const TensorShape           &tensor_shape() const override { return _shape; }
    ITensorInfo                 &set_tensor_shape(const TensorShape &s) override
    {
        _shape = s;
        recompute();
        return *this;
    }
    DataType     data_type() const override { return _dt; }
    ITensorInfo &set_data_type(DataType dt) override
    {
        _dt = dt;
        recompute();
        return *this;
    }
    size_t           element_size() const override { return element_size_from_data_type(_dt); }
    size_t           dimension(size_t i) const override { return _shape[i]; }
    size_t           num_dimensions() const override { return _shape.num_dimensions(); }
    const Strides   &strides_in_bytes() const override { return _strides; }
    size_t           offset_first_element_in_bytes() const override { return _offset; }
    size_t           total_size() const override { return _shape.num_dimensions() == 0 ? 0 : _total; }
    QuantizationInfo quantization_info() const override { return _qinfo; }
    ITensorInfo     &set_quantization_info(const QuantizationInfo &q) override
    {
        _qinfo = q;
        return *this;
    }
    DataLayout   data_layout() const override { return _layout; }
    ITensorInfo &set_data_layout(const DataLayout &l) override
    {
        _layout = l;
        return *this;
    }
    bool         are_values_constant() const override { return _const; }
    ITensorInfo &set_are_values_constant(bool c) override
    {
        _const = c;
        return *this;
    }

private:
    void recompute()
    {
        const size_t es = element_size_from_data_type(_dt);
        _strides[0]     = es;
        size_t row      = _shape[0] * es;
        if (_pitch > row) row = _pitch;
        _strides[1] = row;
        for (size_t i = 2; i < TensorShape::num_max_dimensions; ++i) _strides[i] = _strides[i - 1] * _shape[i - 1];
        _total = _strides[TensorShape::num_max_dimensions - 1] * _shape[TensorShape::num_max_dimensions - 1];
    }
    TensorShape      _shape{};
    DataType         _dt{DataType::UNKNOWN};
    Strides          _strides{};
    size_t           _offset{0}, _total{0}, _pitch{0};
    QuantizationInfo _qinfo{};
    DataLayout       _layout{DataLayout::NCHW};
    bool             _const{true};
};

class ITensor
{
public:
    virtual ~ITensor()                      = default;
    virtual ITensorInfo *info() const       = 0;
    virtual ITensorInfo *info()             = 0;
    virtual uint8_t     *buffer() const     = 0; // host-visible bytes; for a device tensor only while mapped
    bool                 is_used() const { return _used; }
    void                 mark_as_unused() const { _used = false; }
    void                 mark_as_used() const { _used = true; }

private:
    mutable bool _used{true};
};
} // namespace arm_compute
