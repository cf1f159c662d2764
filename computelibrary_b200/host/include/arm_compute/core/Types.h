// Minimal stand-ins for the arm_compute core types the quantized GEMM path touches: DataType, DataLayout,
// TensorShape, Strides, Size2D, PadStrideInfo, WeightsInfo, PoolingLayerInfo, ConvertPolicy.  Member names and meanings follow the library
// (arm_compute/core/CoreTypes.h, TensorShape.h, Types.h); only what the CUDA functions use is present.
#pragma once
#include <array>
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <utility>

namespace arm_compute
{
enum class DataType
{
    UNKNOWN,
    U8,
    S8,
    QSYMM8,
    QASYMM8,
    QASYMM8_SIGNED,
    QSYMM8_PER_CHANNEL,
    QSYMM16,
    S32,
    F32
};
enum class DataLayout
{
    UNKNOWN,
    NCHW,
    NHWC
};
enum class DimensionRoundingType
{
    FLOOR,
    CEIL
};

inline size_t element_size_from_data_type(DataType dt)
{
    return (dt == DataType::S32 || dt == DataType::F32) ? 4 : (dt == DataType::QSYMM16 ? 2 : 1);
}
inline bool is_data_type_quantized_per_channel(DataType dt)
{
    return dt == DataType::QSYMM8_PER_CHANNEL;
}
inline bool is_data_type_quantized_asymmetric(DataType dt)
{
    return dt == DataType::QASYMM8 || dt == DataType::QASYMM8_SIGNED;
}
inline bool is_data_type_quantized(DataType dt)
{
    return is_data_type_quantized_asymmetric(dt) || dt == DataType::QSYMM8 || dt == DataType::QSYMM8_PER_CHANNEL;
}

// Up to six dimensions, x (dimension 0) fastest; unset dimensions read as 1.
class TensorShape
{
public:
    static constexpr size_t num_max_dimensions = 6;
    TensorShape() { _d.fill(1); }
    template <typename... Ts>
    TensorShape(Ts... dims) : TensorShape()
    {
        const size_t v[] = {static_cast<size_t>(dims)...};
        _n               = sizeof...(Ts);
        for (size_t i = 0; i < _n; ++i) _d[i] = v[i];
    }
    size_t       operator[](size_t i) const { return _d[i]; }
    size_t       x() const { return _d[0]; }
    size_t       y() const { return _d[1]; }
    size_t       z() const { return _d[2]; }
    unsigned int num_dimensions() const { return static_cast<unsigned int>(_n); }
    void         set(size_t i, size_t v)
    {
        _d[i] = v;
        if (i + 1 > _n) _n = i + 1;
    }
    size_t total_size() const
    {
        size_t t = 1;
        for (size_t v : _d) t *= v;
        return t;
    }
    size_t total_size_upper(size_t from) const
    {
        size_t t = 1;
        for (size_t i = from; i < num_max_dimensions; ++i) t *= _d[i];
        return t;
    }
    bool operator==(const TensorShape &o) const { return _d == o._d; }
    bool operator!=(const TensorShape &o) const { return !(*this == o); }

private:
    std::array<size_t, num_max_dimensions> _d{};
    size_t                                 _n{0};
};

using Strides = std::array<size_t, TensorShape::num_max_dimensions>;

struct Size2D
{
    Size2D() = default;
    Size2D(size_t w, size_t h) : width(w), height(h) {}
    size_t x() const { return width; }
    size_t y() const { return height; }
    size_t width{0}, height{0};
};

class PadStrideInfo
{
public:
    PadStrideInfo(unsigned int stride_x = 1, unsigned int stride_y = 1, unsigned int pad_x = 0, unsigned int pad_y = 0,
                  DimensionRoundingType round = DimensionRoundingType::FLOOR)
        : _stride(stride_x, stride_y), _l(pad_x), _t(pad_y), _r(pad_x), _b(pad_y), _round(round)
    {
    }
    PadStrideInfo(unsigned int stride_x, unsigned int stride_y, unsigned int pad_left, unsigned int pad_right,
                  unsigned int pad_top, unsigned int pad_bottom, DimensionRoundingType round)
        : _stride(stride_x, stride_y), _l(pad_left), _t(pad_top), _r(pad_right), _b(pad_bottom), _round(round)
    {
    }
    std::pair<unsigned int, unsigned int> stride() const { return _stride; }
    unsigned int                          pad_left() const { return _l; }
    unsigned int                          pad_right() const { return _r; }
    unsigned int                          pad_top() const { return _t; }
    unsigned int                          pad_bottom() const { return _b; }
    DimensionRoundingType                 round() const { return _round; }

private:
    std::pair<unsigned int, unsigned int> _stride;
    unsigned int                          _l, _t, _r, _b;
    DimensionRoundingType                 _round;
};

enum class ConvertPolicy
{
    WRAP,
    SATURATE
};
enum class PoolingType
{
    MAX,
    AVG,
    L2
};
// arm_compute/core/Types.h (PoolingLayerInfo): global pooling has a zero pool size.
struct PoolingLayerInfo
{
    PoolingLayerInfo() = default;
    PoolingLayerInfo(PoolingType type, unsigned int size, DataLayout layout, PadStrideInfo psi = PadStrideInfo(),
                     bool exclude_pad = false)
        : pool_type(type), pool_size(size, size), data_layout(layout), pad_stride_info(psi), exclude_padding(exclude_pad)
    {
    }
    PoolingLayerInfo(PoolingType type, Size2D size, DataLayout layout, PadStrideInfo psi = PadStrideInfo(),
                     bool exclude_pad = false)
        : pool_type(type), pool_size(size), data_layout(layout), pad_stride_info(psi), exclude_padding(exclude_pad)
    {
    }
    PoolingLayerInfo(PoolingType type, DataLayout layout) // global pooling
        : pool_type(type), pool_size(0, 0), data_layout(layout), is_global_pooling(true)
    {
    }
    PoolingType   pool_type{PoolingType::MAX};
    Size2D        pool_size{};
    DataLayout    data_layout{DataLayout::UNKNOWN};
    PadStrideInfo pad_stride_info{};
    bool          exclude_padding{false};
    bool          is_global_pooling{false};
};

// Convolution weights descriptor; the quantized GEMM path only checks that weights are not pre-reshaped.
class WeightsInfo
{
public:
    WeightsInfo() = default;
    bool are_reshaped() const { return false; }
};
} // namespace arm_compute
