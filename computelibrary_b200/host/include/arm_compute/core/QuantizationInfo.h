// Minimal stand-in for arm_compute/core/QuantizationInfo.h: per-tensor (scale, offset) or per-channel scales.
#pragma once
#include <cmath>
#include <cstdint>
#include <vector>

namespace arm_compute
{
struct UniformQuantizationInfo
{
    UniformQuantizationInfo() = default;
    UniformQuantizationInfo(float s, int32_t o) : scale(s), offset(o) {}
    bool    empty() const { return scale == 0.f; }
    float   scale{0.f};
    int32_t offset{0};
};

class QuantizationInfo
{
public:
    QuantizationInfo() = default;
    QuantizationInfo(float scale) : _scale(1, scale) {}
    QuantizationInfo(float scale, int offset) : _scale(1, scale), _offset(1, offset) {}
    QuantizationInfo(std::vector<float> scale) : _scale(std::move(scale)) {}
    QuantizationInfo(std::vector<float> scale, std::vector<int32_t> offset)
        : _scale(std::move(scale)), _offset(std::move(offset))
    {
    }
    const std::vector<float>   &scale() const { return _scale; }
    const std::vector<int32_t> &offset() const { return _offset; }
    bool                        empty() const { return _scale.empty() && _offset.empty(); }
    UniformQuantizationInfo     uniform() const
    {
        UniformQuantizationInfo u;
        u.scale  = _scale.empty() ? 0.f : _scale[0];
        u.offset = _offset.empty() ? 0 : _offset[0];
        return u;
    }

private:
    std::vector<float>   _scale{};
    std::vector<int32_t> _offset{};
};

// round-to-nearest (ties away from zero) quantisation with saturation, as Qasymm8QuantizationHelper::quantize
inline int quantize_qasymm8(float value, const UniformQuantizationInfo &q)
{
    const long v = std::lround(value / q.scale) + q.offset;
    return static_cast<int>(v < 0 ? 0 : (v > 255 ? 255 : v));
}
inline int quantize_qasymm8_signed(float value, const UniformQuantizationInfo &q)
{
    const long v = std::lround(value / q.scale) + q.offset;
    return static_cast<int>(v < -128 ? -128 : (v > 127 ? 127 : v));
}
} // namespace arm_compute
