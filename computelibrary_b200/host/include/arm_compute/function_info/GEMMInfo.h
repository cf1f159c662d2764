// Minimal stand-ins for GEMMLowpOutputStageInfo / GEMMInfo / ActivationLayerInfo
// (arm_compute/function_info/GEMMInfo.h:40-399, ActivationLayerInfo.h): same member and accessor names.
#pragma once
#include "arm_compute/core/Types.h"

#include <cstdint>
#include <limits>
#include <vector>

namespace arm_compute
{
class ActivationLayerInfo
{
public:
    enum class ActivationFunction
    {
        IDENTITY,
        RELU,
        BOUNDED_RELU,
        LU_BOUNDED_RELU
    };
    ActivationLayerInfo() = default;
    ActivationLayerInfo(ActivationFunction f, float a = 0.f, float b = 0.f) : _f(f), _a(a), _b(b), _enabled(true) {}
    ActivationFunction activation() const { return _f; }
    float              a() const { return _a; }
    float              b() const { return _b; }
    bool               enabled() const { return _enabled; }

private:
    ActivationFunction _f{ActivationFunction::IDENTITY};
    float              _a{0.f}, _b{0.f};
    bool               _enabled{false};
};

enum class GEMMLowpOutputStageType
{
    NONE,
    QUANTIZE_DOWN,
    QUANTIZE_DOWN_FIXEDPOINT,
    QUANTIZE_DOWN_FLOAT
};

struct GEMMLowpOutputStageInfo
{
    GEMMLowpOutputStageType type{GEMMLowpOutputStageType::NONE};
    int32_t                 gemmlowp_offset{0};
    int32_t                 gemmlowp_multiplier{0};
    int32_t                 gemmlowp_shift{0};
    int32_t                 gemmlowp_min_bound{std::numeric_limits<int32_t>::lowest()};
    int32_t                 gemmlowp_max_bound{std::numeric_limits<int32_t>::max()};
    std::vector<int32_t>    gemmlowp_multipliers{};
    std::vector<int32_t>    gemmlowp_shifts{};
    float                   gemmlowp_real_multiplier{0};
    bool                    is_quantized_per_channel{false};
    DataType                output_data_type{DataType::UNKNOWN};
};

class GEMMInfo
{
public:
    GEMMInfo() = default;
    bool                    is_a_reshaped() const { return _a_reshaped; }
    bool                    is_b_reshaped() const { return _b_reshaped; }
    bool                    reshape_b_only_on_first_run() const { return _reshape_b_once; }
    bool                    pretranspose_A() const { return _pre_a; }
    bool                    pretranspose_B() const { return _pre_b; }
    bool                    accumulate() const { return _accumulate; }
    GEMMLowpOutputStageInfo gemmlowp_output_stage() const { return _stage; }
    void set_gemmlowp_output_stage(const GEMMLowpOutputStageInfo &s) { _stage = s; }
    void set_reshape_b_only_on_first_run(bool v) { _reshape_b_once = v; }
    void set_is_a_reshaped(bool v) { _a_reshaped = v; }
    void set_is_b_reshaped(bool v) { _b_reshaped = v; }
    void set_pretranspose_A(bool v) { _pre_a = v; }
    void set_pretranspose_B(bool v) { _pre_b = v; }
    void set_accumulate(bool v) { _accumulate = v; }

private:
    bool                    _a_reshaped{false}, _b_reshaped{false}, _reshape_b_once{true};
    bool                    _pre_a{false}, _pre_b{false}, _accumulate{false};
    GEMMLowpOutputStageInfo _stage{};
};
} // namespace arm_compute
