// CUDA counterpart of NEGEMMLowpMatrixMultiplyCore with the same interface
// (arm_compute/runtime/NEON/functions/NEGEMMLowpMatrixMultiplyCore.h:54-128).
//
// Supported rows of the NE type table (:72-90): src0 QASYMM8 / QASYMM8_SIGNED; src1 QASYMM8, QASYMM8_SIGNED,
// QSYMM8, QSYMM8_PER_CHANNEL; src2 S32 or none; dst QASYMM8 / QASYMM8_SIGNED (QUANTIZE_DOWN_FIXEDPOINT stage) or
// S32 (stage NONE).  The F32 / F16 dequantising rows are not implemented.
#pragma once
#include "arm_compute/core/ITensor.h"
#include "arm_compute/core/Types.h"
#include "arm_compute/function_info/ActivationLayerInfo.h"
#include "arm_compute/function_info/GEMMInfo.h"
#include "arm_compute/runtime/IFunction.h"
#include "arm_compute/runtime/IMemoryManager.h"
#include "arm_compute/runtime/IWeightsManager.h"

#include <memory>

struct cugl_gemm_plan;

namespace arm_compute
{
class CUGEMMLowpMatrixMultiplyCore : public IFunction
{
public:
    CUGEMMLowpMatrixMultiplyCore(std::shared_ptr<IMemoryManager> memory_manager  = nullptr,
                                 IWeightsManager                *weights_manager = nullptr);
    CUGEMMLowpMatrixMultiplyCore(const CUGEMMLowpMatrixMultiplyCore &)            = delete;
    CUGEMMLowpMatrixMultiplyCore &operator=(const CUGEMMLowpMatrixMultiplyCore &) = delete;
    ~CUGEMMLowpMatrixMultiplyCore();
    // a [K, M(, batch)], b [N, K], c S32 [N] or nullptr, output [N, M(, batch)].  The quantization offsets of a
    // and b are ADDED to the operands, exactly as the NE core does; library callers pass negated zero points.
    void configure(const ITensor *a, const ITensor *b, const ITensor *c, ITensor *output,
                   const GEMMInfo &gemm_info = GEMMInfo());
    static Status validate(const ITensorInfo *a, const ITensorInfo *b, const ITensorInfo *c,
                           const ITensorInfo *output, const GEMMInfo &gemm_info = GEMMInfo());
    // As NEGEMMLowpMatrixMultiplyCore::update_quantization_parameters (…MatrixMultiplyCore.cpp:118-159): after the
    // tensors' QuantizationInfo changed, re-derive a per-tensor QUANTIZE_DOWN_FIXEDPOINT stage from the
    // input / weights / output scales (bounds = type range, offset = output offset) and re-read the operand offsets.
    void update_quantization_parameters();
    // Same, with the output stage given explicitly (per-channel vectors allowed).
    void update_quantization_parameters(const GEMMLowpOutputStageInfo &output_stage);
    void run() override;     // enqueues on the scheduler's stream; does not block
    void prepare() override; // B -> K-major operand + column sums; b may be released afterwards

private:
    struct Impl;
    std::unique_ptr<Impl> _impl;
};
} // namespace arm_compute
