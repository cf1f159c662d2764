// CUDA counterpart of NEGEMMLowpOutputStage (arm_compute/runtime/NEON/functions/NEGEMMLowpOutputStage.h:85-102):
// S32 [N, M] (+ S32 bias [N]) -> QASYMM8 / QASYMM8_SIGNED with QUANTIZE_DOWN_FIXEDPOINT.
#pragma once
#include "arm_compute/core/ITensor.h"
#include "arm_compute/core/Types.h"
#include "arm_compute/function_info/ActivationLayerInfo.h"
#include "arm_compute/function_info/GEMMInfo.h"
#include "arm_compute/runtime/IFunction.h"
#include "arm_compute/runtime/IMemoryManager.h"
#include "arm_compute/runtime/IWeightsManager.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"

namespace arm_compute
{
class CUGEMMLowpOutputStage : public IFunction
{
public:
    void          configure(const ITensor *input, const ITensor *bias, ITensor *output, const GEMMLowpOutputStageInfo &info);
    static Status validate(const ITensorInfo *input, const ITensorInfo *bias, const ITensorInfo *output,
                           const GEMMLowpOutputStageInfo &info);
    void          run() override;

private:
    CUOperand               _input{}, _bias{}, _output{};
    GEMMLowpOutputStageInfo _info{};
    void                   *_d_mults{nullptr}; // per-channel vectors on the device
    void                   *_d_shifts{nullptr};

public:
    ~CUGEMMLowpOutputStage();
};
} // namespace arm_compute
