// CUDA counterparts of the QASYMM8 layers a quantized network runs between its convolutions, with the
// signatures of the NEON functions:
//   CUPoolingLayer        NEPoolingLayer        arm_compute/runtime/NEON/functions/NEPoolingLayer.h:48-109
//   CUArithmeticAddition  NEArithmeticAddition  arm_compute/runtime/NEON/functions/NEArithmeticAddition.h:43-109
//   CUActivationLayer     NEActivationLayer     arm_compute/runtime/NEON/functions/NEActivationLayer.h:48-107
//   CUSoftmaxLayer        NESoftmaxLayer        arm_compute/runtime/NEON/functions/NESoftmaxLayer.h:44-99
// QASYMM8 (uint8), NHWC only; results equal the library's scalar oracle (dequantize, float operator, quantize)
// bit for bit, softmax within one step.  run() enqueues on the scheduler's stream and does not block.
#pragma once
#include "arm_compute/core/ITensor.h"
#include "arm_compute/core/Types.h"
#include "arm_compute/function_info/ActivationLayerInfo.h"
#include "arm_compute/function_info/GEMMInfo.h"
#include "arm_compute/runtime/IFunction.h"
#include "arm_compute/runtime/IMemoryManager.h"
#include "arm_compute/runtime/IWeightsManager.h"

#include <memory>

namespace arm_compute
{
class CUPoolingLayer : public IFunction
{
public:
    void          configure(ITensor *input, ITensor *output, const PoolingLayerInfo &pool_info, ITensor *indices = nullptr);
    static Status validate(const ITensorInfo *input, const ITensorInfo *output, const PoolingLayerInfo &pool_info,
                           const ITensorInfo *indices = nullptr);
    void          run() override;

private:
    const ITensor   *_input{nullptr};
    ITensor         *_output{nullptr};
    PoolingLayerInfo _info{};
};

class CUArithmeticAddition : public IFunction
{
public:
    void          configure(const ITensor *input1, const ITensor *input2, ITensor *output, ConvertPolicy policy,
                            const ActivationLayerInfo &act_info = ActivationLayerInfo());
    static Status validate(const ITensorInfo *input1, const ITensorInfo *input2, const ITensorInfo *output,
                           ConvertPolicy policy, const ActivationLayerInfo &act_info = ActivationLayerInfo());
    void          run() override;

private:
    const ITensor      *_input1{nullptr};
    const ITensor      *_input2{nullptr};
    ITensor            *_output{nullptr};
    ActivationLayerInfo _act{};
};

class CUActivationLayer : public IFunction
{
public:
    // output == nullptr: in place, as the NEON function
    void          configure(ITensor *input, ITensor *output, ActivationLayerInfo activation_info);
    static Status validate(const ITensorInfo *input, const ITensorInfo *output, const ActivationLayerInfo &act_info);
    void          run() override;

private:
    ITensor            *_input{nullptr};
    ITensor            *_output{nullptr};
    ActivationLayerInfo _act{};
};

class CUSoftmaxLayer : public IFunction
{
public:
    // the softmax kernel keeps its row in registers and shared memory: no workspace for a memory manager to hold
    explicit CUSoftmaxLayer(std::shared_ptr<IMemoryManager> memory_manager = nullptr) { ARM_COMPUTE_UNUSED(memory_manager); }
    void          configure(ITensor *input, ITensor *output, float beta = 1.0f, int32_t axis = 0);
    static Status validate(const ITensorInfo *input, const ITensorInfo *output, float beta = 1.0f, int32_t axis = 0);
    void          run() override;

private:
    const ITensor *_input{nullptr};
    ITensor       *_output{nullptr};
    float          _beta{1.f};
};

// NEFlattenLayer (arm_compute/runtime/NEON/functions/NEFlattenLayer.h:41-78): [d0, d1, d2, batch] -> [d0*d1*d2, batch].
// The elements keep their order, so for dense tensors the layer is one device-to-device copy.
class CUFlattenLayer : public IFunction
{
public:
    void          configure(const ITensor *input, ITensor *output);
    static Status validate(const ITensorInfo *input, const ITensorInfo *output);
    void          run() override;

private:
    const ITensor *_input{nullptr};
    ITensor       *_output{nullptr};
};
} // namespace arm_compute
