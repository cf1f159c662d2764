// CUDA counterpart of NEFullyConnectedLayer on quantized tensors
// (arm_compute/runtime/NEON/functions/NEFullyConnectedLayer.h:83-168; operator src/cpu/operators/CpuFullyConnected.cpp:
// negated offsets :97-102, the output stage from the three quantizations :165-170, then CpuGemmLowpMatrixMultiplyCore).
//   input   QASYMM8 / QASYMM8_SIGNED, [num_inputs, batch] or a 4-D activation whose first three dimensions flatten
//           to num_inputs (NHWC order, as the weights were trained)
//   weights 8-bit quantized (per-tensor or per-channel), TensorShape(num_inputs, num_outputs) when
//           fc_info.transpose_weights (the default: one row per output neuron), TensorShape(num_outputs, num_inputs)
//           otherwise; constant: consumed by prepare()
//   biases  S32 [num_outputs] or nullptr;   output  input's data type, [num_outputs, batch]
// A fully connected layer is the 1x1 convolution of a 1x1 image with num_inputs channels, so the function runs on
// the convolution plan of the C ABI (plain-GEMM lowering).
#pragma once
#include "arm_compute/core/ITensor.h"
#include "arm_compute/core/Types.h"
#include "arm_compute/function_info/ActivationLayerInfo.h"
#include "arm_compute/function_info/FullyConnectedLayerInfo.h"
#include "arm_compute/function_info/GEMMInfo.h"
#include "arm_compute/runtime/IFunction.h"
#include "arm_compute/runtime/IMemoryManager.h"
#include "arm_compute/runtime/IWeightsManager.h"

#include <memory>

namespace arm_compute
{
class CUFullyConnectedLayer : public IFunction
{
public:
    CUFullyConnectedLayer(std::shared_ptr<IMemoryManager> memory_manager = nullptr, IWeightsManager *weights_manager = nullptr);
    CUFullyConnectedLayer(const CUFullyConnectedLayer &)            = delete;
    CUFullyConnectedLayer &operator=(const CUFullyConnectedLayer &) = delete;
    ~CUFullyConnectedLayer();
    void          configure(const ITensor *input, const ITensor *weights, const ITensor *biases, ITensor *output,
                            FullyConnectedLayerInfo fc_info = FullyConnectedLayerInfo(),
                            const WeightsInfo &weights_info = WeightsInfo());
    static Status validate(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                           const ITensorInfo *output, FullyConnectedLayerInfo fc_info = FullyConnectedLayerInfo(),
                           const WeightsInfo &weights_info = WeightsInfo());
    void          run() override;
    void          prepare() override;

private:
    struct Impl;
    std::unique_ptr<Impl> _impl;
};
} // namespace arm_compute
