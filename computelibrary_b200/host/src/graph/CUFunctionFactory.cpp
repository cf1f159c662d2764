#include "arm_compute/graph/backends/CUDA/CUFunctionFactory.h"

#include "arm_compute/graph/backends/CUDA/CUDeviceBackend.h"
#include "arm_compute/graph/backends/FunctionHelpers.h"
#include "arm_compute/graph/backends/ValidateHelpers.h"
#include "arm_compute/graph/Graph.h"
#include "arm_compute/graph/GraphContext.h"
#include "arm_compute/graph/nodes/Nodes.h"
#include "arm_compute/runtime/CUDA/CUTensor.h"
#include "arm_compute/runtime/CUDA/functions/CUFullyConnectedLayer.h"
#include "arm_compute/runtime/CUDA/functions/CUGEMMConvolutionLayer.h"
#include "arm_compute/runtime/CUDA/functions/CUQuantizedLayers.h"

#include "support/Cast.h"

using namespace arm_compute::utils::cast;

namespace arm_compute
{
namespace graph
{
namespace backends
{
namespace
{
// What the templated helpers of FunctionHelpers.h need to know about the target (precedent: NETargetInfo)
struct CUTargetInfo
{
    using TensorType         = arm_compute::ITensor;
    using SrcTensorType      = const arm_compute::ITensor;
    using TensorConcreteType = arm_compute::CUTensor;
    static Target TargetType;
};
Target CUTargetInfo::TargetType = CUDATarget;

// Stand-in for function slots of the helpers' type collections that this backend does not fill: instantiating the
// helper needs a type; reaching it at run time is an error that names the operation.
struct CUUnsupported : public IFunction
{
    template <typename... Args>
    void configure(Args &&...)
    {
        ARM_COMPUTE_ERROR("operation not implemented by the CUDA backend");
    }
    template <typename... Args>
    static Status validate(Args &&...)
    {
        return Status(ErrorCode::RUNTIME_ERROR, "operation not implemented by the CUDA backend");
    }
    void run() override
    {
    }
};

// Every convolution method runs on the same kernels here: the "direct" and "Winograd" slots forward to the GEMM layer
class CUDirectConvolutionLayer final : public CUGEMMConvolutionLayer
{
public:
    using CUGEMMConvolutionLayer::CUGEMMConvolutionLayer;
    void configure(ITensor *input, const ITensor *weights, const ITensor *biases, ITensor *output, const PadStrideInfo &conv_info,
                   const ActivationLayerInfo &act_info = ActivationLayerInfo())
    {
        CUGEMMConvolutionLayer::configure(input, weights, biases, output, conv_info, WeightsInfo(), Size2D(1U, 1U), act_info);
    }
    static Status validate(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                           const ITensorInfo *output, const PadStrideInfo &conv_info,
                           const ActivationLayerInfo &act_info = ActivationLayerInfo())
    {
        return CUGEMMConvolutionLayer::validate(input, weights, biases, output, conv_info, WeightsInfo(), Size2D(1U, 1U), act_info);
    }
};

class CUWinogradConvolutionLayer final : public CUGEMMConvolutionLayer
{
public:
    using CUGEMMConvolutionLayer::CUGEMMConvolutionLayer;
    void configure(const ITensor *input, const ITensor *weights, const ITensor *biases, ITensor *output,
                   const PadStrideInfo &conv_info, const ActivationLayerInfo &act_info = ActivationLayerInfo(),
                   bool enable_fast_math = false)
    {
        CUGEMMConvolutionLayer::configure(input, weights, biases, output, conv_info, WeightsInfo(), Size2D(1U, 1U), act_info,
                                          enable_fast_math);
    }
    static Status validate(const ITensorInfo *input, const ITensorInfo *weights, const ITensorInfo *biases,
                           const ITensorInfo *output, const PadStrideInfo &conv_info,
                           const ActivationLayerInfo &act_info = ActivationLayerInfo(), bool enable_fast_math = false)
    {
        return CUGEMMConvolutionLayer::validate(input, weights, biases, output, conv_info, WeightsInfo(), Size2D(1U, 1U), act_info,
                                                enable_fast_math);
    }
};

struct CUConvolutionLayerFunctions
{
    using GenericConvolutionLayer  = CUGEMMConvolutionLayer;
    using GEMMConvolutionLayer     = CUGEMMConvolutionLayer;
    using DirectConvolutionLayer   = CUDirectConvolutionLayer;
    using WinogradConvolutionLayer = CUWinogradConvolutionLayer;
};

struct CUEltwiseFunctions
{
    using Addition       = CUArithmeticAddition;
    using Subtraction    = CUUnsupported;
    using Multiplication = CUUnsupported;
    using Maximum        = CUUnsupported;
    using Division       = CUUnsupported;
};

struct CUEltwiseLayerFunctions // the names ValidateHelpers.h uses
{
    using ArithmeticAddition      = CUArithmeticAddition;
    using ArithmeticSubtraction   = CUUnsupported;
    using PixelWiseMultiplication = CUUnsupported;
    using ElementwiseMax          = CUUnsupported;
    using ArithmeticDivision      = CUUnsupported;
};

Status unsupported(const INode *node)
{
    return Status(ErrorCode::RUNTIME_ERROR, "Unsupported operation on the CUDA backend: node type " +
                                                std::to_string(static_cast<int>(node->type())));
}
} // namespace

std::unique_ptr<IFunction> CUFunctionFactory::create(INode *node, GraphContext &ctx)
{
    if (node == nullptr)
    {
        return nullptr;
    }
    switch (node->type())
    {
        case NodeType::ActivationLayer:
            return detail::create_activation_layer<CUActivationLayer, CUTargetInfo>(*polymorphic_downcast<ActivationLayerNode *>(node));
        case NodeType::ConvolutionLayer:
            return detail::create_convolution_layer<CUConvolutionLayerFunctions, CUTargetInfo>(
                *polymorphic_downcast<ConvolutionLayerNode *>(node), ctx);
        case NodeType::EltwiseLayer:
            return detail::create_eltwise_layer<CUEltwiseFunctions, CUTargetInfo>(*polymorphic_downcast<EltwiseLayerNode *>(node));
        case NodeType::FlattenLayer:
            return detail::create_flatten_layer<CUFlattenLayer, CUTargetInfo>(*polymorphic_downcast<FlattenLayerNode *>(node));
        case NodeType::FullyConnectedLayer:
            return detail::create_fully_connected_layer<CUFullyConnectedLayer, CUTargetInfo>(
                *polymorphic_downcast<FullyConnectedLayerNode *>(node), ctx);
        case NodeType::PoolingLayer:
            return detail::create_pooling_layer<CUPoolingLayer, CUTargetInfo>(*polymorphic_downcast<PoolingLayerNode *>(node));
        case NodeType::SoftmaxLayer:
            return detail::create_softmax_layer<CUSoftmaxLayer, CUTargetInfo>(*polymorphic_downcast<SoftmaxLayerNode *>(node), ctx);
        case NodeType::Input:
        case NodeType::Output:
        case NodeType::Const:
            return nullptr; // no function: the graph manager calls their accessors
        default:
            ARM_COMPUTE_ERROR("Unsupported node type on the CUDA backend");
            return nullptr;
    }
}

Status CUNodeValidator::validate(INode *node)
{
    if (node == nullptr)
    {
        return Status{};
    }
    switch (node->type())
    {
        case NodeType::ConvolutionLayer:
            return detail::validate_convolution_layer<CUGEMMConvolutionLayer, CUDirectConvolutionLayer, CUGEMMConvolutionLayer,
                                                      CUWinogradConvolutionLayer>(*polymorphic_downcast<ConvolutionLayerNode *>(node));
        case NodeType::EltwiseLayer:
            return detail::validate_eltwise_Layer<CUEltwiseLayerFunctions>(*polymorphic_downcast<EltwiseLayerNode *>(node));
        case NodeType::ActivationLayer:
        case NodeType::FlattenLayer:
        case NodeType::FullyConnectedLayer:
        case NodeType::PoolingLayer:
        case NodeType::SoftmaxLayer:
        case NodeType::Input:
        case NodeType::Output:
        case NodeType::Const:
            return Status{}; // checked by the function's own validate() inside configure()
        default:
            return unsupported(node);
    }
}
} // namespace backends
} // namespace graph
} // namespace arm_compute
