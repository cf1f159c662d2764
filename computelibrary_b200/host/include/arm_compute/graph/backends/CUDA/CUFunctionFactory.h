// Maps graph nodes to CU* functions (precedent: arm_compute/graph/backends/NEON/NEFunctionFactory.h) and validates
// them (NENodeValidator.h).  The node types a quantized ResNet-50 uses are covered: Convolution, FullyConnected,
// Pooling, Eltwise (Add), Activation, Flatten, Softmax; Input / Output / Const nodes carry no function.
#pragma once
#include "arm_compute/core/Error.h"
#include "arm_compute/runtime/IFunction.h"

#include <memory>

namespace arm_compute
{
namespace graph
{
class INode;
class GraphContext;

namespace backends
{
class CUFunctionFactory final
{
public:
    static std::unique_ptr<arm_compute::IFunction> create(INode *node, GraphContext &ctx);
};

class CUNodeValidator final
{
public:
    static Status validate(INode *node);
};
} // namespace backends
} // namespace graph
} // namespace arm_compute
