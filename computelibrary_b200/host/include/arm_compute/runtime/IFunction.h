// Stand-in for arm_compute/runtime/IFunction.h:33-62.
#pragma once
namespace arm_compute
{
class IFunction
{
public:
    virtual ~IFunction() = default;
    virtual void run()   = 0; // a device backend enqueues and returns; results are valid after sync()
    virtual void prepare() {}
};
} // namespace arm_compute
