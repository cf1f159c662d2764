// Minimal stand-in for arm_compute/core/Error.h (Status, ErrorCode and the throw / return macros the CUDA
// function family uses).  Inside the Compute Library tree the real header is used instead.
#pragma once
#include <stdexcept>
#include <string>

namespace arm_compute
{
enum class ErrorCode
{
    OK,
    RUNTIME_ERROR,
    UNSUPPORTED_EXTENSION_USE
};

class Status
{
public:
    Status() = default;
    Status(ErrorCode code, std::string description = "") : _code(code), _description(std::move(description)) {}
    ErrorCode          error_code() const { return _code; }
    const std::string &error_description() const { return _description; }
    explicit           operator bool() const noexcept { return _code == ErrorCode::OK; }
    void               throw_if_error() const
    {
        if (!bool(*this))
        {
            throw std::runtime_error(_description);
        }
    }

private:
    ErrorCode   _code{ErrorCode::OK};
    std::string _description{};
};
} // namespace arm_compute

#define ARM_COMPUTE_RETURN_ERROR_ON_MSG(cond, msg)                                          \
    do                                                                                      \
    {                                                                                       \
        if (cond)                                                                           \
        {                                                                                   \
            return ::arm_compute::Status(::arm_compute::ErrorCode::RUNTIME_ERROR, (msg));   \
        }                                                                                   \
    } while (false)
#define ARM_COMPUTE_RETURN_ERROR_ON(cond) ARM_COMPUTE_RETURN_ERROR_ON_MSG(cond, #cond)
#define ARM_COMPUTE_RETURN_ON_ERROR(status)  \
    do                                       \
    {                                        \
        const auto _st = (status);           \
        if (!bool(_st))                      \
        {                                    \
            return _st;                      \
        }                                    \
    } while (false)
#define ARM_COMPUTE_ERROR_THROW_ON(status) (status).throw_if_error()
#define ARM_COMPUTE_ERROR_ON_MSG(cond, msg)       \
    do                                            \
    {                                             \
        if (cond)                                 \
        {                                         \
            throw std::runtime_error(msg);        \
        }                                         \
    } while (false)
#define ARM_COMPUTE_ERROR_ON(cond) ARM_COMPUTE_ERROR_ON_MSG(cond, #cond)
#define ARM_COMPUTE_ERROR_ON_NULLPTR(...)                                     \
    do                                                                        \
    {                                                                         \
        const void *_ptrs[] = {__VA_ARGS__};                                  \
        for (const void *_p : _ptrs)                                          \
        {                                                                     \
            if (_p == nullptr) throw std::runtime_error("nullptr argument");  \
        }                                                                     \
    } while (false)
#define ARM_COMPUTE_ERROR(msg) throw std::runtime_error(msg)
#define ARM_COMPUTE_UNUSED(...) (void)sizeof(0, ##__VA_ARGS__)
