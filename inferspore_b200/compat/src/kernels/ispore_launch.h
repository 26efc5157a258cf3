// Glue between the InferSpore launch templates and the C ABI in
// ispore_kernels.h.  Not part of the reference's header set.
#pragma once
#include <cuda_fp16.h>

#include <stdexcept>
#include <string>
#include <type_traits>

#include "ispore_kernels.h"

namespace ispore_compat {

// A failed C-ABI call becomes std::runtime_error, the exception type the
// reference's LLM_CHECK raises (src/utils/macro.h:90-110).
inline void throw_on_error(int status, const char* launcher) {
    if (status == ISPORE_OK) return;
    throw std::runtime_error(std::string("[oneLLM][ERROR] ") + launcher + " failed (" +
                             std::to_string(status) + "): " + ispore_last_error_string());
}

template <typename T>
struct is_half : std::is_same<typename std::remove_cv<T>::type, half> {};

template <typename T>
constexpr void require_float_or_half() {
    static_assert(std::is_same<typename std::remove_cv<T>::type, float>::value || is_half<T>::value,
                  "the layer kernels are instantiated for float and half only");
}

}  // namespace ispore_compat
