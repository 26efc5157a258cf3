// Weight descriptors with the names and fields of the InferSpore sources
// (reference: src/weights/base_weights.h).  Non-owning: data/bias are raw
// device pointers; a NULL bias means "no bias".  Unlike the reference struct the
// pointers start out NULL, so a default-constructed weight (as in
// tests/unittests/test_fused_addresidual_norm.cu:118) means "no bias" instead of
// carrying an indeterminate pointer into a kernel.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>
#include <type_traits>
#include <vector>

enum class WeightType { FP32_W, FP16_W, INT8_W, UNSUPPORTED_W };

template <typename T>
inline WeightType getWeightType() {
    using U = typename std::remove_cv<T>::type;
    if (std::is_same<U, float>::value) return WeightType::FP32_W;
    if (std::is_same<U, half>::value) return WeightType::FP16_W;
    if (std::is_same<U, int8_t>::value) return WeightType::INT8_W;
    return WeightType::UNSUPPORTED_W;
}

template <typename T>
struct BaseWeight {
    std::vector<int> shape;
    T* data = nullptr;
    WeightType type = getWeightType<T>();
    T* bias = nullptr;
};
