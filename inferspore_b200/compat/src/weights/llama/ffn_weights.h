// Feed-forward weights (reference: src/weights/llama/ffn_weights.h).
#pragma once
#include "src/weights/base_weights.h"
template <typename T>
struct LLaMAFFNWeights {
    BaseWeight<T> gate;
    BaseWeight<T> up;
    BaseWeight<T> down;
    BaseWeight<T> gateAndup;
};
