// RMSNorm weight (reference: src/weights/llama/norm_weights.h).
#pragma once
template <typename T>
struct LayerNormWeight {
    T* gamma;
};
