// Embedding table [vocab, hidden] (reference: src/weights/llama/embedding_weights.h).
#pragma once
#include "src/weights/base_weights.h"
template <typename T>
struct EmbeddingWeight : public BaseWeight<T> {};
