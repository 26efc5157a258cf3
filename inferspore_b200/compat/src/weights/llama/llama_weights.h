// Weight descriptors of a LLaMA decoder layer, under the names and member names the InferSpore
// launchers and unit tests use (reference: src/weights/llama/{attention,ffn,norm,embedding}_weights.h).
// All of them are non-owning views: BaseWeight carries raw device pointers and a NULL bias means
// "no bias".  The four per-struct headers of the reference tree forward to this file.
#pragma once
#include "src/weights/base_weights.h"

// Table [vocab, hidden] read by launchInputEmbedding.
template <typename T>
struct EmbeddingWeight : public BaseWeight<T> {};

// gamma [hidden] of an RMSNorm; launchFusedAddBiasResidualRMSNorm takes the pointer itself.
template <typename T>
struct LayerNormWeight {
    T* gamma = nullptr;
};

// Projections of self-attention.  qkv is the fused [hidden, (heads + 2*kv_heads) * head_size]
// matrix whose bias launchAddFusedQKVBiasTransposeAndRoPE and launchDecoderMaskedMHA add.
template <typename T>
struct LLaMAattentionWeights {
    BaseWeight<T> q, k, v;
    BaseWeight<T> qkv;
    BaseWeight<T> output;
};

// Gated feed-forward: gateAndup is the fused [hidden, 2 * inter] matrix whose output launchAct splits.
template <typename T>
struct LLaMAFFNWeights {
    BaseWeight<T> gate, up, down;
    BaseWeight<T> gateAndup;
};
