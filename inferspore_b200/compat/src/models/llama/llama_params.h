// Attention parameter structs.  The reference includes this header from
// src/kernels/qkv_bias_and_RoPE.h:5 and src/kernels/fused_decoder_self_attention.h:6
// but does not ship it; the fields are the ones its sources read
// (src/kernels/qkv_bias_and_RoPE.cu:322-325, tests/unittests/test_bias_and_RoPE.cu:163-167,
// src/utils/model_utils.h:25-29).
#pragma once

struct LLaMAAttentionStaticParams {
    int rotary_embedding_dim;
    float rotary_embedding_base;
    int max_position_embeddings;
    bool use_dynamic_ntk;  // placeholder upstream; ignored
};

struct LLaMAAttentionDynParams {
    int batch_size;
    int num_tokens;
    int max_q_len;
    int max_k_len;
    int num_layers;
    bool is_ctx = false;
};
