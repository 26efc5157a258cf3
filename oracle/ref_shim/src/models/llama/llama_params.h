// Stand-in for a header the reference includes (src/kernels/qkv_bias_and_RoPE.h:5)
// but does not ship.  Only used to compile the reference's own sources into
// oracle/_ref/; the fields are the ones src/kernels/qkv_bias_and_RoPE.cu:322-325 reads.
#pragma once
struct LLaMAAttentionStaticParams {
    int rotary_embedding_dim;
    float rotary_embedding_base;
    int max_position_embeddings;
    bool use_dynamic_ntk;
};
