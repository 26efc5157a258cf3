// launchAddFusedQKVBiasTransposeAndRoPE and launchRoPE — same names and
// argument lists as the reference (src/kernels/qkv_bias_and_RoPE.h:10-25);
// they run the sm_100a kernels through ispore_qkv_bias_rope_transpose_* and
// ispore_rope_decode_*.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/models/llama/llama_params.h"
#include "src/utils/tensor.h"
#include "src/utils/vectorize_utils.h"
#include "src/weights/base_weights.h"

// Prefill.  QKV [num_tokens, head_num + 2*kv_head_num, head_size] (packed, no
// padding) -> q_buf [bs, head_num, seq_len, head_size], k_buf / v_buf
// [bs, kv_head_num, seq_len, head_size]; qkv.bias (nullable) is added first,
// q and k are rotated at position history_length[b] + s.
template <typename T>
void launchAddFusedQKVBiasTransposeAndRoPE(TensorWrapper<T>* q_buf, TensorWrapper<T>* k_buf,
                                           TensorWrapper<T>* v_buf, TensorWrapper<T>* QKV,
                                           BaseWeight<T>& qkv, TensorWrapper<int>* padding_offset,
                                           TensorWrapper<int>* history_length,
                                           TensorWrapper<int>* input_length,
                                           LLaMAAttentionStaticParams& params) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(QKV->shape.size() == 3 && q_buf->shape.size() == 4,
                        "QKV must be [tokens, heads, head_size] and q_buf [bs, heads, seq, head_size]");
    const int64_t token_num = QKV->shape[0];
    const int64_t qkv_head_num = QKV->shape[1];
    const int64_t head_size = QKV->shape[2];
    const int64_t batch_size = q_buf->shape[0];
    const int64_t head_num = q_buf->shape[1];
    const int64_t seq_len = q_buf->shape[2];
    const int64_t kv_head_num = (qkv_head_num - head_num) / 2;
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_qkv_bias_rope_transpose_f16(
            q_buf->data, k_buf->data, v_buf->data, QKV->data, qkv.bias, padding_offset->data,
            history_length->data, input_length ? input_length->data : nullptr, batch_size, seq_len, token_num,
            head_num, kv_head_num, head_size, params.rotary_embedding_dim, params.rotary_embedding_base,
            params.max_position_embeddings, params.use_dynamic_ntk ? 1 : 0, ispore_get_stream());
    else
        rc = ispore_qkv_bias_rope_transpose_f32(
            (float*)q_buf->data, (float*)k_buf->data, (float*)v_buf->data, (const float*)QKV->data,
            (const float*)qkv.bias, padding_offset->data, history_length->data,
            input_length ? input_length->data : nullptr, batch_size, seq_len, token_num, head_num, kv_head_num,
            head_size, params.rotary_embedding_dim, params.rotary_embedding_base,
            params.max_position_embeddings, params.use_dynamic_ntk ? 1 : 0, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchAddFusedQKVBiasTransposeAndRoPE");
}

// Decode step.  qkv_buf [batch, head_num + 2*kv_head_num, head_size] is rotated
// in place at position step-1; `step` is a CPU tensor, as in the reference.
// The reference hard-codes 32 q heads out of 96 and batch 1; here any batch is
// accepted and MHA (kv_head_num == head_num == heads/3) is assumed, which is
// what the reference's constants describe.
template <typename T>
void launchRoPE(TensorWrapper<T>* qkv_buf, TensorWrapper<int>* step, LLaMAAttentionStaticParams& static_params) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(qkv_buf->shape.size() == 3, "qkv_buf must be [batch, qkv_head_num, head_size]");
    const int64_t batch_size = qkv_buf->shape[0];
    const int64_t qkv_head_num = qkv_buf->shape[1];
    const int64_t head_size = qkv_buf->shape[2];
    LLM_CHECK_WITH_INFO(qkv_head_num % 3 == 0, "launchRoPE expects head_num == kv_head_num (heads divisible by 3)");
    const int64_t head_num = qkv_head_num / 3;
    const int cur_step = step->getVal();
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_rope_decode_f16(qkv_buf->data, batch_size, head_num, head_num, head_size, cur_step,
                                    static_params.rotary_embedding_dim, static_params.rotary_embedding_base,
                                    ispore_get_stream());
    else
        rc = ispore_rope_decode_f32((float*)qkv_buf->data, batch_size, head_num, head_num, head_size, cur_step,
                                    static_params.rotary_embedding_dim, static_params.rotary_embedding_base,
                                    ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchRoPE");
}
