// launchConcatKVCache — same name and argument list as the reference
// (src/kernels/concat_past_kv.h:7-14); runs the sm_100a scatter through
// ispore_concat_kv_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"

// k_src, v_src [bs, kv_heads, max_q_len, head_size]; layer_id is a CPU tensor;
// cur_query_length, history_length are device int [bs].
// k_dst, v_dst are the caches.  Two layouts are accepted:
//   5-D {num_layers, bs, kv_heads, max_seq_len, head_size} — the documented one
//       (src/kernels/concat_past_kv.cu:81), max_seq_len = shape[3];
//   4-D {bs, kv_heads, max_seq_len, head_size} — a single-layer cache, which is
//       what tests/unittests/test_concat_kv.cu:81-82 passes; max_seq_len =
//       shape[2] and layer_id must be 0.  (The reference launcher reads shape[3]
//       in both cases and so takes head_size for max_seq_len on the 4-D form.)
template <typename T>
void launchConcatKVCache(TensorWrapper<T>* k_src, TensorWrapper<T>* v_src, TensorWrapper<int>* layer_id,
                         TensorWrapper<int>* cur_query_length, TensorWrapper<int>* history_length,
                         TensorWrapper<T>* k_dst, TensorWrapper<T>* v_dst) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(k_src->shape.size() == 4, "k_src must be [bs, kv_heads, max_q_len, head_size]");
    const int64_t batch_size = k_src->shape[0];
    const int64_t kv_head_num = k_src->shape[1];
    const int64_t max_q_len = k_src->shape[2];
    const int64_t head_size = k_src->shape[3];
    const int64_t layer = layer_id->getVal();
    int64_t num_layers, max_seq_len;
    if (k_dst->shape.size() == 5) {
        num_layers = k_dst->shape[0];
        max_seq_len = k_dst->shape[3];
    } else {
        LLM_CHECK_WITH_INFO(k_dst->shape.size() == 4, "KV cache must be 5-D (with layers) or 4-D (one layer)");
        num_layers = 1;
        max_seq_len = k_dst->shape[2];
    }
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_concat_kv_f16(k_dst->data, v_dst->data, k_src->data, v_src->data, cur_query_length->data,
                                  history_length->data, layer, num_layers, batch_size, kv_head_num, max_q_len,
                                  max_seq_len, head_size, ispore_get_stream());
    else
        rc = ispore_concat_kv_f32((float*)k_dst->data, (float*)v_dst->data, (const float*)k_src->data,
                                  (const float*)v_src->data, cur_query_length->data, history_length->data,
                                  layer, num_layers, batch_size, kv_head_num, max_q_len, max_seq_len, head_size,
                                  ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchConcatKVCache");
}
