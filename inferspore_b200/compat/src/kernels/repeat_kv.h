// launchRepeatKVCache — same name and argument list as the reference
// (src/kernels/repeat_kv.h:7-13); runs the sm_100a kernel through ispore_repeat_kv_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"

// k/v_cache_src {num_layers, bs, kv_heads, max_seq_len, head_size}; context_length device int [bs];
// layer_id CPU tensor; k/v_cache_dst {bs, heads, max_k_len, head_size}.
template <typename T>
void launchRepeatKVCache(TensorWrapper<T>* k_cache_src, TensorWrapper<T>* v_cache_src,
                         TensorWrapper<int>* context_length, TensorWrapper<int>* layer_id,
                         TensorWrapper<T>* k_cache_dst, TensorWrapper<T>* v_cache_dst) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(k_cache_src->shape.size() == 5 && k_cache_dst->shape.size() == 4,
                        "caches must be 5-D (with layers) and the destination 4-D");
    const int64_t batch = context_length->shape[0];
    const int64_t num_layers = k_cache_src->shape[0], kv_heads = k_cache_src->shape[2];
    const int64_t max_seq_len = k_cache_src->shape[3];
    const int64_t heads = k_cache_dst->shape[1], max_k_len = k_cache_dst->shape[2], head_size = k_cache_dst->shape[3];
    const int64_t layer = layer_id->getVal();
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_repeat_kv_f16(k_cache_dst->data, v_cache_dst->data, k_cache_src->data, v_cache_src->data,
                                  context_length->data, layer, num_layers, batch, kv_heads, heads, max_seq_len,
                                  max_k_len, head_size, ispore_get_stream());
    else
        rc = ispore_repeat_kv_f32((float*)k_cache_dst->data, (float*)v_cache_dst->data, (const float*)k_cache_src->data,
                                  (const float*)v_cache_src->data, context_length->data, layer, num_layers, batch,
                                  kv_heads, heads, max_seq_len, max_k_len, head_size, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchRepeatKVCache");
}
