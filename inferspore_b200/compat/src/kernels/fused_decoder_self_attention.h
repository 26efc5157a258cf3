// Drop-in for the reference's src/kernels/fused_decoder_self_attention.h: same launcher name and
// arguments (:10-18), forwarding to the C ABI of libispore_kernels.  The reference launcher takes
// no scratch; this one keeps a per-thread device buffer that grows on demand so that long
// sequences at small batch can be split over several CTAs.  Build with
// -DISPORE_MHA_NO_WORKSPACE to forbid that allocation (one CTA per sequence and head group then).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/models/llama/llama_params.h"
#include "src/utils/tensor.h"
#include "src/utils/vectorize_utils.h"
#include "src/weights/base_weights.h"

namespace ispore_compat {
inline void* mha_workspace(int64_t bytes) {
#ifdef ISPORE_MHA_NO_WORKSPACE
    (void)bytes;
    return nullptr;
#else
    thread_local void* buf = nullptr;
    thread_local int64_t cap = 0;
    if (bytes > cap) {
        if (buf) cudaFree(buf);
        buf = nullptr;
        cap = 0;
        if (cudaMalloc(&buf, static_cast<size_t>(bytes)) != cudaSuccess) {
            cudaGetLastError();
            buf = nullptr;
            return nullptr;  // the launcher then runs unsplit
        }
        cap = bytes;
    }
    return buf;
#endif
}
}  // namespace ispore_compat

template <typename T>
void launchDecoderMaskedMHA(TensorWrapper<T>* qkv_buf, BaseWeight<T>& qkv, TensorWrapper<int>* layer_id,
                            TensorWrapper<T>* k_cache, TensorWrapper<T>* v_cache, TensorWrapper<bool>* finished,
                            TensorWrapper<int>* step, TensorWrapper<T>* mha_output,
                            LLaMAAttentionStaticParams& static_params) {
    (void)finished;  // unused by the reference kernel as well
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(qkv_buf->shape.size() == 3, "qkv_buf must be [batch, qkv_head_num, head_size]");
    LLM_CHECK_WITH_INFO(k_cache->shape.size() == 5, "k_cache must be [layers, batch, kv_heads, max_seq_len, head_size]");
    const int64_t batch_size = qkv_buf->shape[0];
    const int64_t qkv_head_num = qkv_buf->shape[1];
    const int64_t head_size = qkv_buf->shape[2];
    const int64_t kv_head_num = k_cache->shape[2];
    const int64_t max_seq_len = k_cache->shape[3];
    const int64_t head_num = qkv_head_num - 2 * kv_head_num;
    const int64_t cur_step = step->getVal();
    const int64_t layer = layer_id->getVal();
    // The reference's own test declares the cache with a leading extent of 0 (its layer id);
    // only a positive extent is checked against the layer.
    const int64_t num_layers = k_cache->shape[0] > 0 ? k_cache->shape[0] : 0;
    const int64_t ws_bytes =
        ispore_decoder_masked_mha_workspace_bytes(batch_size, head_num, kv_head_num, head_size, cur_step);
    void* ws = ws_bytes > 0 ? ispore_compat::mha_workspace(ws_bytes) : nullptr;
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_decoder_masked_mha_f16(mha_output->data, qkv_buf->data, qkv.bias, k_cache->data, v_cache->data,
                                           layer, num_layers, batch_size, head_num, kv_head_num, max_seq_len,
                                           head_size, cur_step, static_params.rotary_embedding_dim,
                                           static_params.rotary_embedding_base, static_cast<float>(cur_step), ws,
                                           ws ? ws_bytes : 0, ispore_get_stream());
    else
        rc = ispore_decoder_masked_mha_f32((float*)mha_output->data, (const float*)qkv_buf->data,
                                           (const float*)qkv.bias, (float*)k_cache->data, (float*)v_cache->data,
                                           layer, num_layers, batch_size, head_num, kv_head_num, max_seq_len,
                                           head_size, cur_step, static_params.rotary_embedding_dim,
                                           static_params.rotary_embedding_base, static_cast<float>(cur_step), ws,
                                           ws ? ws_bytes : 0, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchDecoderMaskedMHA");
}
