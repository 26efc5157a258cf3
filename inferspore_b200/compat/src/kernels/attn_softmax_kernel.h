// launchScaleMaskAndSoftmax — same name and argument list as the reference
// (src/kernels/attn_softmax_kernel.h:7-11); runs the sm_100a kernel through
// ispore_scale_mask_softmax_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"
#include "src/utils/vectorize_utils.h"

// qk, attn_score [bs, heads, q_len, k_len]; mask [bs, q_len, k_len] (1 keep, 0 drop).
// Unlike the reference, odd k_len and k_len > 4096 are accepted for both types.
template <typename T>
void launchScaleMaskAndSoftmax(TensorWrapper<T>* qk, TensorWrapper<T>* mask, TensorWrapper<T>* attn_score,
                               float scale) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(qk->shape.size() == 4, "qk must be [bs, heads, q_len, k_len]");
    const int64_t batch_size = qk->shape[0];
    const int64_t head_nums = qk->shape[1];
    const int64_t q_length = qk->shape[2];
    const int64_t k_length = qk->shape[3];
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_scale_mask_softmax_f16(attn_score->data, qk->data, mask->data, batch_size, head_nums,
                                           q_length, k_length, scale, ispore_get_stream());
    else
        rc = ispore_scale_mask_softmax_f32((float*)attn_score->data, (const float*)qk->data,
                                           (const float*)mask->data, batch_size, head_nums, q_length, k_length,
                                           scale, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchScaleMaskAndSoftmax");
}

// No reference counterpart: the mask builder (src/kernels/build_casual_mask.h:7-10) and the softmax
// above in one launch.  q_lens, k_lens are the int tensors launchBuildCausalMasks takes.
template <typename T>
void launchScaleCausalSoftmax(TensorWrapper<T>* qk, TensorWrapper<int>* q_lens, TensorWrapper<int>* k_lens,
                              TensorWrapper<T>* attn_score, float scale) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(qk->shape.size() == 4, "qk must be [bs, heads, q_len, k_len]");
    LLM_CHECK_WITH_INFO(q_lens->shape[0] == qk->shape[0] && k_lens->shape[0] == qk->shape[0],
                        "q_lens and k_lens must hold one length per batch entry");
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_scale_causal_softmax_f16(attn_score->data, qk->data, q_lens->data, k_lens->data, qk->shape[0],
                                             qk->shape[1], qk->shape[2], qk->shape[3], scale, ispore_get_stream());
    else
        rc = ispore_scale_causal_softmax_f32((float*)attn_score->data, (const float*)qk->data, q_lens->data,
                                             k_lens->data, qk->shape[0], qk->shape[1], qk->shape[2], qk->shape[3],
                                             scale, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchScaleCausalSoftmax");
}
