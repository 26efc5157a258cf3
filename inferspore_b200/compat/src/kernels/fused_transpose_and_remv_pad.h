// launchTransposeOutRemovePadding — the name and argument list the reference declares
// (src/kernels/fused_transpose_and_remv_pad.h:7-10) but never defines; semantics from
// tests/unittests/test_fused_trans_remv_pad.cu:3-4.  Runs through
// ispore_transpose_remove_padding_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"

// qkv_buf_w_pad [bs, heads, seq_len, head_size]; padding_offset [num_tokens];
// qkv_buf_wo_pad_1 [num_tokens, heads, head_size].
template <typename T>
void launchTransposeOutRemovePadding(TensorWrapper<T>* qkv_buf_w_pad, TensorWrapper<int>* padding_offset,
                                     TensorWrapper<T>* qkv_buf_wo_pad_1) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(qkv_buf_w_pad->shape.size() == 4, "input must be [bs, heads, seq_len, head_size]");
    const int64_t batch = qkv_buf_w_pad->shape[0], heads = qkv_buf_w_pad->shape[1];
    const int64_t seq_len = qkv_buf_w_pad->shape[2], head_size = qkv_buf_w_pad->shape[3];
    const int64_t num_tokens = qkv_buf_wo_pad_1->shape[0];
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_transpose_remove_padding_f16(qkv_buf_wo_pad_1->data, qkv_buf_w_pad->data, padding_offset->data,
                                                 batch, heads, seq_len, head_size, num_tokens, ispore_get_stream());
    else
        rc = ispore_transpose_remove_padding_f32((float*)qkv_buf_wo_pad_1->data, (const float*)qkv_buf_w_pad->data,
                                                 padding_offset->data, batch, heads, seq_len, head_size, num_tokens,
                                                 ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchTransposeOutRemovePadding");
}
