// launchCalPaddingoffset — same name and argument list as the reference
// (src/kernels/cal_paddingoffset.h:8-11); runs the sm_100a scan through
// ispore_cal_padding_offset.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/macro.h"
#include "src/utils/tensor.h"

// padding_offset [bs, max_q_len], cum_seqlens [bs + 1], input_lengths [bs] (all device int).
inline void launchCalPaddingoffset(TensorWrapper<int>* padding_offset, TensorWrapper<int>* cum_seqlens,
                                   TensorWrapper<int>* input_lengths) {
    const int batch_size = padding_offset->shape[0];
    const int max_q_len = padding_offset->shape[1];
    LLM_CHECK_WITH_INFO(batch_size == input_lengths->shape[0],
                        "input lenghts numbers should equal to padding offset bs dim!");
    LLM_CHECK_WITH_INFO(batch_size == cum_seqlens->shape[0] - 1,
                        "cum seqlen numbers should equal to padding offset bs dim + 1!");
    ispore_compat::throw_on_error(
        ispore_cal_padding_offset(padding_offset->data, cum_seqlens->data, input_lengths->data, batch_size, max_q_len,
                                  ispore_get_stream()),
        "launchCalPaddingoffset");
}
