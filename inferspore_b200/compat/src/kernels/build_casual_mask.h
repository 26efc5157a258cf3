// launchBuildCausalMasks — same name and argument list as the reference
// (src/kernels/build_casual_mask.h:7-10); runs the sm_100a kernel through
// ispore_build_causal_mask_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/macro.h"
#include "src/utils/tensor.h"

// mask [bs, max_q_len, max_k_len]; q_lens, k_lens: device int [bs].
template <typename T>
void launchBuildCausalMasks(TensorWrapper<T>* mask, TensorWrapper<int>* q_lens, TensorWrapper<int>* k_lens) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(mask->shape.size() == 3, "mask must be [bs, max_q_len, max_k_len]");
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_build_causal_mask_f16(mask->data, q_lens->data, k_lens->data, mask->shape[0], mask->shape[1],
                                          mask->shape[2], ispore_get_stream());
    else
        rc = ispore_build_causal_mask_f32((float*)mask->data, q_lens->data, k_lens->data, mask->shape[0],
                                          mask->shape[1], mask->shape[2], ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchBuildCausalMasks");
}
