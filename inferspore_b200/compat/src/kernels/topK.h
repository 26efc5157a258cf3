// launchTopKforBeamSearch — same name and argument list as the reference
// (src/kernels/topK.h:41-46); runs the sm_100a two-round top-K through
// ispore_topk_{f32,f16}.  launchSampling is an addition in the same style (the
// reference has no sampling kernel).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"

// probs [rows, vocab]; topk_ids / topk_vals: scratch [rows, slices, K] (the
// reference allocates slices = 8); final_topk_ids / final_topk_vals [rows, K].
// K comes from final_topk_ids->shape[1] (the reference compiles K = 5 in).
// Output order: value descending, ties on the lower index.
template <typename T>
void launchTopKforBeamSearch(TensorWrapper<T>* probs, TensorWrapper<int>* topk_ids, TensorWrapper<T>* topk_vals,
                             TensorWrapper<int>* final_topk_ids, TensorWrapper<T>* final_topk_vals) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(probs->shape.size() == 2 && final_topk_ids->shape.size() == 2,
                        "probs must be [rows, vocab] and final_topk_ids [rows, K]");
    const int64_t rows = probs->shape[0];
    const int64_t vocab = probs->shape[1];
    const int K = final_topk_ids->shape[1];
    // Scratch capacity in K-sized lists per row, from whatever shape the caller gave.
    const int64_t scratch_elems = topk_ids->numel();
    const int64_t slices = (rows > 0 && K > 0) ? scratch_elems / (rows * K) : 0;
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_topk_f16(probs->data, rows, vocab, K, topk_ids->data, topk_vals->data, (int)slices,
                             final_topk_ids->data, final_topk_vals->data, 0, nullptr, 1.0f, nullptr,
                             ispore_get_stream());
    else
        rc = ispore_topk_f32((const float*)probs->data, rows, vocab, K, topk_ids->data, (float*)topk_vals->data,
                             (int)slices, final_topk_ids->data, (float*)final_topk_vals->data, 0, nullptr, 1.0f,
                             nullptr, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchTopKforBeamSearch");
}

// topk_id / topk_val [rows, K] (descending), uniform [rows] in [0,1) drawn by the
// caller, output_id [rows]: inverse-CDF draw from softmax(topk_val / temperature).
template <typename T>
void launchSampling(TensorWrapper<int>* topk_id, TensorWrapper<T>* topk_val, TensorWrapper<float>* uniform,
                    TensorWrapper<int>* output_id, float temperature) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(topk_id->shape.size() == 2, "topk_id must be [rows, K]");
    const int64_t rows = topk_id->shape[0];
    const int K = topk_id->shape[1];
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_sampling_f16(topk_id->data, topk_val->data, uniform->data, output_id->data, rows, K,
                                 temperature, ispore_get_stream());
    else
        rc = ispore_sampling_f32(topk_id->data, (const float*)topk_val->data, uniform->data, output_id->data,
                                 rows, K, temperature, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchSampling");
}
