// launchFusedAddBiasResidualRMSNorm — same name and argument list as the
// reference (src/kernels/fused_addresidual_norm.h:9-15); runs the sm_100a
// kernel through ispore_add_residual_rmsnorm_{f32,f16}.
// launchRMSNorm is an addition in the same style (the reference has no plain
// RMSNorm launcher; it reaches that behaviour through a NULL residual).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"
#include "src/utils/vectorize_utils.h"
#include "src/weights/base_weights.h"
#include "src/weights/llama/norm_weights.h"

// residual, decoder_out: [num_tokens, hidden].  In place on both:
// residual <- decoder_out + residual;  decoder_out <- RMSNorm(that (+ norm.bias)) * scale.
// residual->data == nullptr skips the add; norm.bias == nullptr skips the bias.
template <typename T>
void launchFusedAddBiasResidualRMSNorm(TensorWrapper<T>* residual, TensorWrapper<T>* decoder_out,
                                       BaseWeight<T>& norm, T* scale, float eps) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(decoder_out->shape.size() == 2, "decoder_out must be [num_tokens, hidden_units]");
    const int64_t num_tokens = decoder_out->shape[0];
    const int64_t hidden = decoder_out->shape[1];
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_add_residual_rmsnorm_f16(decoder_out->data, residual ? residual->data : nullptr, norm.bias,
                                             scale, eps, num_tokens, hidden, ispore_get_stream());
    else
        rc = ispore_add_residual_rmsnorm_f32((float*)decoder_out->data,
                                             (float*)(residual ? residual->data : nullptr),
                                             (const float*)norm.bias, (const float*)scale, eps, num_tokens,
                                             hidden, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchFusedAddBiasResidualRMSNorm");
}

// decoder_out [num_tokens, hidden] is normalised in place; when
// decoder_residual->data != nullptr it first receives the un-normed input.
template <typename T>
void launchRMSNorm(TensorWrapper<T>* decoder_out, TensorWrapper<T>* decoder_residual,
                   LayerNormWeight<T>& attn_norm_weight, float eps) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(decoder_out->shape.size() == 2, "decoder_out must be [num_tokens, hidden_units]");
    const int64_t num_tokens = decoder_out->shape[0];
    const int64_t hidden = decoder_out->shape[1];
    T* copy = decoder_residual ? decoder_residual->data : nullptr;
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_rmsnorm_f16(decoder_out->data, copy, attn_norm_weight.gamma, eps, num_tokens, hidden,
                                ispore_get_stream());
    else
        rc = ispore_rmsnorm_f32((float*)decoder_out->data, (float*)copy, (const float*)attn_norm_weight.gamma,
                                eps, num_tokens, hidden, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchRMSNorm");
}
