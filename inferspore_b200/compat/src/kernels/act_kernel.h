// launchAct — same name and argument list as the reference
// (src/kernels/act_kernel.h:8-9); runs the sm_100a SiLU(gate)*up kernel
// through ispore_silu_mul_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"
#include "src/utils/vectorize_utils.h"

// input [rows, 2, inter] (gate row, then up row) -> out [rows, inter].
template <typename T>
void launchAct(TensorWrapper<T>* input, TensorWrapper<T>* out) {
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK(input->shape.size() == 3);
    LLM_CHECK(input->shape[1] == 2);
    const int64_t rows = input->shape[0];
    const int64_t inter = input->shape[2];
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_silu_mul_f16(out->data, input->data, rows, inter, ispore_get_stream());
    else
        rc = ispore_silu_mul_f32((float*)out->data, (const float*)input->data, rows, inter, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchAct");
}
