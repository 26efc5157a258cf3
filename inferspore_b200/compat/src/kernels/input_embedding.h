// launchInputEmbedding — same name and argument list as the reference
// (src/kernels/input_embedding.h:6-9); runs the sm_100a gather through
// ispore_input_embedding_{f32,f16}.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/utils/tensor.h"
#include "src/weights/llama/embedding_weights.h"

// input_ids [num_tokens] (int), output [num_tokens, hidden], embed_table [vocab, hidden].
// When embed_table->shape is filled in ({vocab, hidden}) ids are range-checked on
// the device; the reference's tests leave it empty, which means "trust the ids".
template <typename T>
void launchInputEmbedding(TensorWrapper<int>* input_ids, TensorWrapper<T>* output,
                          EmbeddingWeight<T>* embed_table) {
    ispore_compat::require_float_or_half<T>();
    const int64_t num_tokens = output->shape[0];
    const int64_t hidden = output->shape[1];
    LLM_CHECK_WITH_INFO(num_tokens == input_ids->shape[0],
                        "input ids 1st shape should equal to 1st shape of output");
    int64_t vocab = 0;
    if (embed_table->shape.size() == 2) {
        LLM_CHECK_WITH_INFO(embed_table->shape[1] == hidden, "embedding table width must equal output width");
        vocab = embed_table->shape[0];
    }
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_input_embedding_f16(input_ids->data, output->data, embed_table->data, num_tokens, hidden,
                                        vocab, ispore_get_stream());
    else
        rc = ispore_input_embedding_f32(input_ids->data, (float*)output->data, (const float*)embed_table->data,
                                        num_tokens, hidden, vocab, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchInputEmbedding");
}
