// TEST INFRASTRUCTURE.  Compiles the reference's own unit test
// tests/unittests/test_bias_and_RoPE.cu from where it lies (its main() renamed)
// and exports its CPU function CPUfunc (:12-76) and the reference's fp32 GPU
// launcher (src/kernels/qkv_bias_and_RoPE.cu:286-330).  CPUfunc uses its own
// un-transposed [b, s, head, d] layout for q/k and reads QKV with q-only strides
// (:36-37, :56-59); callers must feed it inputs for which that is well defined.
// The fp16 launcher is not exported (empty kernel body, .cu:194-280).
#define main ref_test_bias_and_rope_main
#include "tests/unittests/test_bias_and_RoPE.cu"
#undef main

extern "C" {
__attribute__((visibility("default"))) void ref_cpu_qkv_rope_f32(float* q, float* k, float* v, float* QKV,
                                                                const float* bias, const int* padding_offset,
                                                                const int* history_length, const int* input_length,
                                                                int batch, int seq_len, int token_num, int head_num,
                                                                int kv_head_num, int head_size, int rot_dim,
                                                                float base) {
    CPUfunc(q, k, v, QKV, bias, padding_offset, history_length, input_length, batch, seq_len, token_num, head_num,
            kv_head_num, head_size, rot_dim, base);
}
// head_size must be a multiple of 32 (one thread per element, whole warps).
__attribute__((visibility("default"))) int ref_gpu_qkv_rope_f32(float* d_q, float* d_k, float* d_v, float* d_QKV,
                                                               float* d_bias, int* d_padding_offset,
                                                               int* d_history_length, int* d_input_length, int batch,
                                                               int seq_len, int token_num, int head_num,
                                                               int kv_head_num, int head_size, int rot_dim,
                                                               float base) {
    if (head_size % 32 != 0 || head_size > 1024 || head_size <= 0 || kv_head_num > head_num) return -1;
    TensorWrapper<float> q(GPU, FP32, {batch, head_num, seq_len, head_size}, d_q);
    TensorWrapper<float> k(GPU, FP32, {batch, kv_head_num, seq_len, head_size}, d_k);
    TensorWrapper<float> v(GPU, FP32, {batch, kv_head_num, seq_len, head_size}, d_v);
    TensorWrapper<float> qkv(GPU, FP32, {token_num, head_num + 2 * kv_head_num, head_size}, d_QKV);
    TensorWrapper<int> pad(GPU, INT32, {batch, seq_len}, d_padding_offset);
    TensorWrapper<int> hist(GPU, INT32, {batch}, d_history_length);
    TensorWrapper<int> inlen(GPU, INT32, {batch}, d_input_length);
    BaseWeight<float> w;
    w.bias = d_bias;
    LLaMAAttentionStaticParams params;
    params.rotary_embedding_dim = rot_dim;
    params.rotary_embedding_base = base;
    params.max_position_embeddings = 4096;
    params.use_dynamic_ntk = false;
    launchAddFusedQKVBiasTransposeAndRoPE(&q, &k, &v, &qkv, w, &pad, &hist, &inlen, params);
    return 0;
}
}
