// TEST INFRASTRUCTURE.  Compiles, from where they lie, the reference's decode attention kernel
// (src/kernels/fused_decoder_self_attention.cu) and its unit test
// (tests/unittests/test_fused_decoder_attention.cu, main() renamed), and exports the test's CPU
// function CPUMaskedAttn (:12-143) and the GPU launcher launchDecoderMaskedMHA (.cu:381-441).
// The kernel file uses assert and CHECK_CUDA_ERROR without defining them (.cu:412-424, :440);
// this translation unit supplies both before including it.
//
// The GPU wrappers refuse what the reference kernel is not safe or not meaningful for:
//  * batch must be 1 (the kernel strides qkv_buf by heads*d per sequence, .cu:132,:141);
//  * head_size/vec threads per block must be a whole number of warps (its block reductions
//    shuffle with a full mask, .cu:9-30) and step must not exceed that thread count (its softmax
//    normalises only logits[tid], .cu:224-236);
//  * step <= max_seq_len, and every offset must fit its 32-bit arithmetic.
#include <cassert>
#include <cstdio>
#include <stdexcept>
#define CHECK_CUDA_ERROR(call)                                                        \
    do {                                                                              \
        cudaError_t err__ = (call);                                                   \
        if (err__ != cudaSuccess) throw std::runtime_error(cudaGetErrorString(err__)); \
    } while (0)
#include "src/kernels/fused_decoder_self_attention.cu"
#define main ref_test_fused_decoder_attention_main
#include "tests/unittests/test_fused_decoder_attention.cu"
#undef main

template <typename T>
static int run_mha(T* d_qkv, T* d_bias, int layer, T* d_k_cache, T* d_v_cache, T* d_out, int num_layers, int batch,
                   int heads, int kv_heads, int max_seq_len, int head_size, int step, int rot_dim, float base,
                   DataType dt) {
    const int threads = head_size / Vec<T>::size;
    if (batch != 1 || head_size % Vec<T>::size != 0 || threads % 32 != 0 || threads > 1024) return -1;
    if (step < 1 || step > threads || step > max_seq_len || kv_heads <= 0 || heads % kv_heads != 0) return -1;
    if (1ll * num_layers * batch * kv_heads * max_seq_len * head_size >= (1ll << 31) || layer >= num_layers) return -1;
    TensorWrapper<T> qkv(GPU, dt, {batch, heads + 2 * kv_heads, head_size}, d_qkv);
    TensorWrapper<T> kc(GPU, dt, {num_layers, batch, kv_heads, max_seq_len, head_size}, d_k_cache);
    TensorWrapper<T> vc(GPU, dt, {num_layers, batch, kv_heads, max_seq_len, head_size}, d_v_cache);
    TensorWrapper<T> out(GPU, dt, {batch, heads, head_size}, d_out);
    TensorWrapper<int> lid(CPU, INT32, {1}, &layer), st(CPU, INT32, {1}, &step);
    TensorWrapper<bool> fin(GPU, BOOL, {batch}, nullptr);
    BaseWeight<T> w;
    w.bias = d_bias;
    LLaMAAttentionStaticParams params;
    params.rotary_embedding_dim = rot_dim;
    params.rotary_embedding_base = base;
    params.max_position_embeddings = 4096;
    params.use_dynamic_ntk = false;
    launchDecoderMaskedMHA(&qkv, w, &lid, &kc, &vc, &fin, &st, &out, params);
    return 0;
}

extern "C" {
// q [bs, heads, d], k and v [bs, kv_heads, d], caches [bs, kv_heads, step, d] (the cache length IS
// step in the CPU function, :55-57); caches are updated in place at step-1; output fp32.
__attribute__((visibility("default"))) void ref_cpu_masked_attn_f32(float* q, float* k, float* v, float* k_cache,
                                                                   float* v_cache, float* out, int batch, int heads,
                                                                   int kv_heads, int head_size, int step) {
    CPUMaskedAttn<float>(q, k, v, k_cache, v_cache, out, batch, heads, kv_heads, head_size, step, 0, 10000.0f);
}
__attribute__((visibility("default"))) int ref_gpu_masked_mha_f32(float* d_qkv, float* d_bias, int layer,
                                                                 float* d_k_cache, float* d_v_cache, float* d_out,
                                                                 int num_layers, int batch, int heads, int kv_heads,
                                                                 int max_seq_len, int head_size, int step, int rot_dim,
                                                                 float base) {
    return run_mha<float>(d_qkv, d_bias, layer, d_k_cache, d_v_cache, d_out, num_layers, batch, heads, kv_heads,
                          max_seq_len, head_size, step, rot_dim, base, FP32);
}
__attribute__((visibility("default"))) int ref_gpu_masked_mha_f16(void* d_qkv, void* d_bias, int layer, void* d_k_cache,
                                                                 void* d_v_cache, void* d_out, int num_layers,
                                                                 int batch, int heads, int kv_heads, int max_seq_len,
                                                                 int head_size, int step, int rot_dim, float base) {
    return run_mha<half>(static_cast<half*>(d_qkv), static_cast<half*>(d_bias), layer, static_cast<half*>(d_k_cache),
                         static_cast<half*>(d_v_cache), static_cast<half*>(d_out), num_layers, batch, heads, kv_heads,
                         max_seq_len, head_size, step, rot_dim, base, FP16);
}
}
