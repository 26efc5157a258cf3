// TEST INFRASTRUCTURE.  Exports the reference's GPU launchers for KV concat
// (src/kernels/concat_past_kv.cu:75-113) and scale+mask+softmax
// (src/kernels/attn_softmax_kernel.cu:265-297); the reference has no CPU
// function for either (tests/unittests/test_concat_kv.cu:10-13,
// tests/unittests/test_mask_softmax.cu:10-14).  The wrappers refuse shapes the
// reference kernels are not safe for:
//  * concat: head_size must be a multiple of 32 (one thread per element), and
//    the layer offset must fit the reference's 32-bit arithmetic (.cu:91).
//  * softmax: k_len must be a multiple of 32*items so no thread takes the early
//    `return` in front of the block barriers (.cu:65-68, :153-156), and the
//    resulting block must stay under 1024 threads (host assert at .cu:218-220).
#include "src/kernels/attn_softmax_kernel.h"
#include "src/kernels/concat_past_kv.h"

extern "C" {
__attribute__((visibility("default"))) int ref_gpu_concat_kv_f32(float* d_k_src, float* d_v_src, int layer,
                                                                int* d_cur_len, int* d_hist_len, float* d_k_dst,
                                                                float* d_v_dst, int num_layers, int batch,
                                                                int kv_heads, int max_q_len, int max_seq_len,
                                                                int head_size) {
    const long long per_layer = 1ll * batch * kv_heads * max_seq_len * head_size;
    if (head_size % 32 != 0 || head_size > 1024 || per_layer * (layer + 1) >= (1ll << 31)) return -1;
    TensorWrapper<float> ks(GPU, FP32, {batch, kv_heads, max_q_len, head_size}, d_k_src);
    TensorWrapper<float> vs(GPU, FP32, {batch, kv_heads, max_q_len, head_size}, d_v_src);
    TensorWrapper<int> lid(CPU, INT32, {1}, &layer);
    TensorWrapper<int> cur(GPU, INT32, {batch}, d_cur_len), hist(GPU, INT32, {batch}, d_hist_len);
    TensorWrapper<float> kd(GPU, FP32, {num_layers, batch, kv_heads, max_seq_len, head_size}, d_k_dst);
    TensorWrapper<float> vd(GPU, FP32, {num_layers, batch, kv_heads, max_seq_len, head_size}, d_v_dst);
    launchConcatKVCache(&ks, &vs, &lid, &cur, &hist, &kd, &vd);
    return 0;
}
__attribute__((visibility("default"))) int ref_gpu_concat_kv_f16(void* d_k_src, void* d_v_src, int layer,
                                                                int* d_cur_len, int* d_hist_len, void* d_k_dst,
                                                                void* d_v_dst, int num_layers, int batch, int kv_heads,
                                                                int max_q_len, int max_seq_len, int head_size) {
    const long long per_layer = 1ll * batch * kv_heads * max_seq_len * head_size;
    if (head_size % 32 != 0 || head_size > 1024 || per_layer * (layer + 1) >= (1ll << 31)) return -1;
    TensorWrapper<half> ks(GPU, FP16, {batch, kv_heads, max_q_len, head_size}, static_cast<half*>(d_k_src));
    TensorWrapper<half> vs(GPU, FP16, {batch, kv_heads, max_q_len, head_size}, static_cast<half*>(d_v_src));
    TensorWrapper<int> lid(CPU, INT32, {1}, &layer);
    TensorWrapper<int> cur(GPU, INT32, {batch}, d_cur_len), hist(GPU, INT32, {batch}, d_hist_len);
    TensorWrapper<half> kd(GPU, FP16, {num_layers, batch, kv_heads, max_seq_len, head_size},
                           static_cast<half*>(d_k_dst));
    TensorWrapper<half> vd(GPU, FP16, {num_layers, batch, kv_heads, max_seq_len, head_size},
                           static_cast<half*>(d_v_dst));
    launchConcatKVCache(&ks, &vs, &lid, &cur, &hist, &kd, &vd);
    return 0;
}

static int softmax_shape_ok(int k_len, int vec) {
    // Mirrors the block-size arithmetic of LAUNCH_SOFTMAX (.cu:214-263).
    int block = (k_len + 31) / 32 * 32;
    int items = block > 2048 && block <= 4096 ? 4 : (block > 1024 ? 2 : 1);
    if (block > 4096) return 0;
    if (k_len % (32 * items * vec) != 0) return 0;
    block = block / (items * vec);
    return block < 1024 && block >= 32;
}
__attribute__((visibility("default"))) int ref_gpu_softmax_f32(float* d_qk, float* d_mask, float* d_score, int batch,
                                                              int heads, int q_len, int k_len, float scale) {
    if (!softmax_shape_ok(k_len, 1)) return -1;
    TensorWrapper<float> qk(GPU, FP32, {batch, heads, q_len, k_len}, d_qk), mask(GPU, FP32, {batch, q_len, k_len}, d_mask),
        score(GPU, FP32, {batch, heads, q_len, k_len}, d_score);
    launchScaleMaskAndSoftmax(&qk, &mask, &score, scale);
    return 0;
}
__attribute__((visibility("default"))) int ref_gpu_softmax_f16(void* d_qk, void* d_mask, void* d_score, int batch,
                                                              int heads, int q_len, int k_len, float scale) {
    if (!softmax_shape_ok(k_len, 2)) return -1;
    TensorWrapper<half> qk(GPU, FP16, {batch, heads, q_len, k_len}, static_cast<half*>(d_qk)),
        mask(GPU, FP16, {batch, q_len, k_len}, static_cast<half*>(d_mask)),
        score(GPU, FP16, {batch, heads, q_len, k_len}, static_cast<half*>(d_score));
    launchScaleMaskAndSoftmax(&qk, &mask, &score, scale);
    return 0;
}
}
