// TEST INFRASTRUCTURE.  Compiles the reference's unit test tests/unittests/test_casual_mask.cu
// from where it lies (its main() renamed) and exports its CPU function CPUbuildCasualMask
// (test_casual_mask.cu:12-32) together with the reference's GPU launchers for the causal mask
// (src/kernels/build_casual_mask.cu:23-33), the padding offsets (src/kernels/cal_paddingoffset.cu:31-45)
// and repeat-KV (src/kernels/repeat_kv.cu:52-101).  The wrappers refuse shapes the reference kernels
// are not safe for:
//  * padding offsets: every length must lie in [0, max_q_len] (the kernel writes sum(len) entries
//    into a [batch, max_q_len] buffer, .cu:18-24); the wrapper is given the lengths on the host too.
//  * repeat-KV: context lengths must not exceed max_k_len <= max_seq_len (the guard at .cu:30 only
//    compares with the context length), and every offset must fit 32-bit arithmetic (.cu:34-45, :71).
#define main ref_test_casual_mask_main
#include "tests/unittests/test_casual_mask.cu"
#undef main
#include "src/kernels/cal_paddingoffset.h"
#include "src/kernels/repeat_kv.h"

template <typename T>
static int repeat_kv(T* d_k_src, T* d_v_src, int* d_ctx_len, const int* h_ctx_len, int layer, T* d_k_dst, T* d_v_dst,
                     int num_layers, int batch, int kv_heads, int heads, int max_seq_len, int max_k_len,
                     int head_size, DataType dt) {
    if (max_k_len > max_seq_len || kv_heads <= 0 || heads % kv_heads != 0) return -1;
    if (1ll * num_layers * batch * kv_heads * max_seq_len * head_size >= (1ll << 31)) return -1;
    if (1ll * batch * heads * max_k_len * head_size >= (1ll << 31) || batch > 65535 || heads > 65535) return -1;
    for (int b = 0; b < batch; ++b)
        if (h_ctx_len[b] < 0 || h_ctx_len[b] > max_k_len) return -1;
    TensorWrapper<T> ks(GPU, dt, {num_layers, batch, kv_heads, max_seq_len, head_size}, d_k_src);
    TensorWrapper<T> vs(GPU, dt, {num_layers, batch, kv_heads, max_seq_len, head_size}, d_v_src);
    TensorWrapper<int> ctx(GPU, INT32, {batch}, d_ctx_len), lid(CPU, INT32, {1}, &layer);
    TensorWrapper<T> kd(GPU, dt, {batch, heads, max_k_len, head_size}, d_k_dst);
    TensorWrapper<T> vd(GPU, dt, {batch, heads, max_k_len, head_size}, d_v_dst);
    launchRepeatKVCache(&ks, &vs, &ctx, &lid, &kd, &vd);
    return 0;
}
extern "C" {
__attribute__((visibility("default"))) void ref_cpu_causal_mask_f32(float* mask, const int* q_lens, const int* k_lens,
                                                                   int max_q_len, int max_k_len, int batch) {
    CPUbuildCasualMask(mask, q_lens, k_lens, max_q_len, max_k_len, batch);
}
__attribute__((visibility("default"))) int ref_gpu_causal_mask_f32(float* d_mask, int* d_q_lens, int* d_k_lens,
                                                                  int batch, int max_q_len, int max_k_len) {
    if (1ll * batch * max_q_len * max_k_len >= (1ll << 31)) return -1;
    TensorWrapper<float> mask(GPU, FP32, {batch, max_q_len, max_k_len}, d_mask);
    TensorWrapper<int> ql(GPU, INT32, {batch}, d_q_lens), kl(GPU, INT32, {batch}, d_k_lens);
    launchBuildCausalMasks(&mask, &ql, &kl);
    return 0;
}
__attribute__((visibility("default"))) int ref_gpu_causal_mask_f16(void* d_mask, int* d_q_lens, int* d_k_lens,
                                                                  int batch, int max_q_len, int max_k_len) {
    if (1ll * batch * max_q_len * max_k_len >= (1ll << 31)) return -1;
    TensorWrapper<half> mask(GPU, FP16, {batch, max_q_len, max_k_len}, static_cast<half*>(d_mask));
    TensorWrapper<int> ql(GPU, INT32, {batch}, d_q_lens), kl(GPU, INT32, {batch}, d_k_lens);
    launchBuildCausalMasks(&mask, &ql, &kl);
    return 0;
}
__attribute__((visibility("default"))) int ref_gpu_cal_padding_offset(int* d_padding_offset, int* d_cum_seqlens,
                                                                     int* d_input_lengths,
                                                                     const int* h_input_lengths, int batch,
                                                                     int max_q_len) {
    for (int b = 0; b < batch; ++b)
        if (h_input_lengths[b] < 0 || h_input_lengths[b] > max_q_len) return -1;
    TensorWrapper<int> po(GPU, INT32, {batch, max_q_len}, d_padding_offset);
    TensorWrapper<int> cum(GPU, INT32, {batch + 1}, d_cum_seqlens), il(GPU, INT32, {batch}, d_input_lengths);
    launchCalPaddingoffset(&po, &cum, &il);
    return 0;
}

__attribute__((visibility("default"))) int ref_gpu_repeat_kv_f32(float* d_k_src, float* d_v_src, int* d_ctx_len,
                                                                const int* h_ctx_len, int layer, float* d_k_dst,
                                                                float* d_v_dst, int num_layers, int batch,
                                                                int kv_heads, int heads, int max_seq_len,
                                                                int max_k_len, int head_size) {
    return repeat_kv<float>(d_k_src, d_v_src, d_ctx_len, h_ctx_len, layer, d_k_dst, d_v_dst, num_layers, batch,
                            kv_heads, heads, max_seq_len, max_k_len, head_size, FP32);
}
__attribute__((visibility("default"))) int ref_gpu_repeat_kv_f16(void* d_k_src, void* d_v_src, int* d_ctx_len,
                                                                const int* h_ctx_len, int layer, void* d_k_dst,
                                                                void* d_v_dst, int num_layers, int batch,
                                                                int kv_heads, int heads, int max_seq_len,
                                                                int max_k_len, int head_size) {
    return repeat_kv<half>(static_cast<half*>(d_k_src), static_cast<half*>(d_v_src), d_ctx_len, h_ctx_len, layer,
                           static_cast<half*>(d_k_dst), static_cast<half*>(d_v_dst), num_layers, batch, kv_heads,
                           heads, max_seq_len, max_k_len, head_size, FP16);
}
}
