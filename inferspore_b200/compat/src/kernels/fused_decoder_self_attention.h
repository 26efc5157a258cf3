// Drop-in for the reference's src/kernels/fused_decoder_self_attention.h: same launcher name and
// arguments (:10-18), forwarding to the C ABI of libispore_kernels.
//
// Scratch.  The reference launcher takes no scratch argument; the kernel here can use one to split
// long sequences at small batch over several CTAs (without it: one CTA per sequence and head
// group — still correct, slower below ~64 sequences).  By default this header allocates NOTHING:
// the host hands a device buffer over once per thread and device,
//     ispore_compat::set_mha_workspace(ptr, bytes);   // with that device current
// sized with ispore_decoder_masked_mha_workspace_bytes() for its largest batch and step, and keeps
// ownership of it.  A host that prefers the header to manage the buffer builds with
// -DISPORE_MHA_ALLOC_WORKSPACE: then one buffer per (thread, device) is allocated on first use,
// grown when a call needs more (cudaFree + cudaMalloc: both synchronise the device, so size the
// first call generously) and freed when the thread exits.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "src/kernels/ispore_launch.h"
#include "src/models/llama/llama_params.h"
#include "src/utils/tensor.h"
#include "src/utils/vectorize_utils.h"
#include "src/weights/base_weights.h"

namespace ispore_compat {

constexpr int kMhaMaxDevices = 64;

// One slot per device for the calling thread: a buffer belongs to the device it was allocated
// on and is never offered to a kernel running on another one.
struct MhaWorkspaceSlots {
    void* buf[kMhaMaxDevices] = {};
    int64_t cap[kMhaMaxDevices] = {};
    bool owned[kMhaMaxDevices] = {};
    ~MhaWorkspaceSlots() {
        for (int d = 0; d < kMhaMaxDevices; ++d) {
            if (!owned[d] || buf[d] == nullptr) continue;
            int prev = 0;
            if (cudaGetDevice(&prev) != cudaSuccess) break;  // the runtime is already shutting down
            if (cudaSetDevice(d) == cudaSuccess) cudaFree(buf[d]);
            cudaSetDevice(prev);
            cudaGetLastError();
        }
    }
};
inline MhaWorkspaceSlots& mha_slots() {
    thread_local MhaWorkspaceSlots slots;
    return slots;
}
inline int mha_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMhaMaxDevices) return -1;
    return dev;
}

// Hands the calling thread's decode-attention scratch for the CURRENT device to the launcher
// (ptr == nullptr or bytes == 0 withdraws it).  The buffer stays the caller's.
inline void set_mha_workspace(void* ptr, int64_t bytes) {
    const int dev = mha_current_device();
    if (dev < 0) return;
    MhaWorkspaceSlots& s = mha_slots();
    if (s.owned[dev] && s.buf[dev] != nullptr) cudaFree(s.buf[dev]);
    s.buf[dev] = bytes > 0 ? ptr : nullptr;
    s.cap[dev] = ptr != nullptr && bytes > 0 ? bytes : 0;
    s.owned[dev] = false;
}

// The scratch the next call on the current device may use for `bytes`; nullptr = run unsplit.
inline void* mha_workspace(int64_t bytes) {
    const int dev = mha_current_device();
    if (dev < 0) return nullptr;
    MhaWorkspaceSlots& s = mha_slots();
    if (bytes <= s.cap[dev]) return s.buf[dev];
#ifdef ISPORE_MHA_ALLOC_WORKSPACE
    if (s.buf[dev] == nullptr || s.owned[dev]) {  // a buffer the caller handed over is never replaced
        if (s.buf[dev] != nullptr) cudaFree(s.buf[dev]);
        s.buf[dev] = nullptr;
        s.cap[dev] = 0;
        s.owned[dev] = true;
        if (cudaMalloc(&s.buf[dev], static_cast<size_t>(bytes)) != cudaSuccess) {
            cudaGetLastError();
            s.buf[dev] = nullptr;
            return nullptr;
        }
        s.cap[dev] = bytes;
        return s.buf[dev];
    }
#endif
    return nullptr;  // too small for a split plan of this size: the launcher runs unsplit
}
}  // namespace ispore_compat

template <typename T>
void launchDecoderMaskedMHA(TensorWrapper<T>* qkv_buf, BaseWeight<T>& qkv, TensorWrapper<int>* layer_id,
                            TensorWrapper<T>* k_cache, TensorWrapper<T>* v_cache, TensorWrapper<bool>* finished,
                            TensorWrapper<int>* step, TensorWrapper<T>* mha_output,
                            LLaMAAttentionStaticParams& static_params) {
    (void)finished;  // unused by the reference kernel as well
    ispore_compat::require_float_or_half<T>();
    LLM_CHECK_WITH_INFO(qkv_buf->shape.size() == 3, "qkv_buf must be [batch, qkv_head_num, head_size]");
    LLM_CHECK_WITH_INFO(k_cache->shape.size() == 5, "k_cache must be [layers, batch, kv_heads, max_seq_len, head_size]");
    const int64_t batch_size = qkv_buf->shape[0];
    const int64_t qkv_head_num = qkv_buf->shape[1];
    const int64_t head_size = qkv_buf->shape[2];
    const int64_t kv_head_num = k_cache->shape[2];
    const int64_t max_seq_len = k_cache->shape[3];
    const int64_t head_num = qkv_head_num - 2 * kv_head_num;
    const int64_t cur_step = step->getVal();
    const int64_t layer = layer_id->getVal();
    // The reference's own test declares the cache with a leading extent of 0 (its layer id);
    // only a positive extent is checked against the layer.
    const int64_t num_layers = k_cache->shape[0] > 0 ? k_cache->shape[0] : 0;
    const int64_t ws_bytes =
        ispore_decoder_masked_mha_workspace_bytes(batch_size, head_num, kv_head_num, head_size, cur_step);
    void* ws = ws_bytes > 0 ? ispore_compat::mha_workspace(ws_bytes) : nullptr;
    int rc;
    if (ispore_compat::is_half<T>::value)
        rc = ispore_decoder_masked_mha_f16(mha_output->data, qkv_buf->data, qkv.bias, k_cache->data, v_cache->data,
                                           layer, num_layers, batch_size, head_num, kv_head_num, max_seq_len,
                                           head_size, cur_step, static_params.rotary_embedding_dim,
                                           static_params.rotary_embedding_base, static_cast<float>(cur_step), ws,
                                           ws ? ws_bytes : 0, ispore_get_stream());
    else
        rc = ispore_decoder_masked_mha_f32((float*)mha_output->data, (const float*)qkv_buf->data,
                                           (const float*)qkv.bias, (float*)k_cache->data, (float*)v_cache->data,
                                           layer, num_layers, batch_size, head_num, kv_head_num, max_seq_len,
                                           head_size, cur_step, static_params.rotary_embedding_dim,
                                           static_params.rotary_embedding_base, static_cast<float>(cur_step), ws,
                                           ws ? ws_bytes : 0, ispore_get_stream());
    ispore_compat::throw_on_error(rc, "launchDecoderMaskedMHA");
}
