// KV-cache concat for sm_100a.
//
// Semantics: src/kernels/concat_past_kv.cu:8-73 of the reference —
// cache[layer, b, h, history[b] + t, :] = src[b, h, t, :] for t < cur_len[b].
// For a fixed (b, h) both sides are one contiguous span of cur_len[b]*head_size
// elements, so the op is a batch of contiguous copies.  K and V go out in one
// launch (blockIdx.z selects the tensor); every thread moves UNROLL 128-bit
// vectors with all loads issued before the first store.  All offsets are
// 64-bit: one layer of the cache reaches 2^30 elements at batch 64 / 32 heads /
// 4096 positions / head size 128.
#include "common.cuh"

namespace ispore {
namespace {

template <int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
concat_kv_vec_kernel(uint4* __restrict__ k_dst, uint4* __restrict__ v_dst,
                     const uint4* __restrict__ k_src, const uint4* __restrict__ v_src,
                     const int32_t* __restrict__ cur_query_length,
                     const int32_t* __restrict__ history_length, int64_t layer_offset_vecs,
                     int kv_head_num, int max_q_len, int64_t max_seq_len, int head_vecs,
                     unsigned* __restrict__ status) {
    const int bh = blockIdx.y;  // b * kv_head_num + h
    const int b = bh / kv_head_num;
    const bool is_v = blockIdx.z != 0;
    const uint4* src = (is_v ? v_src : k_src) + static_cast<int64_t>(bh) * max_q_len * head_vecs;
    uint4* dst = (is_v ? v_dst : k_dst) + layer_offset_vecs +
                 static_cast<int64_t>(bh) * max_seq_len * head_vecs;

    int cur = __ldg(cur_query_length + b);
    const int64_t hist = __ldg(history_length + b);
    if (cur > max_q_len) cur = max_q_len;
    if (hist < 0 || hist + cur > max_seq_len) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, ISPORE_DEV_KV_OVERRUN);
        const int64_t room = hist < 0 ? 0 : max_seq_len - hist;
        cur = room < 0 ? 0 : static_cast<int>(room < cur ? room : cur);
    }
    const int64_t span = static_cast<int64_t>(cur) * head_vecs;  // contiguous vectors to move
    dst += hist * head_vecs;

    const int64_t tile = static_cast<int64_t>(THREADS) * UNROLL;
    for (int64_t base = blockIdx.x * tile; base < span; base += gridDim.x * tile) {
        uint4 buf[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const int64_t i = base + k * THREADS + threadIdx.x;
            if (i < span) buf[k] = ld_stream(src + i);
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const int64_t i = base + k * THREADS + threadIdx.x;
            if (i < span) st_stream(dst + i, buf[k]);
        }
    }
}

template <typename T>
__global__ void concat_kv_scalar_kernel(T* __restrict__ k_dst, T* __restrict__ v_dst,
                                        const T* __restrict__ k_src, const T* __restrict__ v_src,
                                        const int32_t* __restrict__ cur_query_length,
                                        const int32_t* __restrict__ history_length,
                                        int64_t layer_offset, int kv_head_num, int max_q_len,
                                        int64_t max_seq_len, int head_size,
                                        unsigned* __restrict__ status) {
    const int bh = blockIdx.y;
    const int b = bh / kv_head_num;
    const bool is_v = blockIdx.z != 0;
    const T* src = (is_v ? v_src : k_src) + static_cast<int64_t>(bh) * max_q_len * head_size;
    T* dst = (is_v ? v_dst : k_dst) + layer_offset + static_cast<int64_t>(bh) * max_seq_len * head_size;
    int cur = cur_query_length[b];
    const int64_t hist = history_length[b];
    if (cur > max_q_len) cur = max_q_len;
    if (hist < 0 || hist + cur > max_seq_len) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, ISPORE_DEV_KV_OVERRUN);
        const int64_t room = hist < 0 ? 0 : max_seq_len - hist;
        cur = room < 0 ? 0 : static_cast<int>(room < cur ? room : cur);
    }
    const int64_t span = static_cast<int64_t>(cur) * head_size;
    dst += hist * head_size;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < span;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[i] = src[i];
}

template <typename T>
int concat_dispatch(T* k_dst, T* v_dst, const T* k_src, const T* v_src, const int32_t* cur_len,
                    const int32_t* hist_len, int64_t layer, int64_t num_layers, int64_t batch,
                    int64_t kv_heads, int64_t max_q_len, int64_t max_seq_len, int64_t head_size,
                    cudaStream_t st) {
    if (batch < 0 || kv_heads <= 0 || max_q_len < 0 || max_seq_len <= 0 || head_size <= 0 ||
        layer < 0 || (num_layers > 0 && layer >= num_layers) || max_q_len > INT32_MAX)
        return fail(ISPORE_ESHAPE,
                    "concat_kv: bad shape layer=%lld/%lld bs=%lld heads=%lld q=%lld seq=%lld d=%lld",
                    (long long)layer, (long long)num_layers, (long long)batch, (long long)kv_heads,
                    (long long)max_q_len, (long long)max_seq_len, (long long)head_size);
    if (batch * kv_heads > 65535)
        return fail(ISPORE_ELIMIT, "concat_kv: batch*kv_heads %lld > 65535", (long long)(batch * kv_heads));
    if (batch == 0 || max_q_len == 0) return ISPORE_OK;
    if (!k_dst || !v_dst || !k_src || !v_src || !cur_len || !hist_len)
        return fail(ISPORE_ENULL, "concat_kv: NULL buffer");
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "concat_kv: no device status word");

    const int64_t layer_offset = layer * batch * kv_heads * max_seq_len * head_size;  // elements
    constexpr int E = VecTraits<T>::kElems;
    constexpr int THREADS = 128, UNROLL = 4;
    const bool vec_ok = head_size % E == 0 && aligned16(k_dst) && aligned16(v_dst) &&
                        aligned16(k_src) && aligned16(v_src);
    if (vec_ok) {
        const int64_t span_max = max_q_len * (head_size / E);
        int64_t gx = ceil_div(span_max, THREADS * UNROLL);
        if (gx > 64) gx = 64;
        dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(batch * kv_heads), 2);
        concat_kv_vec_kernel<THREADS, UNROLL><<<grid, THREADS, 0, st>>>(
            reinterpret_cast<uint4*>(k_dst), reinterpret_cast<uint4*>(v_dst),
            reinterpret_cast<const uint4*>(k_src), reinterpret_cast<const uint4*>(v_src), cur_len,
            hist_len, layer_offset / E, (int)kv_heads, (int)max_q_len, max_seq_len,
            (int)(head_size / E), status);
        return check_launch("concat_kv_vec_kernel");
    }
    int64_t gx = ceil_div(max_q_len * head_size, 256);
    if (gx > 64) gx = 64;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(batch * kv_heads), 2);
    concat_kv_scalar_kernel<T><<<grid, 256, 0, st>>>(k_dst, v_dst, k_src, v_src, cur_len, hist_len,
                                                     layer_offset, (int)kv_heads, (int)max_q_len,
                                                     max_seq_len, (int)head_size, status);
    return check_launch("concat_kv_scalar_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {
int ispore_concat_kv_f32(float* k_dst, float* v_dst, const float* k_src, const float* v_src,
                         const int32_t* cur_query_length, const int32_t* history_length,
                         int64_t layer, int64_t num_layers, int64_t batch_size, int64_t kv_head_num,
                         int64_t max_q_len, int64_t max_seq_len, int64_t head_size,
                         ispore_stream_t stream) {
    return ispore::concat_dispatch<float>(k_dst, v_dst, k_src, v_src, cur_query_length, history_length,
                                          layer, num_layers, batch_size, kv_head_num, max_q_len,
                                          max_seq_len, head_size, static_cast<cudaStream_t>(stream));
}
int ispore_concat_kv_f16(void* k_dst, void* v_dst, const void* k_src, const void* v_src,
                         const int32_t* cur_query_length, const int32_t* history_length,
                         int64_t layer, int64_t num_layers, int64_t batch_size, int64_t kv_head_num,
                         int64_t max_q_len, int64_t max_seq_len, int64_t head_size,
                         ispore_stream_t stream) {
    return ispore::concat_dispatch<__half>(
        static_cast<__half*>(k_dst), static_cast<__half*>(v_dst), static_cast<const __half*>(k_src),
        static_cast<const __half*>(v_src), cur_query_length, history_length, layer, num_layers,
        batch_size, kv_head_num, max_q_len, max_seq_len, head_size,
        static_cast<cudaStream_t>(stream));
}
}
