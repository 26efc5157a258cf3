// KV-cache concat for sm_100a.
//
// Semantics: src/kernels/concat_past_kv.cu:8-73 of the reference —
// cache[layer, b, h, history[b] + t, :] = src[b, h, t, :] for t < cur_len[b].
// For a fixed (b, h) both sides are one contiguous span of cur_len[b]*head_size
// elements, so the op is a batch of contiguous copies.  K and V go out in one
// launch.  Default path: TMA bulk copies (global -> shared -> global) of up to
// 8 KB pieces, one lane per piece, nothing in registers; at decode shape
// (one 256-byte row per (b, h)) that is 16 rows per one-warp CTA.  Fallback for
// rows that are not a multiple of 16 bytes or unaligned buffers: scalar copies.  All offsets are 64-bit: one layer of
// the cache reaches 2^30 elements at batch 64 / 32 heads / 4096 positions /
// head size 128.
#include "common.cuh"
#include "tma.cuh"

namespace ispore {
namespace {

// TMA variant: the spans are contiguous on both sides, so each piece of up to chunk_bytes is one
// bulk copy into shared memory and one bulk copy out, issued by the lane that owns the piece;
// no data passes through registers.  One-warp CTAs, ROWS pieces in flight per CTA.
template <int ROWS>
__global__ void __launch_bounds__(32)
concat_kv_tma_kernel(unsigned char* __restrict__ k_dst, unsigned char* __restrict__ v_dst,
                     const unsigned char* __restrict__ k_src, const unsigned char* __restrict__ v_src,
                     const int32_t* __restrict__ cur_query_length, const int32_t* __restrict__ history_length,
                     int64_t layer_offset_bytes, int kv_head_num, int batch_heads, int max_q_len,
                     int64_t max_seq_len, uint32_t row_bytes, uint32_t chunk_bytes, uint32_t chunks_per_span,
                     unsigned* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char slots[];  // [ROWS][chunk_bytes]
    __shared__ __align__(8) uint64_t full[ROWS];
    chain_begin();
    const int lane = threadIdx.x;
    if (lane < ROWS) tma::mbar_init(&full[lane], 1);
    tma::fence_mbar_init();
    __syncwarp();
    if (lane >= ROWS) return;

    const uint32_t pieces_per_tensor = static_cast<uint32_t>(batch_heads) * chunks_per_span;
    const uint32_t g = blockIdx.x * ROWS + lane;
    if (g >= 2u * pieces_per_tensor) return;
    const bool is_v = g >= pieces_per_tensor;
    const uint32_t r = is_v ? g - pieces_per_tensor : g;
    const uint32_t bh = r / chunks_per_span;
    const uint32_t piece = r - bh * chunks_per_span;
    const uint32_t b = bh / static_cast<uint32_t>(kv_head_num);

    int cur = __ldg(cur_query_length + b);
    const int64_t hist = __ldg(history_length + b);
    if (cur > max_q_len) cur = max_q_len;
    if (hist < 0 || hist + cur > max_seq_len) {
        if (piece == 0) atomicOr(status, ISPORE_DEV_KV_OVERRUN);
        const int64_t room = hist < 0 ? 0 : max_seq_len - hist;
        cur = room < 0 ? 0 : static_cast<int>(room < cur ? room : cur);
    }
    const int64_t span = static_cast<int64_t>(cur) * row_bytes;
    const int64_t off = static_cast<int64_t>(piece) * chunk_bytes;
    if (off >= span) return;
    const uint32_t bytes = static_cast<uint32_t>(span - off < chunk_bytes ? span - off : chunk_bytes);

    const unsigned char* src = (is_v ? v_src : k_src) + static_cast<int64_t>(bh) * max_q_len * row_bytes + off;
    unsigned char* dst = (is_v ? v_dst : k_dst) + layer_offset_bytes +
                         (static_cast<int64_t>(bh) * max_seq_len + hist) * row_bytes + off;
    unsigned char* slot = slots + static_cast<size_t>(lane) * chunk_bytes;
    tma::mbar_arrive_expect_tx(&full[lane], bytes);
    tma::load(slot, src, bytes, &full[lane]);
    if (!tma::mbar_wait(&full[lane], 0)) {
        atomicOr(status, ISPORE_DEV_TIMEOUT);
        tma::mbar_wait(&full[lane], 0);  // one more bounded wait for the copy in flight, then give up
        return;
    }
    tma::store(dst, slot, bytes);
    tma::commit_group();
    tma::wait_group_read<0>();
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
    if (batch * kv_heads > INT32_MAX)
        return fail(ISPORE_ELIMIT, "concat_kv: batch*kv_heads %lld too large", (long long)(batch * kv_heads));
    if (batch == 0 || max_q_len == 0) return ISPORE_OK;
    if (!k_dst || !v_dst || !k_src || !v_src || !cur_len || !hist_len)
        return fail(ISPORE_ENULL, "concat_kv: NULL buffer");
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "concat_kv: no device status word");

    const int64_t layer_offset = layer * batch * kv_heads * max_seq_len * head_size;  // elements
    constexpr int E = VecTraits<T>::kElems;
    const bool vec_ok = head_size % E == 0 && aligned16(k_dst) && aligned16(v_dst) &&
                        aligned16(k_src) && aligned16(v_src);
    const int64_t row_bytes = head_size * static_cast<int64_t>(sizeof(T));
    if (vec_ok) {  // head rows are whole 16-byte vectors and every base is 16-byte aligned
        // Pieces of at most 8 KB; 4 pieces (<= 32 KB of shared memory) per one-warp CTA, more when
        // the pieces are small (decode: one 256-byte row per (b, h)).
        const int64_t span_max = max_q_len * row_bytes;
        const uint32_t chunk = static_cast<uint32_t>(span_max < 8192 ? span_max : 8192);
        const int64_t cps = ceil_div(span_max, chunk);
        const int64_t pieces = 2 * batch * kv_heads * cps;
        if (pieces < (1ll << 31)) {
            auto kb = reinterpret_cast<unsigned char*>(k_dst);
            auto vb = reinterpret_cast<unsigned char*>(v_dst);
            auto ks = reinterpret_cast<const unsigned char*>(k_src);
            auto vs = reinterpret_cast<const unsigned char*>(v_src);
            const int64_t lo_bytes = layer_offset * static_cast<int64_t>(sizeof(T));
            if (chunk >= 2048) {
                launch_chained(concat_kv_tma_kernel<4>, static_cast<unsigned>(ceil_div(pieces, 4)), 32, 4 * chunk, st,
                    kb, vb, ks, vs, cur_len, hist_len, lo_bytes, (int)kv_heads, (int)(batch * kv_heads), (int)max_q_len,
                    max_seq_len, (uint32_t)row_bytes, chunk, (uint32_t)cps, status);
            } else {
                launch_chained(concat_kv_tma_kernel<16>, static_cast<unsigned>(ceil_div(pieces, 16)), 32, 16 * chunk, st,
                    kb, vb, ks, vs, cur_len, hist_len, lo_bytes, (int)kv_heads, (int)(batch * kv_heads), (int)max_q_len,
                    max_seq_len, (uint32_t)row_bytes, chunk, (uint32_t)cps, status);
            }
            return check_launch("concat_kv_tma_kernel");
        }
    }
    // The scalar kernel puts (b, h) on gridDim.y, which the hardware caps at 65535 (the TMA path's
    // grid is flat and has no such limit).
    if (batch * kv_heads > 65535)
        return fail(ISPORE_ELIMIT, "concat_kv: batch*kv_heads %lld > 65535 on the unaligned path",
                    (long long)(batch * kv_heads));
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
