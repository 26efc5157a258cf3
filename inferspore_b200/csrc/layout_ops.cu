// The small layout kernels either side of attention, for sm_100a:
//   causal/padding mask build     (reference: src/kernels/build_casual_mask.cu:5-42)
//   padding-offset scan            (reference: src/kernels/cal_paddingoffset.cu:18-45, a <<<1,1>>> loop)
//   transpose + remove padding     (reference: declared in src/kernels/fused_transpose_and_remv_pad.h:7-10,
//                                   never defined; semantics from tests/unittests/test_fused_trans_remv_pad.cu:3-4)
//   repeat-KV (GQA head broadcast) (reference: src/kernels/repeat_kv.cu:11-50)
// All four are index/copy work: bit-exact, 64-bit offsets, 128-bit vectors where the rows
// allow it and a scalar path otherwise.
#include <type_traits>

#include "common.cuh"

namespace ispore {
namespace {

// ---- causal mask -------------------------------------------------------------------------------
// mask[b, q, k] = q < qlen && k < klen && k <= q + (klen - qlen) && k >= klen - qlen
// (src/kernels/build_casual_mask.cu:36).  One thread per 128-bit vector (or element) of a row.
template <typename T, typename Index, bool VEC>
__global__ void __launch_bounds__(256)
build_causal_mask_kernel(T* __restrict__ mask, const int32_t* __restrict__ q_lens,
                         const int32_t* __restrict__ k_lens, Index units /* vectors or elements */,
                         uint32_t max_q_len, uint32_t units_per_row) {
    constexpr int E = VEC ? VecTraits<T>::kElems : 1;
    const Index stride = static_cast<Index>(gridDim.x) * blockDim.x;
    for (Index i = static_cast<Index>(blockIdx.x) * blockDim.x + threadIdx.x; i < units; i += stride) {
        const Index row = i / units_per_row;  // b * max_q + q
        const int k0 = static_cast<int>(i - row * units_per_row) * E;
        const uint32_t b = static_cast<uint32_t>(row / max_q_len);
        const int q = static_cast<int>(row - static_cast<Index>(b) * max_q_len);
        const int qlen = __ldg(q_lens + b), klen = __ldg(k_lens + b);
        // ones span k in [lo, hi]: lo = klen - qlen, hi = min(klen - 1, q + klen - qlen); none when q >= qlen
        const int lo = klen - qlen;
        const int hi = q < qlen ? min(klen - 1, q + lo) : -1;
        if (VEC) {
            Unpacked<T> v;
#pragma unroll
            for (int e = 0; e < E; ++e) v.v[e] = (k0 + e >= lo && k0 + e <= hi) ? 1.0f : 0.0f;
            st_stream(reinterpret_cast<uint4*>(mask) + i, pack(v));
        } else {
            mask[i] = from_float<T>((k0 >= lo && k0 <= hi) ? 1.0f : 0.0f);
        }
    }
}

// The same for rows of whole 128-bit vectors, a warp per row and kMaskRowsPerWarp rows per warp: the
// row's span of ones is worked out once per row (one division per row instead of two per vector),
// a vector wholly inside or outside it is a constant, and only the two vectors at the span's ends
// are built element by element.  (Measured on [128, 512, 512] fp16, 67 MB, replayed from a graph:
// 11.9 us against 19.1 us for the kernel above, which stays for rows that are not whole vectors.)
constexpr int kMaskWarps = 8;
constexpr int kMaskRowsPerWarp = 4;

template <typename T>
__global__ void __launch_bounds__(kMaskWarps * 32)
build_causal_mask_rows_kernel(T* __restrict__ mask, const int32_t* __restrict__ q_lens,
                              const int32_t* __restrict__ k_lens, int64_t rows, uint32_t max_q_len, int vecs_per_row) {
    constexpr int E = VecTraits<T>::kElems;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    Unpacked<T> ones, zeros;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        ones.v[e] = 1.0f;
        zeros.v[e] = 0.0f;
    }
    const uint4 one_v = pack(ones), zero_v = pack(zeros);
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * kMaskWarps + warp) * kMaskRowsPerWarp;
#pragma unroll 1
    for (int r = 0; r < kMaskRowsPerWarp; ++r) {
        const int64_t row = first + r;  // b * max_q + q
        if (row >= rows) break;
        const int64_t b = row / max_q_len;
        const int q = static_cast<int>(row - b * max_q_len);
        const int qlen = __ldg(q_lens + b), klen = __ldg(k_lens + b);
        // ones span k in [lo, hi]: lo = klen - qlen, hi = min(klen - 1, q + klen - qlen); none when q >= qlen
        const int lo = klen - qlen;
        const int hi = q < qlen ? min(klen - 1, q + lo) : -1;
        uint4* out = reinterpret_cast<uint4*>(mask) + row * vecs_per_row;
        for (int v = lane; v < vecs_per_row; v += 32) {
            const int k0 = v * E, k1 = k0 + (E - 1);
            uint4 val = (k0 >= lo && k1 <= hi) ? one_v : zero_v;
            if (!(k0 >= lo && k1 <= hi) && !(k0 > hi || k1 < lo)) {  // an end of the span falls inside this vector
                Unpacked<T> x;
#pragma unroll
                for (int e = 0; e < E; ++e) x.v[e] = (k0 + e >= lo && k0 + e <= hi) ? 1.0f : 0.0f;
                val = pack(x);
            }
            st_stream(out + v, val);
        }
    }
}

// ---- padding offsets ----------------------------------------------------------------------------
// cum_seqlens[b] = sum of lengths before b (cum_seqlens[batch] = total);
// padding_offset[cum_seqlens[b] + i] = b*max_q_len - cum_seqlens[b] for i < len[b]
// (src/kernels/cal_paddingoffset.cu:25-45).  CTA (x, y) owns sequences x*256 .. x*256+255: it sums
// the lengths in front of its chunk (no CTA waits for another), scans its own 256 lengths, and
// its warps fill the tokens, sequence by sequence; the y CTAs of a chunk split every sequence's
// tokens between them.
constexpr int kSeqPerCta = 256;

__device__ __forceinline__ int clamp_len(int len, int max_q_len) { return len < 0 ? 0 : (len > max_q_len ? max_q_len : len); }

__global__ void __launch_bounds__(kSeqPerCta)
padding_offset_kernel(int32_t* __restrict__ padding_offset, int32_t* __restrict__ cum_seqlens,
                      const int32_t* __restrict__ input_lengths, int batch, int max_q_len) {
    constexpr int kWarps = kSeqPerCta / 32;
    __shared__ int warp_tot[2][kWarps];
    __shared__ int seq_start[kSeqPerCta], seq_len[kSeqPerCta];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int base = blockIdx.x * kSeqPerCta;
    const bool writes_cum = blockIdx.y == 0;
    if (batch == 0) {
        if (tid == 0 && writes_cum) cum_seqlens[0] = 0;
        return;
    }
    // tokens in front of this chunk
    int part = 0;
    for (int b = tid; b < base; b += kSeqPerCta) part += clamp_len(__ldg(input_lengths + b), max_q_len);
    part = warp_sum(part);
    // inclusive scan of this chunk's lengths
    const int b = base + tid;
    const int len = b < batch ? clamp_len(__ldg(input_lengths + b), max_q_len) : 0;
    int incl = len;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 0) warp_tot[0][warp] = part;
    if (lane == 31) warp_tot[1][warp] = incl;
    __syncthreads();
    int before = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) before += warp_tot[0][w] + (w < warp ? warp_tot[1][w] : 0);
    const int start = before + incl - len;  // tokens before sequence b
    if (writes_cum && b < batch) {
        cum_seqlens[b] = start;
        if (b == batch - 1) cum_seqlens[batch] = start + len;
    }
    seq_start[tid] = start;
    seq_len[tid] = len;
    __syncthreads();
    const int in_chunk = min(kSeqPerCta, batch - base);
    const int first = blockIdx.y * 32 + lane, step = gridDim.y * 32;
    for (int j = warp; j < in_chunk; j += kWarps) {
        const int st = seq_start[j], n = seq_len[j], off = (base + j) * max_q_len - st;
        for (int i = first; i < n; i += step) padding_offset[st + i] = off;
    }
}

// ---- transpose + remove padding ---------------------------------------------------------------------
// out[t, h, :] = in[b, h, s, :] with (b, s) = divmod(t + padding_offset[t], seq_len):
// [b, h, s, d] -> [num_tokens, h, d] (tests/unittests/test_fused_trans_remv_pad.cu:3-4).
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
transpose_remove_padding_kernel(T* __restrict__ out, const T* __restrict__ in,
                                const int32_t* __restrict__ padding_offset, int64_t batch, int64_t seq_len,
                                int heads, int head_size, int64_t num_tokens, unsigned* __restrict__ status) {
    constexpr int E = VecTraits<T>::kElems;
    for (int64_t t = blockIdx.x; t < num_tokens; t += gridDim.x) {
        const int64_t dst = t + __ldg(padding_offset + t);
        if (dst < 0 || dst >= batch * seq_len) {
            if (threadIdx.x == 0) atomicOr(status, ISPORE_DEV_BAD_PADDING);
            continue;
        }
        const int64_t b = dst / seq_len, s = dst - b * seq_len;
        if (VEC) {
            const int head_vecs = head_size / E;
            const uint4* src = reinterpret_cast<const uint4*>(in) + ((b * heads) * seq_len + s) * head_vecs;
            uint4* o = reinterpret_cast<uint4*>(out) + t * heads * head_vecs;
            for (int i = threadIdx.x; i < heads * head_vecs; i += blockDim.x) {
                const int h = i / head_vecs, c = i - h * head_vecs;
                st_stream(o + i, ld_stream(src + static_cast<int64_t>(h) * seq_len * head_vecs + c));
            }
        } else {
            const T* src = in + ((b * heads) * seq_len + s) * head_size;
            T* o = out + t * heads * head_size;
            for (int i = threadIdx.x; i < heads * head_size; i += blockDim.x) {
                const int h = i / head_size, c = i - h * head_size;
                o[i] = src[static_cast<int64_t>(h) * seq_len * head_size + c];
            }
        }
    }
}

__device__ __forceinline__ uint4 ld_unit(const uint4* p) { return ld_stream(p); }
template <typename U>
__device__ __forceinline__ U ld_unit(const U* p) { return *p; }
__device__ __forceinline__ void st_unit(uint4* p, const uint4& x) { st_stream(p, x); }
template <typename U>
__device__ __forceinline__ void st_unit(U* p, const U& x) { *p = x; }

// ---- repeat-KV -----------------------------------------------------------------------------------------
// dst[b, h, s, :] = cache[layer, b, h / (heads/kv_heads), s, :] for s < context_length[b]
// (src/kernels/repeat_kv.cu:34-49).  For a fixed (b, kv head) the source and each of its
// heads/kv_heads destinations are contiguous spans: a CTA reads a piece of the source once and
// stores it q_per_kv times.
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
repeat_kv_kernel(T* __restrict__ k_dst, T* __restrict__ v_dst, const T* __restrict__ k_src,
                 const T* __restrict__ v_src, const int32_t* __restrict__ context_length,
                 int64_t layer_offset, int kv_heads, int q_per_kv, int64_t max_seq_len, int64_t max_k_len,
                 int head_size) {
    using Unit = typename std::conditional<VEC, uint4, T>::type;
    constexpr int E = VEC ? VecTraits<T>::kElems : 1;
    const int bkv = blockIdx.x;  // b * kv_heads + kv head
    const int b = bkv / kv_heads, kvh = bkv - b * kv_heads;
    const bool is_v = blockIdx.z != 0;
    int64_t len = __ldg(context_length + b);
    if (len > max_k_len) len = max_k_len;
    if (len > max_seq_len) len = max_seq_len;
    const Unit* src = reinterpret_cast<const Unit*>((is_v ? v_src : k_src) + layer_offset +
                                                    static_cast<int64_t>(bkv) * max_seq_len * head_size);
    const int64_t dst_head = max_k_len * head_size / E;  // units per destination head
    Unit* dst = reinterpret_cast<Unit*>(is_v ? v_dst : k_dst) +
                (static_cast<int64_t>(b) * kv_heads * q_per_kv + static_cast<int64_t>(kvh) * q_per_kv) * dst_head;
    const int64_t span = len * head_size / E;
    for (int64_t i = blockIdx.y * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < span;
         i += static_cast<int64_t>(gridDim.y) * blockDim.x) {
        const Unit x = VEC ? ld_unit(src + i) : src[i];
        for (int r = 0; r < q_per_kv; ++r) st_unit(dst + r * dst_head + i, x);
    }
}

template <typename T>
int mask_dispatch(T* mask, const int32_t* q_lens, const int32_t* k_lens, int64_t batch, int64_t max_q,
                  int64_t max_k, cudaStream_t st) {
    if (batch < 0 || max_q <= 0 || max_k <= 0 || max_q > INT32_MAX || max_k > INT32_MAX || batch > INT32_MAX)
        return fail(ISPORE_ESHAPE, "build_causal_mask: bad shape [%lld,%lld,%lld]", (long long)batch, (long long)max_q,
                    (long long)max_k);
    if (batch == 0) return ISPORE_OK;
    if (!mask || !q_lens || !k_lens) return fail(ISPORE_ENULL, "build_causal_mask: NULL buffer");
    constexpr int E = VecTraits<T>::kElems;
    const bool vec = (max_k % E == 0) && aligned16(mask);
    const int64_t per_row = vec ? max_k / E : max_k;
    const int64_t units = batch * max_q * per_row;
    if (vec) {
        const int64_t rows = batch * max_q;
        const int64_t ctas = ceil_div(rows, static_cast<int64_t>(kMaskWarps * kMaskRowsPerWarp));
        if (ctas <= INT32_MAX) {
            build_causal_mask_rows_kernel<T><<<static_cast<unsigned>(ctas), kMaskWarps * 32, 0, st>>>(
                mask, q_lens, k_lens, rows, static_cast<uint32_t>(max_q), static_cast<int>(per_row));
            return check_launch("build_causal_mask_rows_kernel");
        }
    }
    const int64_t want = ceil_div(units, 256);
    const unsigned blocks = static_cast<unsigned>(want < (1 << 22) ? want : (1 << 22));
    const uint32_t mq = static_cast<uint32_t>(max_q), pr = static_cast<uint32_t>(per_row);
    // 32-bit index arithmetic (one cheap division per vector) whenever the last grid-stride step cannot wrap
    if (units + static_cast<int64_t>(blocks) * 256 < (1ll << 32)) {
        if (vec)
            build_causal_mask_kernel<T, uint32_t, true><<<blocks, 256, 0, st>>>(mask, q_lens, k_lens, (uint32_t)units, mq, pr);
        else
            build_causal_mask_kernel<T, uint32_t, false><<<blocks, 256, 0, st>>>(mask, q_lens, k_lens, (uint32_t)units, mq, pr);
    } else {
        if (vec)
            build_causal_mask_kernel<T, int64_t, true><<<blocks, 256, 0, st>>>(mask, q_lens, k_lens, units, mq, pr);
        else
            build_causal_mask_kernel<T, int64_t, false><<<blocks, 256, 0, st>>>(mask, q_lens, k_lens, units, mq, pr);
    }
    return check_launch("build_causal_mask_kernel");
}

template <typename T>
int transpose_dispatch(T* out, const T* in, const int32_t* padding_offset, int64_t batch, int64_t heads,
                       int64_t seq_len, int64_t head_size, int64_t num_tokens, cudaStream_t st) {
    if (batch <= 0 || heads <= 0 || seq_len <= 0 || head_size <= 0 || num_tokens < 0 || heads > 65535 ||
        head_size > 65536 || num_tokens > batch * seq_len)
        return fail(ISPORE_ESHAPE, "transpose_remove_padding: bad shape");
    if (num_tokens == 0) return ISPORE_OK;
    if (!out || !in || !padding_offset) return fail(ISPORE_ENULL, "transpose_remove_padding: NULL buffer");
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "transpose_remove_padding: no device status word");
    constexpr int E = VecTraits<T>::kElems;
    const int grid = static_cast<int>(num_tokens < (1ll << 30) ? num_tokens : (1ll << 30));
    if (head_size % E == 0 && aligned16(out) && aligned16(in))
        transpose_remove_padding_kernel<T, true><<<grid, 128, 0, st>>>(out, in, padding_offset, batch, seq_len,
                                                                       (int)heads, (int)head_size, num_tokens, status);
    else
        transpose_remove_padding_kernel<T, false><<<grid, 128, 0, st>>>(out, in, padding_offset, batch, seq_len,
                                                                        (int)heads, (int)head_size, num_tokens, status);
    return check_launch("transpose_remove_padding_kernel");
}

template <typename T>
int repeat_dispatch(T* k_dst, T* v_dst, const T* k_src, const T* v_src, const int32_t* context_length,
                    int64_t layer, int64_t num_layers, int64_t batch, int64_t kv_heads, int64_t heads,
                    int64_t max_seq_len, int64_t max_k_len, int64_t head_size, cudaStream_t st) {
    if (batch < 0 || kv_heads <= 0 || heads <= 0 || heads % kv_heads != 0 || max_seq_len <= 0 || max_k_len <= 0 ||
        head_size <= 0 || layer < 0 || (num_layers > 0 && layer >= num_layers) || batch * heads > INT32_MAX)
        return fail(ISPORE_ESHAPE, "repeat_kv: bad shape layer=%lld/%lld bs=%lld heads=%lld/%lld", (long long)layer,
                    (long long)num_layers, (long long)batch, (long long)heads, (long long)kv_heads);
    if (batch == 0) return ISPORE_OK;
    if (!k_dst || !v_dst || !k_src || !v_src || !context_length) return fail(ISPORE_ENULL, "repeat_kv: NULL buffer");
    constexpr int E = VecTraits<T>::kElems;
    const int64_t layer_offset = layer * batch * kv_heads * max_seq_len * head_size;
    const bool vec = head_size % E == 0 && aligned16(k_dst) && aligned16(v_dst) && aligned16(k_src) && aligned16(v_src);
    int64_t gx = ceil_div(max_k_len * head_size / (vec ? E : 1), 128 * 2);
    if (gx > 1024) gx = 1024;
    if (gx < 1) gx = 1;
    dim3 grid(static_cast<unsigned>(batch * kv_heads), static_cast<unsigned>(gx), 2);
    if (vec)
        repeat_kv_kernel<T, true><<<grid, 128, 0, st>>>(k_dst, v_dst, k_src, v_src, context_length, layer_offset,
                                                        (int)kv_heads, (int)(heads / kv_heads), max_seq_len, max_k_len,
                                                        (int)head_size);
    else
        repeat_kv_kernel<T, false><<<grid, 128, 0, st>>>(k_dst, v_dst, k_src, v_src, context_length, layer_offset,
                                                         (int)kv_heads, (int)(heads / kv_heads), max_seq_len, max_k_len,
                                                         (int)head_size);
    return check_launch("repeat_kv_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {

int ispore_build_causal_mask_f32(float* mask, const int32_t* q_lens, const int32_t* k_lens, int64_t batch_size,
                                 int64_t max_q_len, int64_t max_k_len, ispore_stream_t stream) {
    return ispore::mask_dispatch<float>(mask, q_lens, k_lens, batch_size, max_q_len, max_k_len,
                                        static_cast<cudaStream_t>(stream));
}
int ispore_build_causal_mask_f16(void* mask, const int32_t* q_lens, const int32_t* k_lens, int64_t batch_size,
                                 int64_t max_q_len, int64_t max_k_len, ispore_stream_t stream) {
    return ispore::mask_dispatch<__half>(static_cast<__half*>(mask), q_lens, k_lens, batch_size, max_q_len, max_k_len,
                                         static_cast<cudaStream_t>(stream));
}

int ispore_cal_padding_offset(int32_t* padding_offset, int32_t* cum_seqlens, const int32_t* input_lengths,
                              int64_t batch_size, int64_t max_q_len, ispore_stream_t stream) {
    if (batch_size < 0 || max_q_len <= 0 || batch_size > (1 << 24) || batch_size * max_q_len > INT32_MAX)
        return ispore::fail(ISPORE_ESHAPE, "cal_padding_offset: bad shape [%lld,%lld]", (long long)batch_size,
                            (long long)max_q_len);
    if (!cum_seqlens || (batch_size > 0 && (!padding_offset || !input_lengths)))
        return ispore::fail(ISPORE_ENULL, "cal_padding_offset: NULL buffer");
    const unsigned chunks = batch_size > 0 ? static_cast<unsigned>(ispore::ceil_div(batch_size, ispore::kSeqPerCta)) : 1u;
    // split long sequences over up to 16 CTAs per chunk; short ones need no split
    unsigned split = static_cast<unsigned>(ispore::ceil_div(max_q_len, 256));
    if (split > 16) split = 16;
    if (chunks >= 32) split = 1;
    ispore::padding_offset_kernel<<<dim3(chunks, split), ispore::kSeqPerCta, 0, static_cast<cudaStream_t>(stream)>>>(
        padding_offset, cum_seqlens, input_lengths, static_cast<int>(batch_size), static_cast<int>(max_q_len));
    return ispore::check_launch("padding_offset_kernel");
}

int ispore_transpose_remove_padding_f32(float* out, const float* in, const int32_t* padding_offset,
                                        int64_t batch_size, int64_t head_num, int64_t seq_len, int64_t head_size,
                                        int64_t num_tokens, ispore_stream_t stream) {
    return ispore::transpose_dispatch<float>(out, in, padding_offset, batch_size, head_num, seq_len, head_size,
                                             num_tokens, static_cast<cudaStream_t>(stream));
}
int ispore_transpose_remove_padding_f16(void* out, const void* in, const int32_t* padding_offset, int64_t batch_size,
                                        int64_t head_num, int64_t seq_len, int64_t head_size, int64_t num_tokens,
                                        ispore_stream_t stream) {
    return ispore::transpose_dispatch<__half>(static_cast<__half*>(out), static_cast<const __half*>(in), padding_offset,
                                              batch_size, head_num, seq_len, head_size, num_tokens,
                                              static_cast<cudaStream_t>(stream));
}

int ispore_repeat_kv_f32(float* k_dst, float* v_dst, const float* k_src, const float* v_src,
                         const int32_t* context_length, int64_t layer, int64_t num_layers, int64_t batch_size,
                         int64_t kv_head_num, int64_t head_num, int64_t max_seq_len, int64_t max_k_len,
                         int64_t head_size, ispore_stream_t stream) {
    return ispore::repeat_dispatch<float>(k_dst, v_dst, k_src, v_src, context_length, layer, num_layers, batch_size,
                                          kv_head_num, head_num, max_seq_len, max_k_len, head_size,
                                          static_cast<cudaStream_t>(stream));
}
int ispore_repeat_kv_f16(void* k_dst, void* v_dst, const void* k_src, const void* v_src,
                         const int32_t* context_length, int64_t layer, int64_t num_layers, int64_t batch_size,
                         int64_t kv_head_num, int64_t head_num, int64_t max_seq_len, int64_t max_k_len,
                         int64_t head_size, ispore_stream_t stream) {
    return ispore::repeat_dispatch<__half>(static_cast<__half*>(k_dst), static_cast<__half*>(v_dst),
                                           static_cast<const __half*>(k_src), static_cast<const __half*>(v_src),
                                           context_length, layer, num_layers, batch_size, kv_head_num, head_num,
                                           max_seq_len, max_k_len, head_size, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
