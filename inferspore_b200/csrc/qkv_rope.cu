// QKV bias + RoPE + un-pad + head transpose (prefill) and in-place decode RoPE
// for sm_100a.
//
// Semantics: the reference's fp32 kernel, src/kernels/qkv_bias_and_RoPE.cu:110-192,
// with the bias add its fp16 draft describes (:236-252) applied before the
// rotation; rotation pairs are (j, j + head_size/2) (:47-53, :182-190);
// theta_j = m / powf(base, 2j/rot_dim) (:38-45).
//
// The reference launches one CTA per (token, head) and recomputes
// powf+cos+sin for every head.  Here one CTA owns a token: cos/sin for the
// token's position are computed once into shared memory (rot_dim/2 sincosf
// calls) and reused by all q and k heads; every thread moves 128-bit vectors —
// the low-half vector and its partner in the high half — so a warp reads 1 KB
// of contiguous QKV and writes whole 256-byte head rows of the transposed
// outputs.  The powf denominators are evaluated on the host and travel as a
// kernel argument.
#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "tma.cuh"

namespace ispore {
namespace {

constexpr int kMaxRotHalf = 256;
struct RopeDenominators {
    float d[kMaxRotHalf];  // powf(base, 2j / rot_dim)
};

int fill_denominators(RopeDenominators* out, int rot_dim, float base) {
    if (rot_dim < 0 || rot_dim / 2 > kMaxRotHalf) return -1;
    for (int j = 0; j < rot_dim / 2; ++j)
        out->d[j] = powf(base, static_cast<float>(2 * j) / static_cast<float>(rot_dim));
    return 0;
}

// HEAD_SIZE > 0 fixes the head size at compile time (the task -> (head, vector) split becomes
// shifts instead of run-time divisions, which otherwise cost as much as the arithmetic);
// HEAD_SIZE == 0 takes it from the argument.  FULL_ROT: rotary_dim == head_size, so the
// per-element "is this pair rotated" test disappears.  HAS_BIAS likewise.
template <typename T, int THREADS, int HEAD_SIZE, bool FULL_ROT, bool HAS_BIAS, int STORE = 0>
__global__ void __launch_bounds__(THREADS)
qkv_rope_transpose_vec_kernel(T* __restrict__ q_buf, T* __restrict__ k_buf, T* __restrict__ v_buf,
                              const T* __restrict__ QKV, const T* __restrict__ bias,
                              const int32_t* __restrict__ padding_offset,
                              const int32_t* __restrict__ history_length, int64_t batch_size,
                              int64_t seq_len, int64_t token_num, int head_num, int kv_head_num,
                              int head_size_arg, int rot_half, const RopeDenominators freq,
                              unsigned* __restrict__ status) {
    constexpr int E = VecTraits<T>::kElems;
    __shared__ float2 cos_sin[kMaxRotHalf];
    chain_begin();
    const int tid = threadIdx.x;
    const int head_size = HEAD_SIZE > 0 ? HEAD_SIZE : head_size_arg;
    const int head_vecs = head_size / E;
    const int half_vecs = head_vecs / 2;
    const int qkv_heads = head_num + 2 * kv_head_num;
    const int rope_tasks = (head_num + kv_head_num) * half_vecs;
    const int v_tasks = kv_head_num * head_vecs;
    const uint4* bias_v = reinterpret_cast<const uint4*>(bias);

    constexpr int U = 4;  // tasks per thread per trip
    for (int64_t token = blockIdx.x; token < token_num; token += gridDim.x) {
        // The token's data does not depend on where it lands: start the first trip's loads
        // now, so they fly while the position is looked up and cos/sin are evaluated.
        const uint4* src = reinterpret_cast<const uint4*>(QKV) + token * qkv_heads * head_vecs;
        const uint4* vsrc = src + (head_num + kv_head_num) * head_vecs;
        uint4 lo_raw[U], hi_raw[U], v_raw[U];
        auto load_rope_trip = [&](int task0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int task = task0 + u * THREADS;
                if (task < rope_tasks) {
                    const int hh = task / half_vecs;
                    const int c = task - hh * half_vecs;
                    lo_raw[u] = ld_stream(src + hh * head_vecs + c);
                    hi_raw[u] = ld_stream(src + hh * head_vecs + half_vecs + c);
                }
            }
        };
        auto load_v_trip = [&](int task0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int task = task0 + u * THREADS;
                if (task < v_tasks) v_raw[u] = ld_stream(vsrc + task);
            }
        };
        load_rope_trip(tid);
        load_v_trip(tid);
        const int64_t dst_token = token + __ldg(padding_offset + token);
        if (dst_token < 0 || dst_token >= batch_size * seq_len) {
            if (tid == 0) atomicOr(status, ISPORE_DEV_BAD_PADDING);
            continue;  // uniform over the CTA
        }
        // One 64-bit division per token (32-bit when the destination index allows it).
        int64_t b, s;
        if (dst_token < (1ll << 31) && seq_len < (1ll << 31)) {
            const uint32_t bq = static_cast<uint32_t>(dst_token) / static_cast<uint32_t>(seq_len);
            b = bq;
            s = static_cast<uint32_t>(dst_token) - bq * static_cast<uint32_t>(seq_len);
        } else {
            b = dst_token / seq_len;
            s = dst_token - b * seq_len;
        }
        const float m = static_cast<float>(__ldg(history_length + b) + static_cast<int>(s));

        __syncthreads();  // previous token's readers are done with cos_sin
        for (int j = tid; j < rot_half; j += THREADS) {
            float sn, cs;
            sincosf(m / freq.d[j], &sn, &cs);
            cos_sin[j] = make_float2(cs, sn);
        }
        __syncthreads();

        // Row (b, head 0, s) of q and of k/v, in vectors; heads are seq_len*head_vecs apart.
        const int64_t head_stride = seq_len * head_vecs;
        uint4* q_row = reinterpret_cast<uint4*>(q_buf) + (b * head_num * seq_len + s) * head_vecs;
        uint4* k_row = reinterpret_cast<uint4*>(k_buf) + (b * kv_head_num * seq_len + s) * head_vecs;
        uint4* v_row = reinterpret_cast<uint4*>(v_buf) + (b * kv_head_num * seq_len + s) * head_vecs;

        // q and k heads: rotate (low-half vector, high-half vector) pairs, U tasks per trip
        // with all loads of the trip issued before the first use.
        for (int task0 = tid; task0 < rope_tasks; task0 += THREADS * U) {
            if (task0 != tid) load_rope_trip(task0);  // the first trip is already on its way
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int task = task0 + u * THREADS;
                if (task < rope_tasks) {
                    const int hh = task / half_vecs;  // head index inside [q heads | k heads]
                    const int c = task - hh * half_vecs;
                    Unpacked<T> lo, hi;
                    unpack(lo_raw[u], lo);
                    unpack(hi_raw[u], hi);
                    if (HAS_BIAS) {
                        Unpacked<T> blo, bhi;
                        unpack(ld_keep(bias_v + hh * head_vecs + c), blo);
                        unpack(ld_keep(bias_v + hh * head_vecs + half_vecs + c), bhi);
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            lo.v[e] += blo.v[e];
                            hi.v[e] += bhi.v[e];
                        }
                    }
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        const int j = c * E + e;
                        if (FULL_ROT || j < rot_half) {
                            const float2 cs = cos_sin[j];
                            const float x0 = lo.v[e], x1 = hi.v[e];
                            lo.v[e] = cs.x * x0 - cs.y * x1;
                            hi.v[e] = cs.x * x1 + cs.y * x0;
                        }
                    }
                    const bool is_q = hh < head_num;
                    uint4* dst = is_q ? q_row + hh * head_stride : k_row + (hh - head_num) * head_stride;
                    if (STORE == 0) {
                        st_stream(dst + c, pack(lo));
                        st_stream(dst + half_vecs + c, pack(hi));
                    } else {
                        dst[c] = pack(lo);
                        dst[half_vecs + c] = pack(hi);
                    }
                }
            }
        }

        // v heads: bias add and transposed copy.
        for (int task0 = tid; task0 < v_tasks; task0 += THREADS * U) {
            if (task0 != tid) load_v_trip(task0);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int task = task0 + u * THREADS;
                if (task < v_tasks) {
                    const int h = task / head_vecs;
                    const int c = task - h * head_vecs;
                    if (HAS_BIAS) {
                        Unpacked<T> x, bb;
                        unpack(v_raw[u], x);
                        unpack(ld_keep(bias_v + (head_num + kv_head_num) * head_vecs + task), bb);
#pragma unroll
                        for (int e = 0; e < E; ++e) x.v[e] += bb.v[e];
                        v_raw[u] = pack(x);
                    }
                    if (STORE == 0) st_stream(v_row + h * head_stride + c, v_raw[u]);
                    else v_row[h * head_stride + c] = v_raw[u];
                }
            }
        }
    }
}

// The same work with the token staged through shared memory: a token's q, k and v heads are one
// contiguous span of QKV (24 KB for Llama-2-7B in fp16), so one thread starts TMA bulk copies of
// the whole span and the CTA looks up the position and evaluates cos/sin while they fly.  No
// registers are tied up holding loads in flight, which lets eight CTAs (and their 8 x 24 KB of
// outstanding reads) share an SM.  HEAD_SIZE == 0 and FULL_ROT == false cover any head size (a
// multiple of two vectors) and partial rotation at the price of run-time index divisions.
// One token per CTA makes a launch cost a whole number of waves of resident CTAs plus about one
// more for the ramp (8192 tokens: 78 us for 62 us of traffic, 65536 tokens: at the copy rate).
// Measured and not kept: one CTA per resident slot walking the tokens with a ring of two to four
// token buffers and the next token's position and cos/sin table prepared a token ahead — 10 to
// 25 % slower at every token count, more so with more buffers: what carries this kernel is the
// number of CTAs an SM overlaps (nine of these), not the depth of any one CTA's queue.
constexpr int kTmaPiece = 8192;
constexpr int64_t kSplitTokens = 16384;  // launches up to this many tokens run three CTAs per token

template <typename T, int THREADS, int HEAD_SIZE, bool FULL_ROT, bool HAS_BIAS>
__global__ void __launch_bounds__(THREADS)
qkv_rope_transpose_tma_kernel(T* __restrict__ q_buf, T* __restrict__ k_buf, T* __restrict__ v_buf,
                              const T* __restrict__ QKV, const T* __restrict__ bias,
                              const int32_t* __restrict__ padding_offset,
                              const int32_t* __restrict__ history_length, int64_t batch_size,
                              int64_t seq_len, int head_num, int kv_head_num, int head_size_arg, int rot_half_arg,
                              const RopeDenominators freq, unsigned* __restrict__ status) {
    constexpr int E = VecTraits<T>::kElems;
    // compile-time head size: the task -> (head, vector) split is shifts; 0: taken from the argument
    const int head_size = HEAD_SIZE > 0 ? HEAD_SIZE : head_size_arg;
    const int kHeadVecs = head_size / E, kHalfVecs = kHeadVecs / 2;
    const int kRotHalf = FULL_ROT ? head_size / 2 : rot_half_arg;
    extern __shared__ __align__(128) unsigned char token_raw[];
    __shared__ float2 cos_sin[HEAD_SIZE > 0 ? HEAD_SIZE / 2 : kMaxRotHalf];
    __shared__ __align__(8) uint64_t bar;
    chain_begin();
    const int tid = threadIdx.x;
    const int qkv_heads = head_num + 2 * kv_head_num;
    const int64_t token = blockIdx.x;
    // gridDim.y == 3: the CTA takes the token's q heads, its k heads or its v heads only.
    int first_head = 0, last_head = qkv_heads;
    if (gridDim.y == 3) {
        first_head = blockIdx.y == 0 ? 0 : blockIdx.y == 1 ? head_num : head_num + kv_head_num;
        last_head = blockIdx.y == 0 ? head_num : blockIdx.y == 1 ? head_num + kv_head_num : qkv_heads;
    }
    const uint32_t head_bytes = static_cast<uint32_t>(head_size) * sizeof(T);
    const uint32_t bytes = static_cast<uint32_t>(last_head - first_head) * head_bytes;
    if (tid == 0) {
        tma::mbar_init(&bar, 1);
        tma::fence_mbar_init();
        tma::mbar_arrive_expect_tx(&bar, bytes);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(QKV) +
                                   (token * qkv_heads + first_head) * static_cast<int64_t>(head_bytes);
        for (uint32_t off = 0; off < bytes; off += kTmaPiece)
            tma::load(token_raw + off, src + off, min(static_cast<uint32_t>(kTmaPiece), bytes - off), &bar);
    }
    const int64_t dst_token = token + __ldg(padding_offset + token);
    const bool bad = dst_token < 0 || dst_token >= batch_size * seq_len;
    int64_t b = 0, s = 0;
    if (!bad) {
        if (dst_token < (1ll << 31) && seq_len < (1ll << 31)) {
            const uint32_t bq = static_cast<uint32_t>(dst_token) / static_cast<uint32_t>(seq_len);
            b = bq;
            s = static_cast<uint32_t>(dst_token) - bq * static_cast<uint32_t>(seq_len);
        } else {
            b = dst_token / seq_len;
            s = dst_token - b * seq_len;
        }
        if (first_head < head_num + kv_head_num) {  // v heads are not rotated
            const float m = static_cast<float>(__ldg(history_length + b) + static_cast<int>(s));
            for (int j = tid; j < kRotHalf; j += THREADS) {
                float sn, cs;
                sincosf(m / freq.d[j], &sn, &cs);
                cos_sin[j] = make_float2(cs, sn);
            }
        }
    }
    __syncthreads();  // cos/sin written; the barrier's initialisation is visible to every waiter
    // The copies land in this CTA's shared memory: wait for them even when the token is skipped.
    if (!tma::mbar_wait(&bar, 0)) {
        if (tid == 0) atomicOr(status, ISPORE_DEV_TIMEOUT);
        return;
    }
    if (bad) {
        if (tid == 0) atomicOr(status, ISPORE_DEV_BAD_PADDING);
        return;
    }
    const uint4* tok = reinterpret_cast<const uint4*>(token_raw);
    const uint4* bias_v = reinterpret_cast<const uint4*>(bias);
    const int64_t head_stride = seq_len * kHeadVecs;
    uint4* q_row = reinterpret_cast<uint4*>(q_buf) + (b * head_num * seq_len + s) * kHeadVecs;
    uint4* k_row = reinterpret_cast<uint4*>(k_buf) + (b * kv_head_num * seq_len + s) * kHeadVecs;
    uint4* v_row = reinterpret_cast<uint4*>(v_buf) + (b * kv_head_num * seq_len + s) * kHeadVecs;
    // (tok holds the heads first_head .. last_head - 1 of the token)
    const int rope_end = min(last_head, head_num + kv_head_num);
    const int rope_tasks = rope_end > first_head ? (rope_end - first_head) * kHalfVecs : 0;
    const int v_first = max(first_head, head_num + kv_head_num);  // first v head held, as a qkv head index
    const int v_tasks = (last_head - v_first) * kHeadVecs;
    for (int task = tid; task < rope_tasks; task += THREADS) {
        const int hl = task / kHalfVecs, c = task % kHalfVecs;
        const int hh = first_head + hl;
        Unpacked<T> lo, hi;
        unpack(tok[hl * kHeadVecs + c], lo);
        unpack(tok[hl * kHeadVecs + kHalfVecs + c], hi);
        if (HAS_BIAS) {
            Unpacked<T> blo, bhi;
            unpack(ld_keep(bias_v + hh * kHeadVecs + c), blo);
            unpack(ld_keep(bias_v + hh * kHeadVecs + kHalfVecs + c), bhi);
#pragma unroll
            for (int e = 0; e < E; ++e) {
                lo.v[e] += blo.v[e];
                hi.v[e] += bhi.v[e];
            }
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
            if (FULL_ROT || c * E + e < kRotHalf) {
                const float2 cs = cos_sin[c * E + e];
                const float x0 = lo.v[e], x1 = hi.v[e];
                lo.v[e] = cs.x * x0 - cs.y * x1;
                hi.v[e] = cs.x * x1 + cs.y * x0;
            }
        }
        uint4* dst = hh < head_num ? q_row + hh * head_stride : k_row + (hh - head_num) * head_stride;
        st_stream(dst + c, pack(lo));
        st_stream(dst + kHalfVecs + c, pack(hi));
    }
    const uint4* vtok = tok + (v_first - first_head) * kHeadVecs;
    for (int task = tid; task < v_tasks; task += THREADS) {
        const int h = task / kHeadVecs, c = task % kHeadVecs;  // (every v head of the token is held when any is)
        uint4 raw = vtok[task];
        if (HAS_BIAS) {
            Unpacked<T> x, bb;
            unpack(raw, x);
            unpack(ld_keep(bias_v + (head_num + kv_head_num) * kHeadVecs + task), bb);
#pragma unroll
            for (int e = 0; e < E; ++e) x.v[e] += bb.v[e];
            raw = pack(x);
        }
        st_stream(v_row + h * head_stride + c, raw);
    }
}

// Any head size / alignment (head_size even): one thread per rotation pair.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
qkv_rope_transpose_scalar_kernel(T* __restrict__ q_buf, T* __restrict__ k_buf, T* __restrict__ v_buf,
                                 const T* __restrict__ QKV, const T* __restrict__ bias,
                                 const int32_t* __restrict__ padding_offset,
                                 const int32_t* __restrict__ history_length, int64_t batch_size,
                                 int64_t seq_len, int64_t token_num, int head_num, int kv_head_num,
                                 int head_size, int rot_half, const RopeDenominators freq,
                                 unsigned* __restrict__ status) {
    const int tid = threadIdx.x;
    const int half = head_size / 2;
    const int qkv_heads = head_num + 2 * kv_head_num;
    for (int64_t token = blockIdx.x; token < token_num; token += gridDim.x) {
        const int64_t dst_token = token + padding_offset[token];
        if (dst_token < 0 || dst_token >= batch_size * seq_len) {
            if (tid == 0) atomicOr(status, ISPORE_DEV_BAD_PADDING);
            continue;
        }
        const int64_t b = dst_token / seq_len;
        const int64_t s = dst_token - b * seq_len;
        const float m = static_cast<float>(history_length[b] + static_cast<int>(s));
        const T* src = QKV + token * qkv_heads * head_size;
        for (int task = tid; task < (head_num + kv_head_num) * half; task += THREADS) {
            const int hh = task / half, j = task - hh * half;
            float x0 = to_float<T>(src[hh * head_size + j]);
            float x1 = to_float<T>(src[hh * head_size + half + j]);
            if (bias != nullptr) {
                x0 += to_float<T>(bias[hh * head_size + j]);
                x1 += to_float<T>(bias[hh * head_size + half + j]);
            }
            float o0 = x0, o1 = x1;
            if (j < rot_half) {
                float sn, cs;
                sincosf(m / freq.d[j], &sn, &cs);
                o0 = cs * x0 - sn * x1;
                o1 = cs * x1 + sn * x0;
            }
            const bool is_q = hh < head_num;
            const int h = is_q ? hh : hh - head_num;
            T* base = is_q ? q_buf : k_buf;
            const int64_t heads = is_q ? head_num : kv_head_num;
            T* dst = base + ((b * heads + h) * seq_len + s) * head_size;
            dst[j] = from_float<T>(o0);
            dst[half + j] = from_float<T>(o1);
        }
        const int v_at = (head_num + kv_head_num) * head_size;
        for (int task = tid; task < kv_head_num * head_size; task += THREADS) {
            const int h = task / head_size, j = task - h * head_size;
            float x = to_float<T>(src[v_at + task]);
            if (bias != nullptr) x += to_float<T>(bias[v_at + task]);
            v_buf[((b * kv_head_num + h) * seq_len + s) * head_size + j] = from_float<T>(x);
        }
    }
}

// Decode step: rotate q and k heads of qkv_buf[batch, heads, head_size] in place
// at position step-1 (reference: src/kernels/qkv_bias_and_RoPE.cu:352-390).
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
rope_decode_kernel(T* __restrict__ qkv, int head_num, int kv_head_num, int head_size, int rot_half,
                   float position, const RopeDenominators freq) {
    __shared__ float2 cos_sin[kMaxRotHalf];
    chain_begin();
    const int tid = threadIdx.x;
    for (int j = tid; j < rot_half; j += THREADS) {
        float sn, cs;
        sincosf(position / freq.d[j], &sn, &cs);
        cos_sin[j] = make_float2(cs, sn);
    }
    __syncthreads();
    const int half = head_size / 2;
    T* row = qkv + static_cast<int64_t>(blockIdx.x) * (head_num + 2 * kv_head_num) * head_size;
    for (int task = tid; task < (head_num + kv_head_num) * rot_half; task += THREADS) {
        const int hh = task / rot_half, j = task - hh * rot_half;
        T* p = row + hh * head_size;
        const float x0 = to_float<T>(p[j]), x1 = to_float<T>(p[half + j]);
        const float2 cs = cos_sin[j];
        p[j] = from_float<T>(cs.x * x0 - cs.y * x1);
        p[half + j] = from_float<T>(cs.x * x1 + cs.y * x0);
    }
}

template <typename T>
int qkv_dispatch(T* q_buf, T* k_buf, T* v_buf, const T* QKV, const T* bias,
                 const int32_t* padding_offset, const int32_t* history_length, int64_t batch_size,
                 int64_t seq_len, int64_t token_num, int64_t head_num, int64_t kv_head_num,
                 int64_t head_size, int32_t rot_dim, float base, cudaStream_t st) {
    if (batch_size <= 0 || seq_len <= 0 || token_num < 0 || head_num <= 0 || kv_head_num <= 0 ||
        head_size <= 0 || head_size % 2 != 0 || head_num > 65535 || kv_head_num > 65535 ||
        head_size > 65536)
        return fail(ISPORE_ESHAPE,
                    "qkv_bias_rope_transpose: bad shape bs=%lld seq=%lld tokens=%lld heads=%lld/%lld d=%lld",
                    (long long)batch_size, (long long)seq_len, (long long)token_num,
                    (long long)head_num, (long long)kv_head_num, (long long)head_size);
    if (token_num > batch_size * seq_len)
        return fail(ISPORE_ESHAPE, "qkv_bias_rope_transpose: %lld packed tokens exceed bs*seq=%lld",
                    (long long)token_num, (long long)(batch_size * seq_len));
    if (rot_dim < 0 || rot_dim % 2 != 0 || rot_dim > head_size)
        return fail(ISPORE_ESHAPE, "qkv_bias_rope_transpose: rotary dim %d vs head size %lld", rot_dim,
                    (long long)head_size);
    RopeDenominators freq;
    if (fill_denominators(&freq, rot_dim, base) != 0)
        return fail(ISPORE_ELIMIT, "qkv_bias_rope_transpose: rotary dim %d > %d", rot_dim, 2 * kMaxRotHalf);
    if (token_num == 0) return ISPORE_OK;
    if (!q_buf || !k_buf || !v_buf || !QKV || !padding_offset || !history_length)
        return fail(ISPORE_ENULL, "qkv_bias_rope_transpose: NULL buffer");
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "qkv_bias_rope_transpose: no device status word");

    constexpr int THREADS = 256;
    constexpr int E = VecTraits<T>::kElems;
    const bool vec_ok = head_size % (2 * E) == 0 && aligned16(q_buf) && aligned16(k_buf) &&
                        aligned16(v_buf) && aligned16(QKV) && (bias == nullptr || aligned16(bias));
    if (vec_ok) {
        // One token per CTA, as many CTAs as tokens: measured faster on B200 than a persistent
        // grid-stride loop (the CTA scheduler walks the tokens in address order).
        constexpr int TH = 64;
        const int grid = static_cast<int>(token_num < (1ll << 30) ? token_num : (1ll << 30));
        const bool full_rot = rot_dim == head_size;
        const bool has_bias = bias != nullptr;
#define ISPORE_QKV(HS, FR, HB)                                                                           \
    do {                                                                                                 \
        launch_chained(qkv_rope_transpose_vec_kernel<T, TH, HS, FR, HB>, grid, TH, 0, st,                \
            q_buf, k_buf, v_buf, QKV, bias, padding_offset, history_length, batch_size, seq_len,        \
            token_num, (int)head_num, (int)kv_head_num, (int)head_size, rot_dim / 2, freq, status);     \
        return check_launch("qkv_rope_transpose_vec_kernel");                                           \
    } while (0)
        // The shared-memory staged kernel: compile-time head size and full rotation for the usual
        // shapes, run-time head size / partial rotation otherwise.
        const int64_t token_bytes = (head_num + 2 * kv_head_num) * head_size * static_cast<int64_t>(sizeof(T));
        if (token_bytes <= 96 * 1024 && token_num < (1ll << 31) && head_size <= 2 * kMaxRotHalf && tune(kTuneQkv, 0) != 1) {
            // One CTA per token, or three (its q, k and v heads) while the launch is short: a launch
            // costs a whole number of waves of resident CTAs plus about one for the ramp, and CTAs
            // of a third of the bytes make the waves shorter (measured, 32 + 32 + 32 heads of 128:
            // 4096 tokens 45 -> 40 us, 8192 tokens 76 -> 72 us, 16384 tokens 137 -> 135 us; at
            // 65536 tokens the single CTA is 2 % faster; 64-thread CTAs for the thirds: no better; four to
            // twelve equal runs of heads per token instead of three: slower from 4096 tokens up).
            const bool split = tune(kTuneQkv, 0) == 3 || (tune(kTuneQkv, 0) != 2 && token_num <= kSplitTokens);
            const int64_t part_bytes = split ? std::max(head_num, kv_head_num) * head_size * static_cast<int64_t>(sizeof(T)) : token_bytes;
            const dim3 tma_grid(static_cast<unsigned>(token_num), split ? 3u : 1u);
#define ISPORE_QKV_TMA(HS, FR, HB)                                                                          \
    do {                                                                                                    \
        constexpr int TH = 128; /* measured: 64 and 256 threads are 3-6 % slower */                         \
        auto kernel = qkv_rope_transpose_tma_kernel<T, TH, HS, FR, HB>;                                     \
        if (!allow_dynamic_smem(kernel, static_cast<size_t>(part_bytes))) break;                            \
        launch_chained(kernel, tma_grid, TH, static_cast<size_t>(part_bytes), st,                           \
            q_buf, k_buf, v_buf, QKV, bias, padding_offset, history_length, batch_size, seq_len,           \
            (int)head_num, (int)kv_head_num, (int)head_size, rot_dim / 2, freq, status);                    \
        return check_launch("qkv_rope_transpose_tma_kernel");                                               \
    } while (0)
            if (full_rot && head_size == 128) {
                if (has_bias) ISPORE_QKV_TMA(128, true, true);
                else ISPORE_QKV_TMA(128, true, false);
            } else if (full_rot && head_size == 64) {
                if (has_bias) ISPORE_QKV_TMA(64, true, true);
                else ISPORE_QKV_TMA(64, true, false);
            } else if (full_rot) {
                if (has_bias) ISPORE_QKV_TMA(0, true, true);
                else ISPORE_QKV_TMA(0, true, false);
            } else {
                if (has_bias) ISPORE_QKV_TMA(0, false, true);
                else ISPORE_QKV_TMA(0, false, false);
            }
#undef ISPORE_QKV_TMA
        }
        if (head_size == 128 && full_rot) {
            if (has_bias) ISPORE_QKV(128, true, true);
            ISPORE_QKV(128, true, false);
        }
        if (head_size == 64 && full_rot) {
            if (has_bias) ISPORE_QKV(64, true, true);
            ISPORE_QKV(64, true, false);
        }
        if (has_bias) ISPORE_QKV(0, false, true);
        ISPORE_QKV(0, false, false);
#undef ISPORE_QKV
    }
    const int grid = persistent_grid(qkv_rope_transpose_scalar_kernel<T, THREADS>, THREADS, 0, token_num);
    qkv_rope_transpose_scalar_kernel<T, THREADS><<<grid, THREADS, 0, st>>>(
        q_buf, k_buf, v_buf, QKV, bias, padding_offset, history_length, batch_size, seq_len, token_num,
        (int)head_num, (int)kv_head_num, (int)head_size, rot_dim / 2, freq, status);
    return check_launch("qkv_rope_transpose_scalar_kernel");
}

template <typename T>
int rope_decode_dispatch(T* qkv, int64_t batch, int64_t head_num, int64_t kv_head_num,
                         int64_t head_size, int32_t step, int32_t rot_dim, float base, cudaStream_t st) {
    if (batch < 0 || head_num <= 0 || kv_head_num <= 0 || head_size <= 0 || head_size % 2 != 0 ||
        head_num > 65535 || kv_head_num > 65535 || head_size > 65536 || batch > INT32_MAX)
        return fail(ISPORE_ESHAPE, "rope_decode: bad shape");
    if (rot_dim < 0 || rot_dim % 2 != 0 || rot_dim > head_size)
        return fail(ISPORE_ESHAPE, "rope_decode: rotary dim %d vs head size %lld", rot_dim, (long long)head_size);
    RopeDenominators freq;
    if (fill_denominators(&freq, rot_dim, base) != 0)
        return fail(ISPORE_ELIMIT, "rope_decode: rotary dim %d > %d", rot_dim, 2 * kMaxRotHalf);
    if (batch == 0) return ISPORE_OK;
    if (!qkv) return fail(ISPORE_ENULL, "rope_decode: NULL buffer");
    constexpr int THREADS = 256;
    launch_chained(rope_decode_kernel<T, THREADS>, static_cast<int>(batch), THREADS, 0, st,
        qkv, (int)head_num, (int)kv_head_num, (int)head_size, rot_dim / 2,
        static_cast<float>(step - 1), freq);
    return check_launch("rope_decode_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {

int ispore_qkv_bias_rope_transpose_f32(float* q_buf, float* k_buf, float* v_buf, const float* QKV,
                                       const float* bias, const int32_t* padding_offset,
                                       const int32_t* history_length, const int32_t* input_length,
                                       int64_t batch_size, int64_t seq_len, int64_t token_num,
                                       int64_t head_num, int64_t kv_head_num, int64_t head_size,
                                       int32_t rotary_embedding_dim, float rotary_embedding_base,
                                       int32_t max_position_embeddings, int32_t use_dynamic_ntk,
                                       ispore_stream_t stream) {
    (void)input_length;
    (void)max_position_embeddings;
    (void)use_dynamic_ntk;
    return ispore::qkv_dispatch<float>(q_buf, k_buf, v_buf, QKV, bias, padding_offset, history_length,
                                       batch_size, seq_len, token_num, head_num, kv_head_num, head_size,
                                       rotary_embedding_dim, rotary_embedding_base,
                                       static_cast<cudaStream_t>(stream));
}

int ispore_qkv_bias_rope_transpose_f16(void* q_buf, void* k_buf, void* v_buf, const void* QKV,
                                       const void* bias, const int32_t* padding_offset,
                                       const int32_t* history_length, const int32_t* input_length,
                                       int64_t batch_size, int64_t seq_len, int64_t token_num,
                                       int64_t head_num, int64_t kv_head_num, int64_t head_size,
                                       int32_t rotary_embedding_dim, float rotary_embedding_base,
                                       int32_t max_position_embeddings, int32_t use_dynamic_ntk,
                                       ispore_stream_t stream) {
    (void)input_length;
    (void)max_position_embeddings;
    (void)use_dynamic_ntk;
    return ispore::qkv_dispatch<__half>(
        static_cast<__half*>(q_buf), static_cast<__half*>(k_buf), static_cast<__half*>(v_buf),
        static_cast<const __half*>(QKV), static_cast<const __half*>(bias), padding_offset,
        history_length, batch_size, seq_len, token_num, head_num, kv_head_num, head_size,
        rotary_embedding_dim, rotary_embedding_base, static_cast<cudaStream_t>(stream));
}

int ispore_rope_decode_f32(float* qkv_buf, int64_t batch_size, int64_t head_num, int64_t kv_head_num,
                           int64_t head_size, int32_t step, int32_t rotary_embedding_dim,
                           float rotary_embedding_base, ispore_stream_t stream) {
    return ispore::rope_decode_dispatch<float>(qkv_buf, batch_size, head_num, kv_head_num, head_size,
                                               step, rotary_embedding_dim, rotary_embedding_base,
                                               static_cast<cudaStream_t>(stream));
}

int ispore_rope_decode_f16(void* qkv_buf, int64_t batch_size, int64_t head_num, int64_t kv_head_num,
                           int64_t head_size, int32_t step, int32_t rotary_embedding_dim,
                           float rotary_embedding_base, ispore_stream_t stream) {
    return ispore::rope_decode_dispatch<__half>(static_cast<__half*>(qkv_buf), batch_size, head_num,
                                                kv_head_num, head_size, step, rotary_embedding_dim,
                                                rotary_embedding_base,
                                                static_cast<cudaStream_t>(stream));
}

}  // extern "C"
