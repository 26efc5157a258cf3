// Scale + additive mask + row softmax for sm_100a.
//
// Semantics: the reference's fp32 kernel, src/kernels/attn_softmax_kernel.cu:50-125:
//   z = scale*qk + (1 - mask)*(-10000);  m = max(FLT_MIN, max_k z)
//   e = exp(z - m);  out = e * (1 / (sum e + 1e-6))
// (the reference's block max starts from FLT_MIN and its idle warps feed 0 into
// the reduction, so m never drops below FLT_MIN; a fully masked row therefore
// comes out as exact zeros).  Both storage types compute in fp32.
//
// A row lives in registers between the max, the sum and the store, so qk is
// read once and the score written once.  Short rows (prefill: k_len of a few
// hundred) take one warp per row with shuffle-only reductions; long rows
// (decode against a 4096-deep cache) take one CTA per row.  The mask row is
// shared by all heads and stays in L2.
#include <float.h>

#include "common.cuh"

namespace ispore {
namespace {

// exp(z - m) for the two storage types: fp32 keeps the accurate expf the
// reference calls; fp16 uses ex2.approx on a log2e-prescaled argument (relative
// error ~2^-22, far below half precision) because at 8 elements per vector the
// accurate sequence would make a 2 GB prefill softmax issue-bound.
template <typename T>
struct ExpPolicy;
template <>
struct ExpPolicy<float> {
    static constexpr float kPrescale = 1.0f;
    static __device__ __forceinline__ float exp_diff(float z, float m) { return expf(z - m); }
};
template <>
struct ExpPolicy<__half> {
    static constexpr float kPrescale = 1.4426950408889634f;  // log2(e): z and m carry it
    static __device__ __forceinline__ float exp_diff(float z, float m) { return fast_exp2(z - m); }
};

// GROUP threads cooperate on one row; a CTA of THREADS threads holds
// THREADS/GROUP rows.  Each thread keeps VPT 128-bit vectors of its row.
template <typename T, int VPT, int GROUP, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_row_in_regs_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                           int64_t total_rows, int64_t rows_per_batch /* heads*q_len */, int q_len,
                           int row_vecs, float scale) {
    constexpr int E = VecTraits<T>::kElems;
    constexpr int kRowsPerCta = THREADS / GROUP;
    constexpr int kWarpsPerGroup = GROUP / 32;
    using Exp = ExpPolicy<T>;
    __shared__ float red[2][kRowsPerCta][kWarpsPerGroup > 1 ? kWarpsPerGroup : 1];

    const int tid = threadIdx.x;
    const int g = tid / GROUP;    // row slot inside the CTA
    const int gt = tid % GROUP;   // thread inside the row group
    const int lane = tid & 31;
    const int gw = gt >> 5;       // warp inside the row group
    const float a = scale * Exp::kPrescale;
    const float neg = -10000.0f * Exp::kPrescale;
    const float floor_m = FLT_MIN * Exp::kPrescale;

    // All row slots of a CTA run the same trip count (block-level barriers below).
    for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta; row0 < total_rows;
         row0 += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
        const int64_t row = row0 + g;
        const bool live = row < total_rows;
        const int64_t bidx = live ? row / rows_per_batch : 0;
        const int64_t qi = live ? (row - bidx * rows_per_batch) % q_len : 0;
        const uint4* qrow = reinterpret_cast<const uint4*>(qk) + row * row_vecs;
        const uint4* mrow = reinterpret_cast<const uint4*>(mask) + (bidx * q_len + qi) * row_vecs;
        uint4* orow = reinterpret_cast<uint4*>(score) + row * row_vecs;

        uint4 q_raw[VPT], m_raw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = gt + i * GROUP;
            if (live && v < row_vecs) {
                q_raw[i] = ld_stream(qrow + v);
                m_raw[i] = ld_keep(mrow + v);
            }
        }
        Unpacked<T> z[VPT];
        float mx = floor_m;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = gt + i * GROUP;
            if (live && v < row_vecs) {
                Unpacked<T> mk;
                unpack(q_raw[i], z[i]);
                unpack(m_raw[i], mk);
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    z[i].v[e] = fmaf(a, z[i].v[e], (1.0f - mk.v[e]) * neg);
                    mx = fmaxf(mx, z[i].v[e]);
                }
            }
        }
        mx = warp_max(mx);
        if (kWarpsPerGroup > 1) {
            if (lane == 0) red[0][g][gw] = mx;
            __syncthreads();
#pragma unroll
            for (int w = 0; w < kWarpsPerGroup; ++w) mx = fmaxf(mx, red[0][g][w]);
        }
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = gt + i * GROUP;
            if (live && v < row_vecs) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    z[i].v[e] = Exp::exp_diff(z[i].v[e], mx);
                    sum += z[i].v[e];
                }
            }
        }
        sum = warp_sum(sum);
        if (kWarpsPerGroup > 1) {
            if (lane == 0) red[1][g][gw] = sum;
            __syncthreads();
            sum = 0.f;
#pragma unroll
            for (int w = 0; w < kWarpsPerGroup; ++w) sum += red[1][g][w];
        }
        const float inv = 1.0f / (sum + 1e-6f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = gt + i * GROUP;
            if (live && v < row_vecs) {
#pragma unroll
                for (int e = 0; e < E; ++e) z[i].v[e] *= inv;
                st_stream(orow + v, pack(z[i]));
            }
        }
    }
}

// Any k_len / alignment: one CTA per row, three scalar passes (the row is
// re-read from L2).  Also the path for rows too long for the register kernels.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_generic_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                       int64_t total_rows, int64_t rows_per_batch, int q_len, int64_t k_len,
                       float scale) {
    constexpr int kWarps = THREADS / 32;
    __shared__ float red[2][kWarps];
    const int tid = threadIdx.x;
    for (int64_t row = blockIdx.x; row < total_rows; row += gridDim.x) {
        const int64_t bidx = row / rows_per_batch;
        const int64_t qi = (row - bidx * rows_per_batch) % q_len;
        const T* qrow = qk + row * k_len;
        const T* mrow = mask + (bidx * q_len + qi) * k_len;
        T* orow = score + row * k_len;
        float mx = FLT_MIN;
        for (int64_t i = tid; i < k_len; i += THREADS)
            mx = fmaxf(mx, fmaf(scale, to_float<T>(qrow[i]), (1.0f - to_float<T>(mrow[i])) * -10000.0f));
        mx = warp_max(mx);
        if ((tid & 31) == 0) red[0][tid >> 5] = mx;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, red[0][w]);
        float sum = 0.f;
        for (int64_t i = tid; i < k_len; i += THREADS)
            sum += expf(fmaf(scale, to_float<T>(qrow[i]), (1.0f - to_float<T>(mrow[i])) * -10000.0f) - mx);
        sum = warp_sum(sum);
        if ((tid & 31) == 0) red[1][tid >> 5] = sum;
        __syncthreads();
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red[1][w];
        const float inv = 1.0f / (sum + 1e-6f);
        for (int64_t i = tid; i < k_len; i += THREADS) {
            const float e =
                expf(fmaf(scale, to_float<T>(qrow[i]), (1.0f - to_float<T>(mrow[i])) * -10000.0f) - mx);
            orow[i] = from_float<T>(e * inv);
        }
        __syncthreads();
    }
}

template <typename T, int VPT, int GROUP, int THREADS>
int launch_regs(T* score, const T* qk, const T* mask, int64_t total_rows, int64_t rows_per_batch,
                int q_len, int row_vecs, float scale, cudaStream_t st) {
    constexpr int kRowsPerCta = THREADS / GROUP;
    const int64_t ctas = ceil_div(total_rows, kRowsPerCta);
    const int64_t max_ctas = static_cast<int64_t>(kNumSMs) * (2048 / THREADS) * 4;
    softmax_row_in_regs_kernel<T, VPT, GROUP, THREADS>
        <<<static_cast<int>(ctas < max_ctas ? ctas : max_ctas), THREADS, 0, st>>>(
            score, qk, mask, total_rows, rows_per_batch, q_len, row_vecs, scale);
    return check_launch("softmax_row_in_regs_kernel");
}

template <typename T>
int softmax_dispatch(T* score, const T* qk, const T* mask, int64_t batch, int64_t heads, int64_t q_len,
                     int64_t k_len, float scale, cudaStream_t st) {
    if (batch < 0 || heads <= 0 || q_len <= 0 || k_len <= 0 || q_len > INT32_MAX)
        return fail(ISPORE_ESHAPE, "scale_mask_softmax: bad shape [%lld,%lld,%lld,%lld]",
                    (long long)batch, (long long)heads, (long long)q_len, (long long)k_len);
    if (batch == 0) return ISPORE_OK;
    if (!score || !qk || !mask) return fail(ISPORE_ENULL, "scale_mask_softmax: NULL buffer");
    const int64_t total_rows = batch * heads * q_len;
    const int64_t rows_per_batch = heads * q_len;
    constexpr int E = VecTraits<T>::kElems;
    const bool vec_ok = k_len % E == 0 && aligned16(score) && aligned16(qk) && aligned16(mask);
    const int64_t vecs = k_len / E;
    const int q = static_cast<int>(q_len);
    if (vec_ok) {
        const int rv = static_cast<int>(vecs);
        if (vecs <= 32) return launch_regs<T, 1, 32, 256>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
        if (vecs <= 64) return launch_regs<T, 2, 32, 256>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
        if (vecs <= 128) return launch_regs<T, 4, 32, 256>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
        if (vecs <= 256) return launch_regs<T, 1, 256, 256>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
        if (vecs <= 512) return launch_regs<T, 2, 256, 256>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
        if (vecs <= 1024) return launch_regs<T, 4, 256, 256>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
        if (vecs <= 2048) return launch_regs<T, 4, 512, 512>(score, qk, mask, total_rows, rows_per_batch, q, rv, scale, st);
    }
    const int64_t max_ctas = static_cast<int64_t>(kNumSMs) * 8;
    softmax_generic_kernel<T, 256><<<static_cast<int>(total_rows < max_ctas ? total_rows : max_ctas), 256, 0, st>>>(
        score, qk, mask, total_rows, rows_per_batch, q, k_len, scale);
    return check_launch("softmax_generic_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {
int ispore_scale_mask_softmax_f32(float* attn_score, const float* qk, const float* mask,
                                  int64_t batch_size, int64_t head_num, int64_t q_len, int64_t k_len,
                                  float scale, ispore_stream_t stream) {
    return ispore::softmax_dispatch<float>(attn_score, qk, mask, batch_size, head_num, q_len, k_len,
                                           scale, static_cast<cudaStream_t>(stream));
}
int ispore_scale_mask_softmax_f16(void* attn_score, const void* qk, const void* mask,
                                  int64_t batch_size, int64_t head_num, int64_t q_len, int64_t k_len,
                                  float scale, ispore_stream_t stream) {
    return ispore::softmax_dispatch<__half>(static_cast<__half*>(attn_score),
                                            static_cast<const __half*>(qk),
                                            static_cast<const __half*>(mask), batch_size, head_num,
                                            q_len, k_len, scale, static_cast<cudaStream_t>(stream));
}
}
