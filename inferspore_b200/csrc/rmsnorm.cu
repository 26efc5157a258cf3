// Residual add (+bias) + RMSNorm and plain RMSNorm for sm_100a.
//
// Semantics follow the reference's fp32 kernel
// (src/kernels/fused_addresidual_norm.cu:33-98): s = x + r; r = s; s += bias;
// x = (gamma * s) * rsqrt(mean(s^2) + eps).  The reference walks the row three
// times in global memory; here one CTA owns a row, every thread keeps its slice
// of the row in registers between the reduction and the scaled store, so x and
// r each cross HBM once in and once out.  gamma is loaded once per CTA and
// reused over all rows the CTA visits (grid-stride over rows, grid sized in
// multiples of the SM count).
#include "common.cuh"

namespace ispore {
namespace {

enum class ResidualMode : int {
    kNone = 0,      // plain RMSNorm
    kAdd = 1,       // s = x + r, r = s             (fused add-residual norm)
    kCopyOut = 2    // r = x (un-normed copy), no add (plain norm that feeds the next add)
};

// Row held in registers: VPT 128-bit vectors per thread, THREADS threads per row.
template <typename T, int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_row_in_regs_kernel(T* __restrict__ x, T* __restrict__ r, const T* __restrict__ bias,
                           const T* __restrict__ gamma, float eps, int64_t num_tokens,
                           int hidden_vecs, int hidden, int mode_i) {
    constexpr int kWarps = THREADS / 32;
    const ResidualMode mode = static_cast<ResidualMode>(mode_i);
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    __shared__ float partial[2][kWarps];

    // gamma slice of this thread, kept for every row.
    uint4 g_raw[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * THREADS;
        g_raw[i] = (v < hidden_vecs) ? ld_keep(reinterpret_cast<const uint4*>(gamma) + v)
                                     : make_uint4(0, 0, 0, 0);
    }

    int parity = 0;
    for (int64_t row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        uint4* xrow = reinterpret_cast<uint4*>(x) + row * hidden_vecs;
        uint4* rrow = reinterpret_cast<uint4*>(r) + row * hidden_vecs;

        uint4 x_raw[VPT], r_raw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * THREADS;
            if (v < hidden_vecs) {
                x_raw[i] = ld_stream(xrow + v);
                if (mode == ResidualMode::kAdd) r_raw[i] = ld_stream(rrow + v);
            }
        }

        Unpacked<T> s[VPT];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * THREADS;
            if (v < hidden_vecs) {
                unpack(x_raw[i], s[i]);
                if (mode == ResidualMode::kAdd) {
                    Unpacked<T> rr;
                    unpack(r_raw[i], rr);
#pragma unroll
                    for (int e = 0; e < VecTraits<T>::kElems; ++e) s[i].v[e] += rr.v[e];
                    round_to_storage(s[i]);
                    st_stream(rrow + v, pack(s[i]));
                } else if (mode == ResidualMode::kCopyOut) {
                    st_stream(rrow + v, x_raw[i]);
                }
                if (bias != nullptr) {
                    Unpacked<T> bb;
                    unpack(ld_keep(reinterpret_cast<const uint4*>(bias) + v), bb);
#pragma unroll
                    for (int e = 0; e < VecTraits<T>::kElems; ++e) s[i].v[e] += bb.v[e];
                    round_to_storage(s[i]);
                }
#pragma unroll
                for (int e = 0; e < VecTraits<T>::kElems; ++e) acc = fmaf(s[i].v[e], s[i].v[e], acc);
            }
        }

        acc = warp_sum(acc);
        if (lane == 0) partial[parity][warp] = acc;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) total += partial[parity][w];
        const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);

#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * THREADS;
            if (v < hidden_vecs) {
                Unpacked<T> g;
                unpack(g_raw[i], g);
#pragma unroll
                for (int e = 0; e < VecTraits<T>::kElems; ++e) s[i].v[e] = (g.v[e] * s[i].v[e]) * inv;
                st_stream(xrow + v, pack(s[i]));
            }
        }
    }
}

// Any hidden size / any alignment: scalar accesses, the row is re-read from
// global memory (L2-resident) for the scaling pass.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_generic_kernel(T* __restrict__ x, T* __restrict__ r, const T* __restrict__ bias,
                       const T* __restrict__ gamma, float eps, int64_t num_tokens, int64_t hidden,
                       int mode_i) {
    constexpr int kWarps = THREADS / 32;
    const ResidualMode mode = static_cast<ResidualMode>(mode_i);
    const int tid = threadIdx.x;
    __shared__ float partial[2][kWarps];
    int parity = 0;
    for (int64_t row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        T* xrow = x + row * hidden;
        T* rrow = r + row * hidden;
        float acc = 0.f;
        for (int64_t i = tid; i < hidden; i += THREADS) {
            float s = to_float<T>(xrow[i]);
            if (mode == ResidualMode::kAdd) {
                s = to_float<T>(from_float<T>(s + to_float<T>(rrow[i])));
                rrow[i] = from_float<T>(s);
            } else if (mode == ResidualMode::kCopyOut) {
                rrow[i] = xrow[i];
            }
            if (bias != nullptr) s = to_float<T>(from_float<T>(s + to_float<T>(bias[i])));
            // Park the pre-norm value in x so the second pass needs no recompute.
            xrow[i] = from_float<T>(s);
            acc = fmaf(s, s, acc);
        }
        acc = warp_sum(acc);
        if ((tid & 31) == 0) partial[parity][tid >> 5] = acc;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) total += partial[parity][w];
        const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
        for (int64_t i = tid; i < hidden; i += THREADS) {
            const float s = to_float<T>(xrow[i]);
            xrow[i] = from_float<T>((to_float<T>(gamma[i]) * s) * inv);
        }
    }
}

template <typename T, int VPT, int THREADS>
int launch_regs(T* x, T* r, const T* bias, const T* gamma, float eps, int64_t tokens, int64_t hidden,
                ResidualMode mode, cudaStream_t st) {
    const int hidden_vecs = static_cast<int>(hidden / VecTraits<T>::kElems);
    // Enough CTAs to fill every SM to its thread limit; rows beyond that are
    // reached by the grid-stride loop so gamma is fetched once per CTA.
    const int64_t max_ctas = static_cast<int64_t>(kNumSMs) * (2048 / THREADS);
    const int grid = static_cast<int>(tokens < max_ctas ? tokens : max_ctas);
    rmsnorm_row_in_regs_kernel<T, VPT, THREADS><<<grid, THREADS, 0, st>>>(
        x, r, bias, gamma, eps, tokens, hidden_vecs, static_cast<int>(hidden),
        static_cast<int>(mode));
    return check_launch("rmsnorm_row_in_regs_kernel");
}

template <typename T>
int rmsnorm_dispatch(T* x, T* r, const T* bias, const T* gamma, float eps, int64_t tokens,
                     int64_t hidden, ResidualMode mode, cudaStream_t st) {
    if (tokens < 0 || hidden <= 0) return fail(ISPORE_ESHAPE, "rmsnorm: bad shape [%lld, %lld]",
                                               (long long)tokens, (long long)hidden);
    if (hidden > INT32_MAX) return fail(ISPORE_ELIMIT, "rmsnorm: hidden %lld too large", (long long)hidden);
    if (tokens == 0) return ISPORE_OK;  // an empty tensor may legitimately carry a NULL pointer
    if (x == nullptr || gamma == nullptr) return fail(ISPORE_ENULL, "rmsnorm: decoder_out/gamma is NULL");
    if (mode != ResidualMode::kNone && r == nullptr) mode = ResidualMode::kNone;

    constexpr int E = VecTraits<T>::kElems;
    const bool vec_ok = (hidden % E == 0) && aligned16(x) && aligned16(gamma) &&
                        (mode == ResidualMode::kNone || aligned16(r)) &&
                        (bias == nullptr || aligned16(bias));
    const int64_t vecs = hidden / E;
    if (vec_ok && vecs <= 128) return launch_regs<T, 1, 128>(x, r, bias, gamma, eps, tokens, hidden, mode, st);
    if (vec_ok && vecs <= 256) return launch_regs<T, 1, 256>(x, r, bias, gamma, eps, tokens, hidden, mode, st);
    if (vec_ok && vecs <= 512) return launch_regs<T, 2, 256>(x, r, bias, gamma, eps, tokens, hidden, mode, st);
    if (vec_ok && vecs <= 1024) return launch_regs<T, 4, 256>(x, r, bias, gamma, eps, tokens, hidden, mode, st);
    if (vec_ok && vecs <= 2048) return launch_regs<T, 4, 512>(x, r, bias, gamma, eps, tokens, hidden, mode, st);

    constexpr int THREADS = 256;
    const int64_t max_ctas = static_cast<int64_t>(kNumSMs) * 8;
    const int grid = static_cast<int>(tokens < max_ctas ? tokens : max_ctas);
    rmsnorm_generic_kernel<T, THREADS><<<grid, THREADS, 0, st>>>(x, r, bias, gamma, eps, tokens, hidden,
                                                                static_cast<int>(mode));
    return check_launch("rmsnorm_generic_kernel");
}

}  // namespace
}  // namespace ispore

using ispore::ResidualMode;

extern "C" {

int ispore_add_residual_rmsnorm_f32(float* decoder_out, float* residual, const float* bias,
                                    const float* gamma, float eps, int64_t num_tokens,
                                    int64_t hidden, ispore_stream_t stream) {
    return ispore::rmsnorm_dispatch<float>(decoder_out, residual, bias, gamma, eps, num_tokens, hidden,
                                           residual ? ResidualMode::kAdd : ResidualMode::kNone,
                                           static_cast<cudaStream_t>(stream));
}

int ispore_add_residual_rmsnorm_f16(void* decoder_out, void* residual, const void* bias,
                                    const void* gamma, float eps, int64_t num_tokens,
                                    int64_t hidden, ispore_stream_t stream) {
    return ispore::rmsnorm_dispatch<__half>(
        static_cast<__half*>(decoder_out), static_cast<__half*>(residual),
        static_cast<const __half*>(bias), static_cast<const __half*>(gamma), eps, num_tokens, hidden,
        residual ? ResidualMode::kAdd : ResidualMode::kNone, static_cast<cudaStream_t>(stream));
}

int ispore_rmsnorm_f32(float* decoder_out, float* residual_copy, const float* gamma, float eps,
                       int64_t num_tokens, int64_t hidden, ispore_stream_t stream) {
    return ispore::rmsnorm_dispatch<float>(decoder_out, residual_copy, nullptr, gamma, eps, num_tokens,
                                           hidden,
                                           residual_copy ? ResidualMode::kCopyOut : ResidualMode::kNone,
                                           static_cast<cudaStream_t>(stream));
}

int ispore_rmsnorm_f16(void* decoder_out, void* residual_copy, const void* gamma, float eps,
                       int64_t num_tokens, int64_t hidden, ispore_stream_t stream) {
    return ispore::rmsnorm_dispatch<__half>(
        static_cast<__half*>(decoder_out), static_cast<__half*>(residual_copy), nullptr,
        static_cast<const __half*>(gamma), eps, num_tokens, hidden,
        residual_copy ? ResidualMode::kCopyOut : ResidualMode::kNone,
        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
