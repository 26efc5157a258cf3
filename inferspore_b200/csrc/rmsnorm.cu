// Residual add (+bias) + RMSNorm and plain RMSNorm for sm_100a.
//
// Semantics follow the reference's fp32 kernel
// (src/kernels/fused_addresidual_norm.cu:33-98): s = x + r; r = s; s += bias;
// x = (gamma * s) * rsqrt(mean(s^2) + eps).  The reference walks the row three
// times in global memory; here one CTA owns a row, every thread keeps its slice
// of the row in registers between the reduction and the scaled store, so x and
// r each cross HBM once in and once out.  One row per CTA and as many CTAs as
// rows (measured faster on B200 than a persistent grid-stride loop); gamma is
// 8 KB shared by every row and is re-read through L1 for the scaled store.
// Measured and not kept for few rows (8-64 rows of 4096, fewer CTAs than SMs):
// a row split over a four-CTA thread-block cluster with the partial sums of
// squares exchanged through distributed shared memory — 2.5-4.2 us per launch
// against 2.0-3.1 us for one CTA per row (CUDA-graph replay over inputs larger
// than L2); the two cluster barriers cost more than the shorter per-CTA copy saves.
#include <stdint.h>

#include "common.cuh"

namespace ispore {
namespace {

enum class ResidualMode : int {
    kNone = 0,      // plain RMSNorm
    kAdd = 1,       // s = x + r, r = s             (fused add-residual norm)
    kCopyOut = 2    // r = x (un-normed copy), no add (plain norm that feeds the next add)
};

// Row held in registers: VPT 128-bit vectors per thread, THREADS threads per row.
// Between the reduction and the scaled store a thread keeps its slice of the
// pre-norm row PACKED in the storage type (for fp16 that is exactly the rounded
// value the norm is defined on), which keeps the register count low enough for
// MIN_BLOCKS CTAs per SM; gamma is re-read through L1 (it is 8 KB and shared by
// every row) instead of occupying registers.
// MODE is the ResidualMode; FAST means the row is exactly VPT*THREADS vectors long and there is
// no bias, so no per-vector guard (each costs a branch) and no bias test remain in the loop.
// RT: the CTA size is the launch's (any multiple of 32 up to THREADS) instead of THREADS itself, so a
// row of VPT * blockDim.x vectors fits exactly (hidden sizes such as 5120, 2560, 6144) and runs the
// guard-free FAST code.
template <typename T, int VPT, int THREADS, int MIN_BLOCKS, int MODE, bool FAST, bool RT = false>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS)
rmsnorm_row_in_regs_kernel(T* __restrict__ x, T* __restrict__ r, const T* __restrict__ bias_arg,
                           const T* __restrict__ gamma, float eps, int64_t num_tokens,
                           int hidden_vecs_arg, int hidden) {
    chain_begin();
    constexpr int kWarps = THREADS / 32;
    constexpr int E = VecTraits<T>::kElems;
    constexpr ResidualMode mode = static_cast<ResidualMode>(MODE);
    const int nthreads = RT ? static_cast<int>(blockDim.x) : THREADS;
    const int hidden_vecs = FAST ? VPT * nthreads : hidden_vecs_arg;
    const T* bias = FAST ? nullptr : bias_arg;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    __shared__ float partial[2][kWarps];
    const uint4* gamma_v = reinterpret_cast<const uint4*>(gamma);
    const uint4* bias_v = reinterpret_cast<const uint4*>(bias);

    int parity = 0;
    for (int64_t row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        uint4* xrow = reinterpret_cast<uint4*>(x) + row * hidden_vecs;
        uint4* rrow = reinterpret_cast<uint4*>(r) + row * hidden_vecs;

        uint4 s_raw[VPT], r_raw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * nthreads;
            if (FAST || v < hidden_vecs) {
                s_raw[i] = ld_stream(xrow + v);
                if (mode == ResidualMode::kAdd) r_raw[i] = ld_stream(rrow + v);
            }
        }

        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * nthreads;
            if (FAST || v < hidden_vecs) {
                Unpacked<T> s;
                unpack(s_raw[i], s);
                if (mode == ResidualMode::kAdd) {
                    Unpacked<T> rr;
                    unpack(r_raw[i], rr);
#pragma unroll
                    for (int e = 0; e < E; ++e) s.v[e] += rr.v[e];
                    s_raw[i] = pack(s);  // rounds to the storage type: the new residual
                    st_stream(rrow + v, s_raw[i]);
                    unpack(s_raw[i], s);
                } else if (mode == ResidualMode::kCopyOut) {
                    st_stream(rrow + v, s_raw[i]);
                }
                if (bias != nullptr) {
                    Unpacked<T> bb;
                    unpack(ld_keep(bias_v + v), bb);
#pragma unroll
                    for (int e = 0; e < E; ++e) s.v[e] += bb.v[e];
                    s_raw[i] = pack(s);
                    unpack(s_raw[i], s);
                }
#pragma unroll
                for (int e = 0; e < E; ++e) acc = fmaf(s.v[e], s.v[e], acc);
            }
        }

        acc = warp_sum(acc);
        if (lane == 0) partial[parity][warp] = acc;
        __syncthreads();
        float total = 0.f;
        if (RT) {
            for (int w = 0; w < nthreads / 32; ++w) total += partial[parity][w];
        } else {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total += partial[parity][w];
        }
        const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);

#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * nthreads;
            if (FAST || v < hidden_vecs) {
                Unpacked<T> s, g;
                unpack(s_raw[i], s);
                unpack(ld_keep(gamma_v + v), g);
#pragma unroll
                for (int e = 0; e < E; ++e) s.v[e] = (g.v[e] * s.v[e]) * inv;
                st_stream(xrow + v, pack(s));
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

template <typename T, int VPT, int THREADS, int MIN_BLOCKS, int MODE, bool FAST>
int launch_regs_as(T* x, T* r, const T* bias, const T* gamma, float eps, int64_t tokens, int64_t hidden,
                   cudaStream_t st) {
    const int hidden_vecs = static_cast<int>(hidden / VecTraits<T>::kElems);
    auto kernel = rmsnorm_row_in_regs_kernel<T, VPT, THREADS, MIN_BLOCKS, MODE, FAST>;
    // One row per CTA and as many CTAs as rows: measured faster on B200 than a persistent loop.
    const int grid = static_cast<int>(tokens < (1ll << 30) ? tokens : (1ll << 30));
    launch_chained(kernel, grid, THREADS, 0, st, x, r, bias, gamma, eps, tokens, hidden_vecs, static_cast<int>(hidden));
    return check_launch("rmsnorm_row_in_regs_kernel");
}

template <typename T, int VPT, int MAXT, int MIN_BLOCKS, bool FAST>
int launch_rt_as(T* x, T* r, const T* bias, const T* gamma, float eps, int64_t tokens, int64_t hidden,
                 ResidualMode mode, int threads, cudaStream_t st) {
    const int hidden_vecs = static_cast<int>(hidden / VecTraits<T>::kElems);
    const int grid = static_cast<int>(tokens < (1ll << 30) ? tokens : (1ll << 30));
    switch (mode) {
        case ResidualMode::kAdd:
            launch_chained(rmsnorm_row_in_regs_kernel<T, VPT, MAXT, MIN_BLOCKS, 1, FAST, true>, grid, threads, 0, st,
                x, r, bias, gamma, eps, tokens, hidden_vecs, static_cast<int>(hidden));
            break;
        case ResidualMode::kCopyOut:
            launch_chained(rmsnorm_row_in_regs_kernel<T, VPT, MAXT, MIN_BLOCKS, 2, FAST, true>, grid, threads, 0, st,
                x, r, bias, gamma, eps, tokens, hidden_vecs, static_cast<int>(hidden));
            break;
        default:
            launch_chained(rmsnorm_row_in_regs_kernel<T, VPT, MAXT, MIN_BLOCKS, 0, FAST, true>, grid, threads, 0, st,
                x, r, bias, gamma, eps, tokens, hidden_vecs, static_cast<int>(hidden));
    }
    return check_launch("rmsnorm_row_in_regs_kernel");
}

// CTA of `threads` threads (a multiple of 32) holding VPT vectors each; `exact` when the row fills
// every slot and there is no bias (the guard-free code).
template <typename T, int VPT, int MAXT, int MIN_BLOCKS>
int launch_rt(T* x, T* r, const T* bias, const T* gamma, float eps, int64_t tokens, int64_t hidden, ResidualMode mode,
              int threads, bool exact, cudaStream_t st) {
    return exact ? launch_rt_as<T, VPT, MAXT, MIN_BLOCKS, true>(x, r, bias, gamma, eps, tokens, hidden, mode, threads, st)
                 : launch_rt_as<T, VPT, MAXT, MIN_BLOCKS, false>(x, r, bias, gamma, eps, tokens, hidden, mode, threads, st);
}

template <typename T, int VPT, int THREADS, int MIN_BLOCKS>
int launch_regs(T* x, T* r, const T* bias, const T* gamma, float eps, int64_t tokens, int64_t hidden,
                ResidualMode mode, cudaStream_t st) {
    const bool fast = bias == nullptr && hidden == static_cast<int64_t>(VPT) * THREADS * VecTraits<T>::kElems;
#define ISPORE_NORM_MODE(M)                                                                                  \
    return fast ? launch_regs_as<T, VPT, THREADS, MIN_BLOCKS, M, true>(x, r, bias, gamma, eps, tokens, hidden, st) \
                : launch_regs_as<T, VPT, THREADS, MIN_BLOCKS, M, false>(x, r, bias, gamma, eps, tokens, hidden, st)
    switch (mode) {
        case ResidualMode::kAdd: ISPORE_NORM_MODE(1);
        case ResidualMode::kCopyOut: ISPORE_NORM_MODE(2);
        default: ISPORE_NORM_MODE(0);
    }
#undef ISPORE_NORM_MODE
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
    // Launch shapes measured on B200 at hidden 4096 fp16 (512 vectors per row): with one
    // input stream (plain norm) 128-thread CTAs holding 4 vectors per thread run at copy
    // speed; with two input streams (x and the residual) 256-thread CTAs with 2 vectors
    // per thread, 4 CTAs per SM, do.  Wider rows scale the CTA, not the per-thread count.
    const bool one_stream = mode == ResidualMode::kNone;
#define ISPORE_NORM(VPT, THREADS, BLOCKS) \
    return launch_regs<T, VPT, THREADS, BLOCKS>(x, r, bias, gamma, eps, tokens, hidden, mode, st)
    // Rows that match none of the fixed shapes below exactly (5120, 2560, 6144, 7168, 4104 ... at
    // fp16): a CTA just large enough, ceil(vecs / VPT) threads rounded up to whole warps; when the row
    // fills every slot (and there is no bias) the guard-free code runs.
    const bool fixed_fit = vecs == 128 || vecs == 256 || vecs == 512 || vecs == 1024 || vecs == 2048 || vecs == 4096;
    if (vec_ok && !fixed_fit && vecs > 64 && vecs <= 4096) {
        const bool four_first = one_stream || vecs > 640;  // measured: two input streams like 2 vectors per thread up to 5120 halves
        const int prefer[3] = {four_first ? 4 : 2, four_first ? 2 : 4, 1};
        int best_vpt = 0;
        int64_t best_idle = INT64_MAX;
        for (int vpt : prefer) {  // the first preferred count that idles at most an eighth of its slots, else the fewest idle
            const int64_t threads = ceil_div(ceil_div(vecs, static_cast<int64_t>(vpt)), 32) * 32;
            if (threads > 1024) continue;
            const int64_t idle = threads * vpt - vecs;
            if (idle * 8 <= threads * vpt) {
                best_idle = idle;
                best_vpt = vpt;
                break;
            }
            if (idle < best_idle) {
                best_idle = idle;
                best_vpt = vpt;
            }
        }
        if (best_vpt != 0) {
            const int th = static_cast<int>(ceil_div(ceil_div(vecs, static_cast<int64_t>(best_vpt)), 32) * 32);
            const bool exact = best_idle == 0 && bias == nullptr;
#define ISPORE_NORM_RT(VPT, MAXT, BLOCKS) \
    return launch_rt<T, VPT, MAXT, BLOCKS>(x, r, bias, gamma, eps, tokens, hidden, mode, th, exact, st)
            if (best_vpt == 4) {
                if (th <= 256) ISPORE_NORM_RT(4, 256, 4);
                ISPORE_NORM_RT(4, 1024, 1);
            }
            if (best_vpt == 2) {
                if (th <= 512) ISPORE_NORM_RT(2, 512, 2);
                ISPORE_NORM_RT(2, 1024, 1);
            }
            if (th <= 512) ISPORE_NORM_RT(1, 512, 2);
            ISPORE_NORM_RT(1, 1024, 1);
#undef ISPORE_NORM_RT
        }
    }
    if (vec_ok && vecs <= 128) ISPORE_NORM(1, 128, 8);
    if (vec_ok && vecs <= 256) ISPORE_NORM(2, 128, 8);
    if (vec_ok && vecs <= 512) {
        switch (tune(kTuneRmsnorm, one_stream ? 0 : 5)) {
#ifdef ISPORE_TUNING
            case 1: ISPORE_NORM(2, 256, 6);
            case 2: ISPORE_NORM(2, 256, 8);
            case 3: ISPORE_NORM(4, 128, 10);
            case 4: ISPORE_NORM(1, 512, 4);
#endif
            case 5: ISPORE_NORM(2, 256, 4);
            default: ISPORE_NORM(4, 128, 8);
        }
    }
    if (vec_ok && vecs <= 1024) {
        if (one_stream) ISPORE_NORM(4, 256, 4);
        ISPORE_NORM(2, 512, 2);
    }
    if (vec_ok && vecs <= 2048) ISPORE_NORM(4, 512, 2);
    if (vec_ok && vecs <= 4096) ISPORE_NORM(4, 1024, 1);
#undef ISPORE_NORM

    constexpr int THREADS = 256;
    const int grid = persistent_grid(rmsnorm_generic_kernel<T, THREADS>, THREADS, 0, tokens);
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
