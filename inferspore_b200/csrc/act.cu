// SiLU(gate) * up for sm_100a.
//
// Semantics: src/kernels/act_kernel.cu:6-34 of the reference —
// out[r,i] = (g / (1 + expf(-g))) * u with g = input[r,0,i], u = input[r,1,i],
// evaluated in fp32 and rounded once to the storage type (the reference's CPU
// function, tests/unittests/test_act.cu:13-25, rounds the same way).
//
// Pure streaming op: 2 reads + 1 write per element.  Each thread owns UNROLL
// independent 128-bit (gate, up) pairs per trip so that 2*UNROLL loads are in
// flight per thread before the first use.
#include "common.cuh"

namespace ispore {
namespace {

// fp32 storage: the accurate expf and an IEEE divide, as the reference writes
// them.  fp16 storage: ex2.approx / rcp.approx — their ~1e-6 relative error is
// three orders below half precision, and at 8 elements per 128-bit vector the
// accurate sequence would make the kernel issue-bound rather than HBM-bound.
template <typename T>
__device__ __forceinline__ float silu_mul(float g, float u);
template <>
__device__ __forceinline__ float silu_mul<float>(float g, float u) {
    return (g / (1.0f + expf(-g))) * u;
}
template <>
__device__ __forceinline__ float silu_mul<__half>(float g, float u) {
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <typename T, typename Index, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ in, Index total_vecs,
                    uint32_t inter_vecs) {
    chain_begin();
    const uint4* in_v = reinterpret_cast<const uint4*>(in);
    uint4* out_v = reinterpret_cast<uint4*>(out);
    const Index tile = static_cast<Index>(THREADS) * UNROLL;
    for (Index base = static_cast<Index>(blockIdx.x) * tile; base < total_vecs;
         base += static_cast<Index>(gridDim.x) * tile) {
        uint4 g_raw[UNROLL], u_raw[UNROLL];
        Index idx[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            idx[k] = base + static_cast<Index>(k) * THREADS + threadIdx.x;
            if (idx[k] < total_vecs) {
                const Index row = idx[k] / inter_vecs;
                const Index col = idx[k] - row * inter_vecs;
                const Index g_at = (row * 2) * inter_vecs + col;
                g_raw[k] = ld_stream(in_v + g_at);
                u_raw[k] = ld_stream(in_v + g_at + inter_vecs);
            }
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            if (idx[k] < total_vecs) {
                Unpacked<T> g, u;
                unpack(g_raw[k], g);
                unpack(u_raw[k], u);
#pragma unroll
                for (int e = 0; e < VecTraits<T>::kElems; ++e) g.v[e] = silu_mul<T>(g.v[e], u.v[e]);
                st_stream(out_v + idx[k], pack(g));
            }
        }
    }
}

template <typename T>
__global__ void silu_mul_scalar_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows,
                                       int64_t inter) {
    const int64_t total = rows * inter;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = i / inter, col = i - row * inter;
        const float g = to_float<T>(in[row * 2 * inter + col]);
        const float u = to_float<T>(in[row * 2 * inter + inter + col]);
        out[i] = from_float<T>(silu_mul<T>(g, u));
    }
}

template <typename T>
int silu_dispatch(T* out, const T* in, int64_t rows, int64_t inter, cudaStream_t st) {
    if (rows < 0 || inter <= 0) return fail(ISPORE_ESHAPE, "silu_mul: bad shape [%lld,2,%lld]",
                                            (long long)rows, (long long)inter);
    if (rows == 0) return ISPORE_OK;
    if (out == nullptr || in == nullptr) return fail(ISPORE_ENULL, "silu_mul: NULL buffer");
    constexpr int E = VecTraits<T>::kElems;
    constexpr int THREADS = 256, UNROLL = 4;
    if (inter % E == 0 && aligned16(out) && aligned16(in) && inter / E <= UINT32_MAX) {
        const int64_t inter_vecs = inter / E;
        const int64_t total_vecs = rows * inter_vecs;
        const int64_t tiles = ceil_div(total_vecs, THREADS * UNROLL);
        // The input spans 2*total_vecs vectors, so 32-bit indexing needs that to fit.
        const int64_t worst_grid = static_cast<int64_t>(sm_count()) * 8 * 64;
        if (total_vecs * 2 + worst_grid * THREADS * UNROLL < (1ll << 32)) {
            auto kernel = silu_mul_vec_kernel<T, uint32_t, THREADS, UNROLL>;
            launch_chained(kernel, persistent_grid(kernel, THREADS, 0, tiles, tune(kTuneAct, 64)), THREADS, 0, st,
                           out, in, static_cast<uint32_t>(total_vecs), static_cast<uint32_t>(inter_vecs));
        } else {
            auto kernel = silu_mul_vec_kernel<T, uint64_t, THREADS, UNROLL>;
            launch_chained(kernel, persistent_grid(kernel, THREADS, 0, tiles, tune(kTuneAct, 64)), THREADS, 0, st,
                           out, in, static_cast<uint64_t>(total_vecs), static_cast<uint32_t>(inter_vecs));
        }
        return check_launch("silu_mul_vec_kernel");
    }
    const int64_t blocks = ceil_div(rows * inter, 256);
    silu_mul_scalar_kernel<T><<<persistent_grid(silu_mul_scalar_kernel<T>, 256, 0, blocks), 256, 0, st>>>(
        out, in, rows, inter);
    return check_launch("silu_mul_scalar_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {
int ispore_silu_mul_f32(float* out, const float* input, int64_t rows, int64_t inter,
                        ispore_stream_t stream) {
    return ispore::silu_dispatch<float>(out, input, rows, inter, static_cast<cudaStream_t>(stream));
}
int ispore_silu_mul_f16(void* out, const void* input, int64_t rows, int64_t inter,
                        ispore_stream_t stream) {
    return ispore::silu_dispatch<__half>(static_cast<__half*>(out), static_cast<const __half*>(input),
                                         rows, inter, static_cast<cudaStream_t>(stream));
}
}
