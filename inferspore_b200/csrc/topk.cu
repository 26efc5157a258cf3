// Top-K (+ sampling) for sm_100a.
//
// Interface: the reference's two-round block top-K (src/kernels/topK.cu:17-110):
// round 1 reduces each row slice to K candidates in caller-provided scratch
// [rows, slices, K], round 2 merges the slices.  The reference fixes K = 5 and
// keeps a per-thread insertion list merged through cub::BlockReduce, which
// costs O(K) per element and leaves the tie order to thread striding.  Here K
// is a run-time value up to ISPORE_TOPK_MAX_K and the order is total:
// (value descending, index ascending), -0.0 == +0.0.
//
// Round 1 (one CTA per row slice) reads its slice once from HBM into shared
// memory as order-preserving 32-bit keys.  A threshold that is guaranteed to
// keep at least K elements is derived from the per-thread maxima with
// warp ballots only; the few survivors are compacted and ranked by counting
// against each other, which yields the slice's top-K already sorted without a
// sorting network.  Adversarial inputs (e.g. a constant row, where the
// threshold keeps everything) fall back to an exact radix select over the keys
// in shared memory, ties resolved by an index-ordered block scan.
// Round 2 (one CTA per row) ranks the slices' candidates the same way and can
// draw the sampled token in its epilogue.
#include <float.h>
#include <math.h>

#include "common.cuh"

namespace ispore {
namespace {

constexpr int kTopkThreads = 256;
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kCandCap = 1024;        // survivors kept by the threshold path
constexpr int kMergeCap = 4096;       // lists*K candidates the merge kernel holds in smem
constexpr int kMaxSliceElems = 49152; // 192 KB of keys

__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t b = __float_as_uint(f);
    if (b == 0x80000000u) b = 0u;  // -0.0 ties with +0.0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// Larger composite = earlier in the output.  Composite 0 is reserved for "empty".
__device__ __forceinline__ unsigned long long composite(uint32_t key, uint32_t idx) {
    return (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(~idx);
}

template <typename T>
__device__ __forceinline__ T neg_inf();
template <>
__device__ __forceinline__ float neg_inf<float>() {
    return -INFINITY;
}
template <>
__device__ __forceinline__ __half neg_inf<__half>() {
    return __ushort_as_half(0xFC00u);
}

// q-th largest (1-based) of the 32 lane values, by ballots from the top bit down.
__device__ __forceinline__ uint32_t warp_qth_largest(uint32_t v, int q) {
    uint32_t cand = 0xffffffffu;  // lanes still tied with the prefix
    uint32_t prefix = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const uint32_t set = __ballot_sync(0xffffffffu, (v >> bit) & 1u) & cand;
        const int cnt = __popc(set);
        if (cnt >= q) {
            cand = set;
            prefix |= 1u << bit;
        } else {
            q -= cnt;
            cand &= ~set;
        }
    }
    return prefix;
}

// Ranks `count` distinct composites against each other and emits those with
// rank < K at slot `rank` of (out_ids, out_vals).  value_of(idx) returns the
// original stored value for element idx.
template <typename T, typename ValueOf>
__device__ __forceinline__ void rank_and_emit(const unsigned long long* cand, int count, int K,
                                              int32_t* out_ids, T* out_vals, int32_t index_offset,
                                              ValueOf value_of) {
    for (int c = threadIdx.x; c < count; c += kTopkThreads) {
        const unsigned long long mine = cand[c];
        int rank = 0;
        for (int j = 0; j < count; ++j) rank += cand[j] > mine;
        if (rank < K) {
            const uint32_t idx = ~static_cast<uint32_t>(mine);
            out_ids[rank] = static_cast<int32_t>(idx) + index_offset;
            out_vals[rank] = value_of(idx);
        }
    }
    for (int slot = count + threadIdx.x; slot < K; slot += kTopkThreads) {
        out_ids[slot] = -1;
        out_vals[slot] = neg_inf<T>();
    }
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
topk_slice_kernel(const T* __restrict__ probs, int64_t vocab, int slice_len, int slices, int K,
                  int32_t* __restrict__ scratch_ids, T* __restrict__ scratch_vals, int scratch_slices,
                  int32_t index_offset, int vec_loads) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw);  // [slice_len]
    __shared__ unsigned long long cand[kCandCap];
    __shared__ uint32_t warp_thr[kTopkWarps];
    __shared__ int s_count;
    __shared__ int hist[256];
    __shared__ int s_digit, s_need;
    __shared__ int warp_cnt[kTopkWarps];

    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x / slices;
    const int slice = static_cast<int>(blockIdx.x - row * slices);
    const int64_t begin = static_cast<int64_t>(slice) * slice_len;
    int64_t n64 = vocab - begin;
    if (n64 > slice_len) n64 = slice_len;
    const int n = n64 > 0 ? static_cast<int>(n64) : 0;
    const T* src = probs + row * vocab + begin;
    int32_t* out_ids = scratch_ids + (row * scratch_slices + slice) * K;
    T* out_vals = scratch_vals + (row * scratch_slices + slice) * K;

    if (tid == 0) s_count = 0;

    // 1. slice -> keys in shared memory, per-thread maximum on the way.
    uint32_t tmax = 0;
    if (vec_loads) {
        constexpr int E = VecTraits<T>::kElems;
        const int n_vecs = n / E;  // launcher guarantees n % E == 0 on this path
        const uint4* src_v = reinterpret_cast<const uint4*>(src);
#pragma unroll 4
        for (int v = tid; v < n_vecs; v += kTopkThreads) {
            Unpacked<T> x;
            unpack(ld_stream(src_v + v), x);
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const uint32_t k = order_key(x.v[e]);
                keys[v * E + e] = k;
                tmax = max(tmax, k);
            }
        }
    } else {
#pragma unroll 4
        for (int i = tid; i < n; i += kTopkThreads) {
            const uint32_t k = order_key(to_float<T>(src[i]));
            keys[i] = k;
            tmax = max(tmax, k);
        }
    }

    // 2. threshold: the ceil(K/warps)-th largest thread maximum of every warp,
    //    minimum over warps => at least K elements have key >= threshold.
    const int q = (K + kTopkWarps - 1) / kTopkWarps;
    const uint32_t wq = warp_qth_largest(tmax, q);
    if ((tid & 31) == 0) warp_thr[tid >> 5] = wq;
    __syncthreads();
    uint32_t thr = warp_thr[0];
#pragma unroll
    for (int w = 1; w < kTopkWarps; ++w) thr = min(thr, warp_thr[w]);

    // 3. compact the survivors.
    for (int i = tid; i < n; i += kTopkThreads) {
        const uint32_t k = keys[i];
        if (k >= thr) {
            const int pos = atomicAdd(&s_count, 1);
            if (pos < kCandCap) cand[pos] = composite(k, static_cast<uint32_t>(begin + i));
        }
    }
    __syncthreads();
    int count = s_count;

    if (count > kCandCap) {
        // 4'. exact radix select: the K-th largest key, 8 bits per pass.
        uint32_t prefix = 0, prefix_mask = 0;
        int need = K;  // K <= n here because count > kCandCap >= K
        for (int shift = 24; shift >= 0; shift -= 8) {
            hist[tid] = 0;  // kTopkThreads == 256 bins
            __syncthreads();
            for (int i = tid; i < n; i += kTopkThreads) {
                const uint32_t k = keys[i];
                if ((k & prefix_mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int cum = 0, d = 255;
                for (; d > 0; --d) {
                    if (cum + hist[d] >= need) break;
                    cum += hist[d];
                }
                s_digit = d;
                s_need = need - cum;
            }
            __syncthreads();
            prefix |= static_cast<uint32_t>(s_digit) << shift;
            prefix_mask |= 255u << shift;
            need = s_need;
            __syncthreads();
        }
        // keys > prefix: all of them (fewer than K); keys == prefix: the `need`
        // lowest indices, found by an index-ordered scan.
        if (tid == 0) s_count = 0;
        __syncthreads();
        for (int i = tid; i < n; i += kTopkThreads) {
            const uint32_t k = keys[i];
            if (k > prefix) cand[atomicAdd(&s_count, 1)] = composite(k, static_cast<uint32_t>(begin + i));
        }
        __syncthreads();
        const int greater = s_count;
        int taken = 0;
        for (int base = 0; base < n && taken < need; base += kTopkThreads) {
            const int i = base + tid;
            const bool tie = i < n && keys[i] == prefix;
            const uint32_t ballot = __ballot_sync(0xffffffffu, tie);
            if ((tid & 31) == 0) warp_cnt[tid >> 5] = __popc(ballot);
            __syncthreads();
            int before = 0, total = 0;
#pragma unroll
            for (int w = 0; w < kTopkWarps; ++w) {
                if (w < (tid >> 5)) before += warp_cnt[w];
                total += warp_cnt[w];
            }
            const int ordinal = taken + before + __popc(ballot & ((1u << (tid & 31)) - 1u));
            if (tie && ordinal < need)
                cand[greater + ordinal] = composite(prefix, static_cast<uint32_t>(begin + i));
            taken += total;
            __syncthreads();
        }
        count = K;
        __syncthreads();
    }

    // 5. rank the survivors against each other; rank < K are the slice's top-K.
    rank_and_emit<T>(cand, count, K, out_ids, out_vals, index_offset,
                     [&](uint32_t idx) { return src[static_cast<int64_t>(idx) - begin]; });
}

// exp((v - v0)/T) in index order, inverse CDF on a caller-drawn uniform.
// One warp: lanes evaluate the exponentials, lane 0 accumulates sequentially.
template <typename T>
__device__ __forceinline__ void sample_row(const int32_t* ids, const T* vals, int K, float u,
                                           float temperature, float* p_smem, int32_t* out) {
    const int lane = threadIdx.x & 31;
    const float v0 = to_float<T>(vals[0]);
    for (int i = lane; i < K; i += 32)
        p_smem[i] = ids[i] < 0 ? 0.f : expf((to_float<T>(vals[i]) - v0) / temperature);
    __syncwarp();
    if (lane == 0) {
        float total = 0.f;
        int last = -1;
        for (int i = 0; i < K; ++i) {
            if (ids[i] >= 0) {
                total += p_smem[i];
                last = i;
            }
        }
        const float target = u * total;
        float cum = 0.f;
        int pick = last;
        for (int i = 0; i < K; ++i) {
            if (ids[i] < 0) continue;
            cum += p_smem[i];
            if (cum >= target) {
                pick = i;
                break;
            }
        }
        *out = pick >= 0 ? ids[pick] : -1;
    }
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
topk_merge_kernel(const int32_t* __restrict__ cand_ids, const T* __restrict__ cand_vals, int lists,
                  int list_stride /* lists allocated per row */, int K, int32_t* __restrict__ final_ids,
                  T* __restrict__ final_vals, const float* __restrict__ uniform, float temperature,
                  int32_t* __restrict__ sampled_ids) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* comp = reinterpret_cast<unsigned long long*>(smem_raw);  // [lists*K]
    __shared__ int32_t fin_ids[ISPORE_TOPK_MAX_K];
    __shared__ T fin_vals[ISPORE_TOPK_MAX_K];
    __shared__ float p_smem[ISPORE_TOPK_MAX_K];

    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x;
    const int total = lists * K;
    const int32_t* ids = cand_ids + row * list_stride * K;
    const T* vals = cand_vals + row * list_stride * K;

    for (int c = tid; c < total; c += kTopkThreads) {
        const int32_t id = ids[c];
        comp[c] = id < 0 ? 0ull : composite(order_key(to_float<T>(vals[c])), static_cast<uint32_t>(id));
    }
    for (int s = tid; s < K; s += kTopkThreads) {
        fin_ids[s] = -1;
        fin_vals[s] = neg_inf<T>();
    }
    __syncthreads();
    for (int c = tid; c < total; c += kTopkThreads) {
        const unsigned long long mine = comp[c];
        if (mine == 0ull) continue;
        int rank = 0;
        for (int j = 0; j < total; ++j) rank += comp[j] > mine;
        if (rank < K) {
            fin_ids[rank] = ids[c];
            fin_vals[rank] = vals[c];
        }
    }
    __syncthreads();
    for (int s = tid; s < K; s += kTopkThreads) {
        final_ids[row * K + s] = fin_ids[s];
        final_vals[row * K + s] = fin_vals[s];
    }
    if (uniform != nullptr && tid < 32)
        sample_row<T>(fin_ids, fin_vals, K, uniform[row], temperature, p_smem, sampled_ids + row);
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
sampling_kernel(const int32_t* __restrict__ topk_ids, const T* __restrict__ topk_vals,
                const float* __restrict__ uniform, int32_t* __restrict__ output_ids, int64_t rows,
                int K, float temperature) {
    __shared__ float p_smem[kTopkWarps][ISPORE_TOPK_MAX_K];
    const int warp = threadIdx.x >> 5;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTopkWarps + warp;
    if (row >= rows) return;  // whole warps leave; no block barrier follows
    sample_row<T>(topk_ids + row * K, topk_vals + row * K, K, uniform[row], temperature, p_smem[warp],
                  output_ids + row);
}

int check_k(const char* who, int32_t K) {
    if (K < 1 || K > ISPORE_TOPK_MAX_K) return fail(ISPORE_ELIMIT, "%s: K=%d outside [1,%d]", who, K, ISPORE_TOPK_MAX_K);
    return ISPORE_OK;
}

template <typename T>
int merge_dispatch(const int32_t* cand_ids, const T* cand_vals, int64_t rows, int32_t lists,
                   int32_t list_stride, int32_t K, int32_t* final_ids, T* final_vals,
                   const float* uniform, float temperature, int32_t* sampled_ids, cudaStream_t st) {
    if (int rc = check_k("topk_merge", K)) return rc;
    if (rows < 0 || lists < 1 || rows > INT32_MAX) return fail(ISPORE_ESHAPE, "topk_merge: rows=%lld lists=%d", (long long)rows, lists);
    if (static_cast<int64_t>(lists) * K > kMergeCap)
        return fail(ISPORE_ELIMIT, "topk_merge: lists*K=%lld > %d", (long long)lists * K, kMergeCap);
    if (uniform != nullptr && !(temperature > 0.f)) return fail(ISPORE_ESHAPE, "topk_merge: temperature must be > 0");
    if (rows == 0) return ISPORE_OK;
    if (!cand_ids || !cand_vals || !final_ids || !final_vals) return fail(ISPORE_ENULL, "topk_merge: NULL buffer");
    if (uniform != nullptr && sampled_ids == nullptr) return fail(ISPORE_ENULL, "topk_merge: uniform given without sampled_ids");
    const size_t smem = static_cast<size_t>(lists) * K * sizeof(unsigned long long);
    topk_merge_kernel<T><<<static_cast<int>(rows), kTopkThreads, smem, st>>>(
        cand_ids, cand_vals, lists, list_stride, K, final_ids, final_vals, uniform, temperature, sampled_ids);
    return check_launch("topk_merge_kernel");
}

template <typename T>
int topk_dispatch(const T* probs, int64_t rows, int64_t vocab, int32_t K, int32_t* scratch_ids,
                  T* scratch_vals, int32_t scratch_slices, int32_t* final_ids, T* final_vals,
                  int32_t index_offset, const float* uniform, float temperature, int32_t* sampled_ids,
                  cudaStream_t st) {
    if (int rc = check_k("topk", K)) return rc;
    if (rows < 0 || vocab <= 0 || vocab > INT32_MAX || index_offset < 0 ||
        static_cast<int64_t>(index_offset) + vocab > INT32_MAX)
        return fail(ISPORE_ESHAPE, "topk: bad shape rows=%lld vocab=%lld offset=%d", (long long)rows,
                    (long long)vocab, index_offset);
    if (rows == 0) return ISPORE_OK;
    if (!probs || !final_ids || !final_vals) return fail(ISPORE_ENULL, "topk: NULL buffer");
    if (!scratch_ids || !scratch_vals || scratch_slices < 1)
        return fail(ISPORE_ESCRATCH, "topk: scratch [rows, slices>=1, K] is required");

    constexpr int E = VecTraits<T>::kElems;
    // Slices of ~4K elements keep every SM busy at a few hundred rows; never more
    // than the scratch the caller gave, nor than the merge kernel can hold.
    int64_t slices = ceil_div(vocab, 4096);
    if (slices > scratch_slices) slices = scratch_slices;
    if (slices * K > kMergeCap) slices = kMergeCap / K;
    int64_t slice_len = ceil_div(vocab, slices);
    slice_len = ceil_div(slice_len, E) * E;
    if (slice_len > kMaxSliceElems)
        return fail(ISPORE_ESCRATCH, "topk: vocab %lld needs more than %d scratch slices", (long long)vocab,
                    scratch_slices);
    slices = ceil_div(vocab, slice_len);
    if (rows * slices > INT32_MAX) return fail(ISPORE_ELIMIT, "topk: rows*slices too large");
    const int vec_loads = (vocab % E == 0) && aligned16(probs);

    const size_t smem = static_cast<size_t>(slice_len) * sizeof(uint32_t);
    static_assert(kTopkThreads == 256, "radix pass uses one thread per bin");
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(topk_slice_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kMaxSliceElems * (int)sizeof(uint32_t));
        if (e != cudaSuccess) return fail(ISPORE_ELAUNCH, "topk: cannot raise dynamic smem: %s", cudaGetErrorString(e));
    }
    topk_slice_kernel<T><<<static_cast<int>(rows * slices), kTopkThreads, smem, st>>>(
        probs, vocab, static_cast<int>(slice_len), static_cast<int>(slices), K, scratch_ids, scratch_vals,
        scratch_slices, index_offset, vec_loads);
    if (int rc = check_launch("topk_slice_kernel")) return rc;
    return merge_dispatch<T>(scratch_ids, scratch_vals, rows, static_cast<int32_t>(slices), scratch_slices, K,
                             final_ids, final_vals, uniform, temperature, sampled_ids, st);
}

template <typename T>
int sampling_dispatch(const int32_t* ids, const T* vals, const float* uniform, int32_t* out, int64_t rows,
                      int32_t K, float temperature, cudaStream_t st) {
    if (int rc = check_k("sampling", K)) return rc;
    if (rows < 0) return fail(ISPORE_ESHAPE, "sampling: rows=%lld", (long long)rows);
    if (!(temperature > 0.f)) return fail(ISPORE_ESHAPE, "sampling: temperature must be > 0");
    if (rows == 0) return ISPORE_OK;
    if (!ids || !vals || !uniform || !out) return fail(ISPORE_ENULL, "sampling: NULL buffer");
    sampling_kernel<T><<<static_cast<int>(ceil_div(rows, kTopkWarps)), kTopkThreads, 0, st>>>(
        ids, vals, uniform, out, rows, K, temperature);
    return check_launch("sampling_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {

int ispore_topk_f32(const float* probs, int64_t rows, int64_t vocab, int32_t K, int32_t* scratch_ids,
                    float* scratch_vals, int32_t scratch_slices, int32_t* final_ids, float* final_vals,
                    int32_t index_offset, const float* uniform, float temperature,
                    int32_t* sampled_ids, ispore_stream_t stream) {
    return ispore::topk_dispatch<float>(probs, rows, vocab, K, scratch_ids, scratch_vals, scratch_slices,
                                        final_ids, final_vals, index_offset, uniform, temperature,
                                        sampled_ids, static_cast<cudaStream_t>(stream));
}
int ispore_topk_f16(const void* probs, int64_t rows, int64_t vocab, int32_t K, int32_t* scratch_ids,
                    void* scratch_vals, int32_t scratch_slices, int32_t* final_ids, void* final_vals,
                    int32_t index_offset, const float* uniform, float temperature,
                    int32_t* sampled_ids, ispore_stream_t stream) {
    return ispore::topk_dispatch<__half>(static_cast<const __half*>(probs), rows, vocab, K, scratch_ids,
                                         static_cast<__half*>(scratch_vals), scratch_slices, final_ids,
                                         static_cast<__half*>(final_vals), index_offset, uniform,
                                         temperature, sampled_ids, static_cast<cudaStream_t>(stream));
}
int ispore_topk_merge_f32(const int32_t* cand_ids, const float* cand_vals, int64_t rows, int32_t lists,
                          int32_t K, int32_t* final_ids, float* final_vals, const float* uniform,
                          float temperature, int32_t* sampled_ids, ispore_stream_t stream) {
    return ispore::merge_dispatch<float>(cand_ids, cand_vals, rows, lists, lists, K, final_ids, final_vals,
                                         uniform, temperature, sampled_ids,
                                         static_cast<cudaStream_t>(stream));
}
int ispore_topk_merge_f16(const int32_t* cand_ids, const void* cand_vals, int64_t rows, int32_t lists,
                          int32_t K, int32_t* final_ids, void* final_vals, const float* uniform,
                          float temperature, int32_t* sampled_ids, ispore_stream_t stream) {
    return ispore::merge_dispatch<__half>(cand_ids, static_cast<const __half*>(cand_vals), rows, lists, lists,
                                          K, final_ids, static_cast<__half*>(final_vals), uniform,
                                          temperature, sampled_ids, static_cast<cudaStream_t>(stream));
}
int ispore_sampling_f32(const int32_t* topk_ids, const float* topk_vals, const float* uniform,
                        int32_t* output_ids, int64_t rows, int32_t K, float temperature,
                        ispore_stream_t stream) {
    return ispore::sampling_dispatch<float>(topk_ids, topk_vals, uniform, output_ids, rows, K, temperature,
                                            static_cast<cudaStream_t>(stream));
}
int ispore_sampling_f16(const int32_t* topk_ids, const void* topk_vals, const float* uniform,
                        int32_t* output_ids, int64_t rows, int32_t K, float temperature,
                        ispore_stream_t stream) {
    return ispore::sampling_dispatch<__half>(topk_ids, static_cast<const __half*>(topk_vals), uniform,
                                             output_ids, rows, K, temperature,
                                             static_cast<cudaStream_t>(stream));
}

}  // extern "C"
