// Scale + additive mask + row softmax for sm_100a.
//
// Semantics: the reference's fp32 kernel, src/kernels/attn_softmax_kernel.cu:50-125:
//   z = scale*qk + (1 - mask)*(-10000);  m = max(FLT_MIN, max_k z)
//   e = exp(z - m);  out = e * (1 / (sum e + 1e-6))
// (the reference's block max starts from FLT_MIN and its idle warps feed 0 into
// the reduction, so m never drops below FLT_MIN; a fully masked row therefore
// comes out as exact zeros).  Both storage types compute in fp32.
//
// The mask row [b, q] is shared by all heads.  A thread group (one warp for
// short rows, one CTA for long rows) therefore takes a (b, q) pair and a group
// of HG heads: it turns the mask row into the additive term once, keeps it in
// registers, issues the loads of all HG qk rows together and then finishes the
// rows one after the other.  A row lives in registers between the max, the sum
// and the store, so qk is read once and the score written once; the index
// arithmetic (one 32-bit division) is paid per group, not per row.
#include <float.h>

#include "common.cuh"
#include "tma.cuh"

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

// Division of n < 2^31 by a divisor fixed at launch: n / d = umulhi(n, mul) >> shr with
// mul = ceil(2^(31 + ceil(log2 d)) / d), exact because the rounding error of mul, scaled by
// n / 2^(31 + ceil(log2 d)), stays below 1 / d.  d = 1 has mul = 0 and is passed through.
struct InvariantDivisor {
    uint32_t mul, shr;
    explicit InvariantDivisor(uint32_t d) : mul(0), shr(0) {
        if (d > 1) {
            uint32_t l = 0;
            while ((1ull << l) < d) ++l;
            mul = static_cast<uint32_t>(((1ull << (31 + l)) + d - 1) / d);
            shr = l - 1;
        }
    }
    __device__ __forceinline__ uint32_t divide(uint32_t n) const { return mul == 0 ? n : __umulhi(n, mul) >> shr; }
};

// GROUP threads cooperate on one row; a CTA of THREADS threads holds
// THREADS/GROUP groups.  Each thread keeps VPT 128-bit vectors of a row and the
// matching slice of the additive mask term.  A group works on HG heads of one
// (b, q) pair per trip.
// MODE 0 (full): every row is exactly VPT*GROUP vectors long and heads is a multiple of HG, so the
// per-vector and per-head guards (and the branches they cost) disappear.  MODE 1 (tail): rows are
// longer than (VPT-1)*GROUP vectors, so only a thread's last vector needs its guard.  MODE 2: any
// row length and head count.
// CAUSAL: there is no mask tensor; the 0/1 mask row is derived from q_lens[b] and k_lens[b] with
// the predicate of the reference's mask builder (src/kernels/build_casual_mask.cu:36), so the
// result of this kernel is bit-identical to running it on a built mask and the [bs, q, k] tensor is never read.
#define ISPORE_IN_ROW(i, v) (MODE == 0 || (MODE == 1 && (i) < VPT - 1) || (v) < row_vecs)
template <typename T, int VPT, int GROUP, int THREADS, int HG, int MIN_BLOCKS, int MODE, bool CAUSAL>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS)
softmax_head_group_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                          const int32_t* __restrict__ q_lens, const int32_t* __restrict__ k_lens,
                          uint32_t units /* batch*q_len*head_groups */, uint32_t head_groups,
                          uint32_t heads, uint32_t q_len, int row_vecs, float scale, int q_shift, int hg_shift) {
    constexpr int E = VecTraits<T>::kElems;
    constexpr int kGroupsPerCta = THREADS / GROUP;
    constexpr int kWarpsPerGroup = GROUP / 32;
    using Exp = ExpPolicy<T>;
    __shared__ float red[2][kWarpsPerGroup > 1 ? kWarpsPerGroup : 1];  // only used when a CTA is one group
    chain_begin();

    const int tid = threadIdx.x;
    const int g = tid / GROUP;   // group slot inside the CTA
    const int gt = tid % GROUP;  // thread inside the group
    const int lane = tid & 31;
    const int gw = gt >> 5;      // warp inside the group
    const float a = scale * Exp::kPrescale;
    const float neg = -10000.0f * Exp::kPrescale;
    const float floor_m = FLT_MIN * Exp::kPrescale;

    for (uint32_t u0 = blockIdx.x * kGroupsPerCta; u0 < units; u0 += gridDim.x * kGroupsPerCta) {
        const uint32_t u = u0 + g;
        const bool live = u < units;  // with several groups per CTA there are no block barriers below
        // q index fastest: neighbouring groups work on neighbouring rows of the same heads.
        // q_shift / hg_shift: log2 of q_len / head_groups when those are powers of two (the usual
        // case), else -1: a run-time division costs as much as the arithmetic of two elements.
        uint32_t qi, t, hg, b;
        if (q_shift >= 0) {
            qi = live ? u & (q_len - 1) : 0;
            t = live ? u >> q_shift : 0;
        } else {
            qi = live ? u % q_len : 0;
            t = live ? u / q_len : 0;
        }
        if (hg_shift >= 0) {
            hg = t & (head_groups - 1);
            b = t >> hg_shift;
        } else {
            hg = t % head_groups;
            b = t / head_groups;
        }
        const uint32_t h0 = hg * HG;
        const int nh = MODE != 2 ? (live ? HG : 0) : (live ? static_cast<int>(min(static_cast<uint32_t>(HG), heads - h0)) : 0);

        const uint4* mrow = reinterpret_cast<const uint4*>(mask) + (static_cast<int64_t>(b) * q_len + qi) * row_vecs;
        const int64_t row0 = (static_cast<int64_t>(b) * heads + h0) * q_len + qi;  // row of head h0
        const int64_t head_stride_vecs = static_cast<int64_t>(q_len) * row_vecs;
        const uint4* qrow0 = reinterpret_cast<const uint4*>(qk) + row0 * row_vecs;
        uint4* orow0 = reinterpret_cast<uint4*>(score) + row0 * row_vecs;

        // All loads of the trip first: the mask slice and HG x VPT vectors of qk.
        uint4 m_raw[VPT], q_raw[HG][VPT];
        int lo = 0, hi = -1;  // CAUSAL: the ones of the mask row span k in [lo, hi]
        if (CAUSAL) {
            if (live) {
                const int qlen = __ldg(q_lens + b), klen = __ldg(k_lens + b);
                lo = klen - qlen;
                hi = static_cast<int>(qi) < qlen ? min(klen - 1, static_cast<int>(qi) + lo) : -1;
            }
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = gt + i * GROUP;
                if (live && ISPORE_IN_ROW(i, v)) m_raw[i] = ld_keep(mrow + v);
            }
        }
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = gt + i * GROUP;
                if (hh < nh && ISPORE_IN_ROW(i, v)) q_raw[hh][i] = ld_stream(qrow0 + hh * head_stride_vecs + v);
            }
        }
        // Additive mask term (1 - mask) * (-10000), prescaled; -inf-like filler beyond the row.
        Unpacked<T> term[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = gt + i * GROUP;
            if (CAUSAL) {
                // a vector lies wholly inside or outside [lo, hi] except at the two ends of the span:
                // one uniform fill, and the per-element predicate only for those boundary vectors
                const int k0 = v * E, k1 = k0 + (E - 1);
                const bool all_in = k0 >= lo && k1 <= hi;
                const bool all_out = k0 > hi || k1 < lo;
                const float fill = all_in ? 0.0f : neg;
#pragma unroll
                for (int e = 0; e < E; ++e) term[i].v[e] = fill;
                if (!all_in && !all_out) {
#pragma unroll
                    for (int e = 0; e < E; ++e) term[i].v[e] = (k0 + e >= lo && k0 + e <= hi) ? 0.0f : neg;
                }
            } else if (live && ISPORE_IN_ROW(i, v)) {
                unpack(m_raw[i], term[i]);
#pragma unroll
                for (int e = 0; e < E; ++e) term[i].v[e] = fmaf(term[i].v[e], -neg, neg);  // (1 - mask) * neg in one rounding
            }
        }

#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
            if (hh < nh) {  // uniform inside a group; uniform inside the CTA when GROUP == THREADS
                Unpacked<T> z[VPT];
                float mx = floor_m;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = gt + i * GROUP;
                    if (ISPORE_IN_ROW(i, v)) {
                        unpack(q_raw[hh][i], z[i]);
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            z[i].v[e] = fmaf(a, z[i].v[e], term[i].v[e]);
                            mx = fmaxf(mx, z[i].v[e]);
                        }
                    }
                }
                mx = warp_max(mx);
                if (kWarpsPerGroup > 1) {
                    if (lane == 0) red[0][gw] = mx;
                    __syncthreads();
#pragma unroll
                    for (int w = 0; w < kWarpsPerGroup; ++w) mx = fmaxf(mx, red[0][w]);
                }
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = gt + i * GROUP;
                    if (ISPORE_IN_ROW(i, v)) {
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            z[i].v[e] = Exp::exp_diff(z[i].v[e], mx);
                            sum += z[i].v[e];
                        }
                    }
                }
                sum = warp_sum(sum);
                if (kWarpsPerGroup > 1) {
                    if (lane == 0) red[1][gw] = sum;
                    __syncthreads();  // also orders this row's red[0] reads before the next row's writes
                    sum = 0.f;
#pragma unroll
                    for (int w = 0; w < kWarpsPerGroup; ++w) sum += red[1][w];
                }
                const float inv = 1.0f / (sum + 1e-6f);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = gt + i * GROUP;
                    if (ISPORE_IN_ROW(i, v)) {
#pragma unroll
                        for (int e = 0; e < E; ++e) z[i].v[e] *= inv;
                        st_stream(orow0 + hh * head_stride_vecs + v, pack(z[i]));
                    }
                }
                if (kWarpsPerGroup > 1) __syncthreads();  // red[1] is rewritten by the next row
            }
        }
    }
}

#undef ISPORE_IN_ROW

// Any k_len / alignment: one CTA per row, three scalar passes (the row is
// re-read from L2).  Also the path for rows too long for the register kernels.
template <typename T, int THREADS, bool CAUSAL>
__global__ void __launch_bounds__(THREADS)
softmax_generic_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                       const int32_t* __restrict__ q_lens, const int32_t* __restrict__ k_lens, int64_t total_rows, int64_t rows_per_batch, int q_len, int64_t k_len,
                       float scale) {
    constexpr int kWarps = THREADS / 32;
    __shared__ float red[2][kWarps];
    const int tid = threadIdx.x;
    for (int64_t row = blockIdx.x; row < total_rows; row += gridDim.x) {
        const int64_t bidx = row / rows_per_batch;
        const int64_t qi = (row - bidx * rows_per_batch) % q_len;
        const T* qrow = qk + row * k_len;
        const T* mrow = CAUSAL ? nullptr : mask + (bidx * q_len + qi) * k_len;
        T* orow = score + row * k_len;
        int64_t lo = 0, hi = -1;
        if (CAUSAL) {
            const int qlen = __ldg(q_lens + bidx), klen = __ldg(k_lens + bidx);
            lo = klen - qlen;
            hi = qi < qlen ? min(static_cast<int64_t>(klen) - 1, qi + lo) : -1;
        }
        // additive term (1 - mask) * (-10000) of element i
        auto term = [&](int64_t i) -> float {
            if (CAUSAL) return (i >= lo && i <= hi) ? 0.0f : -10000.0f;
            return (1.0f - to_float<T>(mrow[i])) * -10000.0f;
        };
        float mx = FLT_MIN;
        for (int64_t i = tid; i < k_len; i += THREADS) mx = fmaxf(mx, fmaf(scale, to_float<T>(qrow[i]), term(i)));
        mx = warp_max(mx);
        if ((tid & 31) == 0) red[0][tid >> 5] = mx;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, red[0][w]);
        float sum = 0.f;
        for (int64_t i = tid; i < k_len; i += THREADS)
            sum += expf(fmaf(scale, to_float<T>(qrow[i]), term(i)) - mx);
        sum = warp_sum(sum);
        if ((tid & 31) == 0) red[1][tid >> 5] = sum;
        __syncthreads();
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red[1][w];
        const float inv = 1.0f / (sum + 1e-6f);
        for (int64_t i = tid; i < k_len; i += THREADS) {
            const float e = expf(fmaf(scale, to_float<T>(qrow[i]), term(i)) - mx);
            orow[i] = from_float<T>(e * inv);
        }
        __syncthreads();
    }
}

// Rows that cannot be moved as 128-bit vectors (buffers that are not 16-byte aligned, rows shorter
// than two vectors) but fit a CTA's registers: one CTA per row, EPT scalar elements per thread, the row read
// once and written once.
template <typename T, int THREADS, int EPT, bool CAUSAL>
__global__ void __launch_bounds__(THREADS)
softmax_row_scalar_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                          const int32_t* __restrict__ q_lens, const int32_t* __restrict__ k_lens,
                          int64_t total_rows, int64_t rows_per_batch, int q_len, int k_len, float scale) {
    constexpr int kWarps = THREADS / 32;
    __shared__ float red[2][kWarps];
    const int tid = threadIdx.x;
    for (int64_t row = blockIdx.x; row < total_rows; row += gridDim.x) {
        const int64_t bidx = row / rows_per_batch;
        const int qi = static_cast<int>((row - bidx * rows_per_batch) % q_len);
        const T* qrow = qk + row * k_len;
        const T* mrow = CAUSAL ? nullptr : mask + (bidx * q_len + qi) * k_len;
        T* orow = score + row * k_len;
        int lo = 0, hi = -1;
        if (CAUSAL) {
            const int qlen = __ldg(q_lens + bidx), klen = __ldg(k_lens + bidx);
            lo = klen - qlen;
            hi = qi < qlen ? min(klen - 1, qi + lo) : -1;
        }
        float z[EPT];
        float mx = FLT_MIN;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int i = tid + j * THREADS;
            if (i < k_len) {
                const float term = CAUSAL ? ((i >= lo && i <= hi) ? 0.0f : -10000.0f)
                                          : (1.0f - to_float<T>(mrow[i])) * -10000.0f;
                z[j] = fmaf(scale, to_float<T>(qrow[i]), term);
                mx = fmaxf(mx, z[j]);
            }
        }
        mx = warp_max(mx);
        if ((tid & 31) == 0) red[0][tid >> 5] = mx;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, red[0][w]);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            if (tid + j * THREADS < k_len) {
                z[j] = expf(z[j] - mx);
                sum += z[j];
            }
        }
        sum = warp_sum(sum);
        if ((tid & 31) == 0) red[1][tid >> 5] = sum;
        __syncthreads();
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red[1][w];
        const float inv = 1.0f / (sum + 1e-6f);
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int i = tid + j * THREADS;
            if (i < k_len) orow[i] = from_float<T>(z[j] * inv);
        }
        __syncthreads();  // red[] is rewritten by the next row
    }
}

// Where the 0/1 mask comes from: a [batch, q_len, k_len] tensor (the reference's interface) or
// the two length arrays it would have been built from.
template <typename T>
struct MaskSource {
    const T* mask;
    const int32_t* q_lens;
    const int32_t* k_lens;
};

inline int log2_or_minus1(int64_t v) {
    if (v <= 0 || (v & (v - 1)) != 0) return -1;
    int s = 0;
    while ((int64_t{1} << s) < v) ++s;
    return s;
}

template <typename T, bool CAUSAL, int VPT, int GROUP, int THREADS, int HG, int MIN_BLOCKS = 1>
int launch_groups(T* score, const T* qk, const MaskSource<T>& ms, int64_t batch, int64_t heads, int64_t q_len,
                  int row_vecs, float scale, cudaStream_t st) {
    constexpr int kGroupsPerCta = THREADS / GROUP;
    const int64_t head_groups = ceil_div(heads, HG);
    const int64_t units = batch * q_len * head_groups;
    const int64_t ctas = ceil_div(units, kGroupsPerCta);
    const bool whole_groups = heads % HG == 0;
    auto kernel = softmax_head_group_kernel<T, VPT, GROUP, THREADS, HG, MIN_BLOCKS, 2, CAUSAL>;
    if (whole_groups && row_vecs == VPT * GROUP)
        kernel = softmax_head_group_kernel<T, VPT, GROUP, THREADS, HG, MIN_BLOCKS, 0, CAUSAL>;
    else if (whole_groups && row_vecs > (VPT - 1) * GROUP)
        kernel = softmax_head_group_kernel<T, VPT, GROUP, THREADS, HG, MIN_BLOCKS, 1, CAUSAL>;
    // One trip per CTA for any realistic size: the hardware scheduler hands out CTAs in
    // address order, which keeps the DRAM access front compact.
    const int grid = static_cast<int>(ctas < (1 << 30) ? ctas : (1 << 30));
    launch_chained(kernel, grid, THREADS, 0, st, score, qk, ms.mask, ms.q_lens, ms.k_lens, static_cast<uint32_t>(units),
                   static_cast<uint32_t>(head_groups), static_cast<uint32_t>(heads), static_cast<uint32_t>(q_len),
                   row_vecs, scale, log2_or_minus1(q_len), log2_or_minus1(head_groups));
    return check_launch("softmax_head_group_kernel");
}

// (Measured and not kept for these rows: eight consecutive rows — a span that is 16-byte aligned
// whatever the row length — staged through shared memory with TMA bulk copies and worked on there
// element by element, one warp per row: 0.44 of the copy rate on 777-long fp16 rows against 0.72
// for the kernel below; 2-byte shared- and global-memory accesses cost more issue slots than the
// register shifts they replace.  Likewise a row split over a thread-block cluster for rows of
// 8 K to 32 K elements, with a distributed-shared-memory max/sum exchange: 0.53 against 0.60.)
// Rows of any length in 16-byte aligned buffers, without shared memory: a group (a warp, or the
// CTA for long rows) takes one row.  The whole aligned vectors inside the row go through the
// vector trips; the up to E-1 elements in front of the first one and the up to E-1 behind the
// last one (they share their vectors with the neighbouring rows) are taken one per lane by the
// first lanes of the group, loaded and stored as single elements.  The mask row of (b, q) starts
// at another element offset than the qk row: the two aligned mask vectors that hold a qk
// vector's eight (four) positions are loaded and shifted into place in registers — the shift is
// the same for the whole row, so one uniform switch per row picks the routine compiled for it.
// The last mask row, whose second vector could reach past the buffer, takes a plain
// element-wise path.  The kernel is bound by instruction issue, so the trips are kept free of
// guards (the launch shape guarantees that only a thread's last vector can lie past the row) and
// the grid is three-dimensional (q, head, sequence) so that no index is recovered by division.
template <typename T, int S>
__device__ __forceinline__ uint4 shift_into_place(const uint4& a, const uint4& b) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (sizeof(T) == 4) return make_uint4(w[S & 3], w[(S & 3) + 1], w[(S & 3) + 2], w[(S & 3) + 3]);
    constexpr int J = (S >> 1) & 3;
    if ((S & 1) == 0) return make_uint4(w[J], w[J + 1], w[J + 2], w[J + 3]);
    return make_uint4(__funnelshift_r(w[J], w[J + 1], 16), __funnelshift_r(w[J + 1], w[J + 2], 16),
                      __funnelshift_r(w[J + 2], w[J + 3], 16), __funnelshift_r(w[J + 3], w[J + 4], 16));
}

template <typename T>
struct OffsetRow {
    T* score;
    const T* qk;
    const T* mask;
    int64_t row_elem0, mrow_elem0;  // first element of the qk row and of the mask row
    float* red_max;
    float* red_sum;
    int k_len, head, lo, hi, group, gt;
    float a;
};

// One row, for a mask row whose element under the row's first whole vector sits S elements into
// its own aligned vector.
template <typename T, int VPT, bool kBlock, bool CAUSAL, int S>
__device__ __forceinline__ void offset_row_fast(const OffsetRow<T>& row) {
    constexpr int E = VecTraits<T>::kElems;
    using Exp = ExpPolicy<T>;
    const float neg = -10000.0f * Exp::kPrescale;
    const int k_len = row.k_len, head = row.head, group = row.group, gt = row.gt;
    const float a = row.a;
    const int tail = (k_len - head) & (E - 1);   // elements behind the last whole vector
    const int n_whole = (k_len - head) / E;      // whole vectors of the row
    const bool tail_valid = gt + (VPT - 1) * group < n_whole;  // earlier trips are full by the launch shape
    const uint4* qp = reinterpret_cast<const uint4*>(row.qk + row.row_elem0 + head) + gt;
    uint4* op = reinterpret_cast<uint4*>(row.score + row.row_elem0 + head) + gt;
    // the single elements: lanes 0..head-1 the front ones, the next `tail` lanes the back ones
    const int single = gt < head ? gt : (gt < head + tail ? k_len - tail + (gt - head) : -1);

    uint4 raw[VPT], mraw[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i)
        raw[i] = (i < VPT - 1 || tail_valid) ? ld_stream(qp + i * group) : make_uint4(0, 0, 0, 0);
    // (the single elements are only loaded here and used after the mask vectors are on their way:
    // their arithmetic in between would hold back the loads behind it for a full memory latency)
    T single_x = from_float<T>(0.f), single_m = from_float<T>(0.f);
    if (single >= 0) {
        single_x = row.qk[row.row_elem0 + single];
        if (!CAUSAL) single_m = row.mask[row.mrow_elem0 + single];
    }
    // every load of the row is issued before the first value is used
    uint4 mnext[S == 0 ? 1 : VPT];  // the second mask vector of each trip
    if (!CAUSAL) {
        const uint4* mp = reinterpret_cast<const uint4*>(row.mask + (row.mrow_elem0 + head - S)) + gt;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (i < VPT - 1 || tail_valid) {
                mraw[i] = ld_keep(mp + i * group);
                if (S != 0) mnext[i] = ld_keep(mp + i * group + 1);
            }
        }
    }
    float zs = -FLT_MAX;
    if (single >= 0) {
        const float term = CAUSAL ? ((single >= row.lo && single <= row.hi) ? 0.0f : neg) : fmaf(to_float<T>(single_m), -neg, neg);
        zs = fmaf(a, to_float<T>(single_x), term);
    }
    Unpacked<T> z[VPT];
    float mx = fmaxf(FLT_MIN * Exp::kPrescale, zs);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        unpack(raw[i], z[i]);
        if (i < VPT - 1 || tail_valid) {
            if (CAUSAL) {
                const int k0 = head + (gt + i * group) * E;  // position of the vector's first element
                if (k0 >= row.lo && k0 + E - 1 <= row.hi) {
#pragma unroll
                    for (int e = 0; e < E; ++e) z[i].v[e] *= a;
                } else if (k0 > row.hi || k0 + E - 1 < row.lo) {
#pragma unroll
                    for (int e = 0; e < E; ++e) z[i].v[e] = fmaf(a, z[i].v[e], neg);
                } else {
#pragma unroll
                    for (int e = 0; e < E; ++e)
                        z[i].v[e] = fmaf(a, z[i].v[e], (k0 + e >= row.lo && k0 + e <= row.hi) ? 0.0f : neg);
                }
            } else {
                Unpacked<T> m;
                unpack(S == 0 ? mraw[i] : shift_into_place<T, S>(mraw[i], mnext[S == 0 ? 0 : i]), m);
#pragma unroll
                for (int e = 0; e < E; ++e) z[i].v[e] = fmaf(a, z[i].v[e], fmaf(m.v[e], -neg, neg));
            }
#pragma unroll
            for (int e = 0; e < E; ++e) mx = fmaxf(mx, z[i].v[e]);
        }
    }
    mx = warp_max(mx);
    if (kBlock) {
        if ((threadIdx.x & 31) == 0) row.red_max[threadIdx.x >> 5] = mx;
        __syncthreads();
        mx = row.red_max[0];
        for (int w = 1; w < (group >> 5); ++w) mx = fmaxf(mx, row.red_max[w]);
    }
    float sum = single >= 0 ? (zs = Exp::exp_diff(zs, mx)) : 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (i < VPT - 1 || tail_valid) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
                z[i].v[e] = Exp::exp_diff(z[i].v[e], mx);
                sum += z[i].v[e];
            }
        }
    }
    sum = warp_sum(sum);
    if (kBlock) {
        if ((threadIdx.x & 31) == 0) row.red_sum[threadIdx.x >> 5] = sum;
        __syncthreads();
        sum = row.red_sum[0];
        for (int w = 1; w < (group >> 5); ++w) sum += row.red_sum[w];
    }
    const float inv = 1.0f / (sum + 1e-6f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (i < VPT - 1 || tail_valid) {
#pragma unroll
            for (int e = 0; e < E; ++e) z[i].v[e] *= inv;
            st_stream(op + i * group, pack(z[i]));
        }
    }
    if (single >= 0) row.score[row.row_elem0 + single] = from_float<T>(zs * inv);
}

// GROUP lanes per row: 32 (a warp; THREADS / 32 consecutive rows per CTA) or 0 = the whole CTA,
// whose size is then chosen at launch to fit the row.  The grid is flat over the rows; (sequence,
// head, q) come back through two multiply-shift divisions.
// (five CTAs of eight rows per SM: 48 registers; measured +6 % on 1001-long fp16 rows, six spill)
template <typename T, int VPT, int GROUP, int THREADS, bool CAUSAL>
__global__ void __launch_bounds__(THREADS, (GROUP == 32 && THREADS == 256 ? 5 : 1))
softmax_offset_row_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                          const int32_t* __restrict__ q_lens, const int32_t* __restrict__ k_lens, uint32_t total_rows,
                          int batch, int q_len, int k_len, InvariantDivisor by_q_len, InvariantDivisor by_heads,
                          float scale) {
    constexpr int E = VecTraits<T>::kElems;
    static_assert(GROUP == 32 || GROUP == 0, "a group is a warp or the CTA");
    constexpr bool kBlock = GROUP == 0;
    using Exp = ExpPolicy<T>;
    __shared__ float red_max[THREADS / 32], red_sum[THREADS / 32];  // each written once per row: no barrier after the read
    chain_begin();
    const int tid = threadIdx.x;
    const int group = kBlock ? static_cast<int>(blockDim.x) : GROUP;
    const int gt = kBlock ? tid : (tid & 31);
    const uint32_t r = kBlock ? blockIdx.x : blockIdx.x * (THREADS / 32) + (tid >> 5);  // flat row
    if (r >= total_rows) return;  // a whole warp leaves
    const uint32_t bh = by_q_len.divide(r);
    const int qi = static_cast<int>(r - bh * static_cast<uint32_t>(q_len));
    const int b = static_cast<int>(by_heads.divide(bh));
    const float a = scale * Exp::kPrescale;
    const float neg = -10000.0f * Exp::kPrescale;
    const int64_t row_elem0 = static_cast<int64_t>(r) * k_len;
    const int64_t mrow_elem0 = (static_cast<int64_t>(b) * q_len + qi) * k_len;
    int lo = 0, hi = -1;  // CAUSAL: positions lo..hi are visible
    if (CAUSAL) {
        const int qlen = __ldg(q_lens + b), klen = __ldg(k_lens + b);
        lo = klen - qlen;
        hi = qi < qlen ? min(klen - 1, qi + lo) : -1;
    }

    // (the same rows with and without a mask tensor, so that both give the same bits)
    if (b == batch - 1 && qi == q_len - 1) {  // uniform over the group: element-wise, three passes over the row
        const T* in = qk + row_elem0;
        T* out = score + row_elem0;
        const T* mrow = CAUSAL ? nullptr : mask + mrow_elem0;
        auto z_at = [&](int k) {
            const float term = CAUSAL ? ((k >= lo && k <= hi) ? 0.0f : neg) : fmaf(to_float<T>(mrow[k]), -neg, neg);
            return fmaf(a, to_float<T>(in[k]), term);
        };
        float mx = FLT_MIN * Exp::kPrescale;
        for (int k = gt; k < k_len; k += group) mx = fmaxf(mx, z_at(k));
        mx = warp_max(mx);
        if (kBlock) {
            if ((tid & 31) == 0) red_max[tid >> 5] = mx;
            __syncthreads();
            mx = red_max[0];
            for (int w = 1; w < (group >> 5); ++w) mx = fmaxf(mx, red_max[w]);
        }
        float sum = 0.f;
        for (int k = gt; k < k_len; k += group) sum += Exp::exp_diff(z_at(k), mx);
        sum = warp_sum(sum);
        if (kBlock) {
            if ((tid & 31) == 0) red_sum[tid >> 5] = sum;
            __syncthreads();
            sum = red_sum[0];
            for (int w = 1; w < (group >> 5); ++w) sum += red_sum[w];
        }
        const float inv = 1.0f / (sum + 1e-6f);
        for (int k = gt; k < k_len; k += group) out[k] = from_float<T>(Exp::exp_diff(z_at(k), mx) * inv);
        return;
    }

    OffsetRow<T> row;
    row.score = score;
    row.qk = qk;
    row.mask = mask;
    row.row_elem0 = row_elem0;
    row.mrow_elem0 = mrow_elem0;
    row.red_max = red_max;
    row.red_sum = red_sum;
    row.k_len = k_len;
    row.head = static_cast<int>(-row_elem0 & (E - 1));  // elements in front of the row's first whole vector
    row.lo = lo;
    row.hi = hi;
    row.group = group;
    row.gt = gt;
    row.a = a;
    if (CAUSAL) {
        offset_row_fast<T, VPT, kBlock, true, 0>(row);
        return;
    }
    switch (static_cast<int>((mrow_elem0 + row.head) & (E - 1))) {
        case 1: offset_row_fast<T, VPT, kBlock, CAUSAL, 1>(row); break;
        case 2: offset_row_fast<T, VPT, kBlock, CAUSAL, 2>(row); break;
        case 3: offset_row_fast<T, VPT, kBlock, CAUSAL, 3>(row); break;
        case 4: offset_row_fast<T, VPT, kBlock, CAUSAL, E == 8 ? 4 : 0>(row); break;
        case 5: offset_row_fast<T, VPT, kBlock, CAUSAL, E == 8 ? 5 : 0>(row); break;
        case 6: offset_row_fast<T, VPT, kBlock, CAUSAL, E == 8 ? 6 : 0>(row); break;
        case 7: offset_row_fast<T, VPT, kBlock, CAUSAL, E == 8 ? 7 : 0>(row); break;
        default: offset_row_fast<T, VPT, kBlock, CAUSAL, 0>(row); break;
    }
}

// Long rows of whole vectors (up to 64 values per thread of a 256-thread CTA: 16384 elements).
// The register kernels above keep a row's loads in flight in registers, which bounds the bytes an
// SM has under way by its register file: measured 0.59 of the copy rate on 16384-long fp16 rows,
// 0.75 with the launch shape that has the most of them.  Here the rows travel through the copy
// engine instead: a CTA walks the rows b, b + grid, ... with a ring of shared-memory row buffers,
// the next two rows requested (cp.async.bulk, one mbarrier per buffer) while one is worked on;
// the normalised row is written back into its buffer and leaves as one bulk store.  A thread
// holds the same vectors of every row (v = tid, tid + 256, ...), so nothing but the two
// reductions crosses threads.  Same arithmetic as the head-group kernel.
constexpr int kStagedMaxBuf = 4;

template <typename T, int VPT, int kStagedThreads, bool CAUSAL>
__global__ void __launch_bounds__(kStagedThreads, (kStagedThreads > 256 ? 1 : kStagedThreads > 128 ? 2 : kStagedThreads > 64 ? 4 : kStagedThreads > 32 ? 8 : 16))
softmax_staged_row_kernel(T* __restrict__ score, const T* __restrict__ qk, const T* __restrict__ mask,
                          const int32_t* __restrict__ q_lens, const int32_t* __restrict__ k_lens,
                          uint32_t total_rows, uint32_t heads, uint32_t q_len, int row_vecs, float scale,
                          int nbuf, unsigned* __restrict__ status) {
    constexpr int E = VecTraits<T>::kElems;
    constexpr int kWarps = kStagedThreads / 32;
    using Exp = ExpPolicy<T>;
    extern __shared__ __align__(128) unsigned char rows_raw[];  // [nbuf][row_vecs * 16]
    __shared__ __align__(8) uint64_t full[kStagedMaxBuf];
    __shared__ float red[2][kWarps];
    __shared__ int s_timeout;
    chain_begin();

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const uint32_t row_bytes = static_cast<uint32_t>(row_vecs) * 16u;
    const float a = scale * Exp::kPrescale;
    const float neg = -10000.0f * Exp::kPrescale;
    const float floor_m = FLT_MIN * Exp::kPrescale;
    const uint32_t rows_per_batch = heads * q_len;

    // Trip i of this CTA works on row blockIdx.x + i * gridDim.x, in buffer i % nbuf.
    auto row_of = [&](uint32_t i) { return static_cast<uint64_t>(blockIdx.x) + static_cast<uint64_t>(i) * gridDim.x; };
    auto request_row = [&](uint32_t i) {  // thread 0 only
        const uint64_t r = row_of(i);
        if (r >= total_rows) return;
        const uint32_t b = i % static_cast<uint32_t>(nbuf);
        tma::mbar_arrive_expect_tx(&full[b], row_bytes);
        tma::load(rows_raw + static_cast<size_t>(b) * row_bytes, qk + r * static_cast<uint64_t>(row_vecs) * E, row_bytes, &full[b]);
    };
    if (tid == 0) {
        for (int b = 0; b < nbuf; ++b) tma::mbar_init(&full[b], 1);
        tma::fence_mbar_init();
        s_timeout = 0;
        for (int i = 0; i < nbuf - 1; ++i) request_row(static_cast<uint32_t>(i));
    }
    __syncthreads();

    // The mask slice of a row comes from L2 and is needed as soon as the row's buffer has landed,
    // which, thanks to the ring, is at once: it is requested a trip ahead, right after the previous
    // row has consumed its own (the registers are free from there on), and is there in time.
    uint4 m_raw[VPT];
    auto request_mask = [&](uint32_t i) {
        const uint64_t r = row_of(i);
        if (CAUSAL || r >= total_rows) return;
        const uint32_t b = static_cast<uint32_t>(r / rows_per_batch);
        const uint32_t qi = static_cast<uint32_t>(r - static_cast<uint64_t>(b) * rows_per_batch) % q_len;
        const uint4* mrow = reinterpret_cast<const uint4*>(mask) + (static_cast<int64_t>(b) * q_len + qi) * row_vecs;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = tid + j * kStagedThreads;
            if (v < row_vecs) m_raw[j] = ld_keep(mrow + v);
        }
    };
    request_mask(0);

    for (uint32_t i = 0;; ++i) {
        const uint64_t r = row_of(i);
        if (r >= total_rows) break;  // uniform
        const uint32_t buf = i % static_cast<uint32_t>(nbuf);
        const uint32_t parity = (i / static_cast<uint32_t>(nbuf)) & 1u;
        const uint32_t b = static_cast<uint32_t>(r / rows_per_batch);
        const uint32_t qi = static_cast<uint32_t>(r - static_cast<uint64_t>(b) * rows_per_batch) % q_len;

        int lo = 0, hi = -1;  // CAUSAL: the ones of the mask row span k in [lo, hi]
        if (CAUSAL) {
            const int qlen = __ldg(q_lens + b), klen = __ldg(k_lens + b);
            lo = klen - qlen;
            hi = static_cast<int>(qi) < qlen ? min(klen - 1, static_cast<int>(qi) + lo) : -1;
        }
        // A wait that runs out is recorded here and acted on by the whole CTA after the next barrier.
        if (!tma::mbar_wait(&full[buf], parity)) s_timeout = 1;
        uint4* srow = reinterpret_cast<uint4*>(rows_raw + static_cast<size_t>(buf) * row_bytes);

        Unpacked<T> z[VPT];
        float mx = floor_m;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = tid + j * kStagedThreads;
            if (v < row_vecs) {
                Unpacked<T> term;
                if (CAUSAL) {
                    const int k0 = v * E, k1 = k0 + (E - 1);
                    const bool all_in = k0 >= lo && k1 <= hi;
                    const bool all_out = k0 > hi || k1 < lo;
                    const float fill = all_in ? 0.0f : neg;
#pragma unroll
                    for (int e = 0; e < E; ++e) term.v[e] = fill;
                    if (!all_in && !all_out) {
#pragma unroll
                        for (int e = 0; e < E; ++e) term.v[e] = (k0 + e >= lo && k0 + e <= hi) ? 0.0f : neg;
                    }
                } else {
                    unpack(m_raw[j], term);
#pragma unroll
                    for (int e = 0; e < E; ++e) term.v[e] = fmaf(term.v[e], -neg, neg);  // (1 - mask) * neg in one rounding
                }
                unpack(srow[v], z[j]);
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    z[j].v[e] = fmaf(a, z[j].v[e], term.v[e]);
                    mx = fmaxf(mx, z[j].v[e]);
                }
            }
        }
        request_mask(i + 1);
        mx = warp_max(mx);
        if (lane == 0) red[0][warp] = mx;
        __syncthreads();
        if (s_timeout) {  // uniform: give up, but not before the copies under way have landed
            if (tid == 0) {
                atomicOr(status, ISPORE_DEV_TIMEOUT);
                for (uint32_t i2 = i; i2 < i + static_cast<uint32_t>(nbuf) - 1u && row_of(i2) < total_rows; ++i2)
                    tma::mbar_wait(&full[i2 % static_cast<uint32_t>(nbuf)], (i2 / static_cast<uint32_t>(nbuf)) & 1u);
                tma::wait_group_read<0>();
            }
            return;
        }
        // The buffer of the previous row is free once its bulk store has read it: row i + nbuf - 1 goes there.
        if (tid == 0) {
            tma::wait_group_read<0>();
            request_row(i + static_cast<uint32_t>(nbuf) - 1u);
        }
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, red[0][w]);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = tid + j * kStagedThreads;
            if (v < row_vecs) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    z[j].v[e] = Exp::exp_diff(z[j].v[e], mx);
                    sum += z[j].v[e];
                }
            }
        }
        sum = warp_sum(sum);
        if (lane == 0) red[1][warp] = sum;
        __syncthreads();
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red[1][w];
        const float inv = 1.0f / (sum + 1e-6f);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = tid + j * kStagedThreads;
            if (v < row_vecs) {
#pragma unroll
                for (int e = 0; e < E; ++e) z[j].v[e] *= inv;
                srow[v] = pack(z[j]);
            }
        }
        tma::fence_proxy_async();  // the row written above is read by the copy engine
        __syncthreads();
        if (tid == 0) {
            tma::store(score + r * static_cast<uint64_t>(row_vecs) * E, srow, row_bytes);
            tma::commit_group();
        }
    }
    if (tid == 0) tma::wait_group_read<0>();  // shared memory must outlive the last store's read
}

template <typename T, bool CAUSAL, int VPT, int kStagedThreads>
int launch_staged_rows(T* score, const T* qk, const MaskSource<T>& ms, int64_t total_rows, int64_t heads, int64_t q_len,
                       int row_vecs, float scale, cudaStream_t st) {
    auto kernel = softmax_staged_row_kernel<T, VPT, kStagedThreads, CAUSAL>;
    const size_t row_bytes = static_cast<size_t>(row_vecs) * 16;
    // Two CTAs of 256 threads with three buffers each, or one of 512 with as many as fit (up to four).
    int nbuf = 3;
    if (kStagedThreads > 256 && 4 * row_bytes <= 220 * 1024) nbuf = 4;
    if (kStagedThreads < 256) nbuf = 4;
    const size_t smem = nbuf * row_bytes;
    if (!allow_dynamic_smem(kernel, smem)) return fail(ISPORE_ELAUNCH, "softmax: %zu bytes of dynamic shared memory refused", smem);
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "softmax: no device status word");
    const int64_t resident = resident_ctas(reinterpret_cast<const void*>(kernel), kStagedThreads, smem);
    const int grid = static_cast<int>(total_rows < resident ? total_rows : resident);
    launch_chained(kernel, grid, kStagedThreads, smem, st, score, qk, ms.mask, ms.q_lens, ms.k_lens,
                   static_cast<uint32_t>(total_rows), static_cast<uint32_t>(heads), static_cast<uint32_t>(q_len), row_vecs,
                   scale, nbuf, status);
    return check_launch("softmax_staged_row_kernel");
}

template <typename T, bool CAUSAL>
int softmax_dispatch(T* score, const T* qk, const MaskSource<T>& ms, int64_t batch, int64_t heads, int64_t q_len,
                     int64_t k_len, float scale, cudaStream_t st) {
    const char* name = CAUSAL ? "scale_causal_softmax" : "scale_mask_softmax";
    if (batch < 0 || heads <= 0 || q_len <= 0 || k_len <= 0 || q_len > INT32_MAX || (CAUSAL && k_len > INT32_MAX))
        return fail(ISPORE_ESHAPE, "%s: bad shape [%lld,%lld,%lld,%lld]", name, (long long)batch, (long long)heads,
                    (long long)q_len, (long long)k_len);
    if (batch == 0) return ISPORE_OK;
    if (!score || !qk || (CAUSAL ? (!ms.q_lens || !ms.k_lens) : !ms.mask))
        return fail(ISPORE_ENULL, "%s: NULL buffer", name);
    const int64_t total_rows = batch * heads * q_len;
    constexpr int E = VecTraits<T>::kElems;
    const bool vec_ok = k_len % E == 0 && aligned16(score) && aligned16(qk) && (CAUSAL || aligned16(ms.mask)) &&
                        total_rows < (1ll << 32) && heads < (1ll << 31);
    const int64_t vecs = k_len / E;
    // Two families of kernels.  The head-group kernels (rows of whole vectors only) share a mask row
    // between heads and win where a row fills their launch shape: short rows and powers of two.
    // The row kernels take any length and win elsewhere, by a wide margin on lengths such as 640,
    // 3000 or 5000 and on every fp32 row without a mask tensor.  Measured on B200, both families,
    // fp16 and fp32, k_len 128 .. 16384.
    const int64_t whole = k_len / E;  // a row holds `whole` or `whole - 1` whole aligned vectors
    const bool rows_ok = aligned16(score) && aligned16(qk) && (CAUSAL || aligned16(ms.mask)) && k_len >= 2 * E &&
                         whole <= 4096 && total_rows < (1ll << 31);
    const bool pow2 = (k_len & (k_len - 1)) == 0;
    bool prefer_rows;
    if (sizeof(T) == 2)
        prefer_rows = CAUSAL ? (k_len > 512 && k_len != 4096) : (k_len > 512 && !(pow2 && k_len >= 4096));
    else
        prefer_rows = CAUSAL ? k_len >= 288 : (k_len > 256 && !pow2 && !(k_len >= 1000 && k_len <= 2048));
    // Rows of more than 16 KB (whole vectors, up to 4096 of them) go through the staged kernel:
    // measured on B200 against the kernels below, with and without a mask tensor, 0.74-0.93 of the
    // copy rate against 0.51-0.74 (fp32 from 6000 elements, fp16 from 12000; 16384: 0.84-0.92
    // against 0.55-0.67).  Shorter rows lose there: one CTA per row synchronises too often.
    // Rows of 8 to 16 KB that are not a power of two long (where the head-group shapes fit badly and
    // the row kernels run at 0.63-0.80), and fp16 rows of 8192 without a mask tensor: the same
    // staged kernel with four warps per row and four CTAs per SM — measured 0.72-0.89 (fp16 5000,
    // 6000; fp32 3000), 0.82 against 0.72 on the 8192-long mask-free fp16 rows.
    // fp16 rows of 3 to 4 KB (beyond what the warp-per-row kernel holds in registers), one warp per
    // row and no block barrier at all: 1792 elements 0.68 -> 0.84 with a mask tensor, 0.73 -> 0.82
    // without; 2048 with a mask tensor 0.73 -> 0.78 (without: the head-group kernel's 0.81 stands).
    if (vec_ok && sizeof(T) == 2 && vecs > 192 && vecs <= 256 && !(CAUSAL && pow2) && tune(kTuneSoftmax, 0) != 1)
        return launch_staged_rows<T, CAUSAL, 8, 32>(score, qk, ms, total_rows, heads, q_len, static_cast<int>(vecs), scale, st);
    // Rows of 4 to 8 KB between the powers of two, two warps per row and eight CTAs per SM: fp16
    // 2560 / 3000 / 3584 elements 0.67-0.74 -> 0.73-0.79 with a mask tensor, 0.69-0.80 -> 0.74-0.80
    // without; fp32 1536 with a mask tensor 0.81 -> 0.89 (without: the row kernel's 0.93 stands).
    if (vec_ok && vecs > 256 && vecs < 512 && (sizeof(T) == 2 || !CAUSAL) && tune(kTuneSoftmax, 0) != 1)
        return launch_staged_rows<T, CAUSAL, 8, 64>(score, qk, ms, total_rows, heads, q_len, static_cast<int>(vecs), scale, st);
    if (vec_ok && vecs > 512 && vecs <= 1024 && (!pow2 || (CAUSAL && sizeof(T) == 2)) && tune(kTuneSoftmax, 0) != 1)
        return launch_staged_rows<T, CAUSAL, 8, 128>(score, qk, ms, total_rows, heads, q_len, static_cast<int>(vecs), scale, st);
    if (vec_ok && vecs <= 4096 && vecs > 1024 && tune(kTuneSoftmax, 0) != 1) {
        const int rv = static_cast<int>(vecs);
        // rows of which only one CTA's ring fits an SM, or with more than 8 vectors per thread, get twice the threads
        const bool wide = vecs * 16 * 3 * 2 > 220 * 1024 || vecs > 8 * 256;
        const int64_t per_thread = ceil_div(vecs, static_cast<int64_t>(wide ? 512 : 256));
#define ISPORE_STAGED(VPT, THREADS) \
    return launch_staged_rows<T, CAUSAL, VPT, THREADS>(score, qk, ms, total_rows, heads, q_len, rv, scale, st)
        if (wide) {
            if (per_thread <= 4) ISPORE_STAGED(4, 512);
            ISPORE_STAGED(8, 512);
        } else {
            if (per_thread <= 4) ISPORE_STAGED(4, 256);
            ISPORE_STAGED(8, 256);
        }
#undef ISPORE_STAGED
    }
    if (vec_ok && !(rows_ok && prefer_rows)) {
        const int rv = static_cast<int>(vecs);
#define ISPORE_SOFTMAX(VPT, GROUP, THREADS, HG, MINB) \
    return launch_groups<T, CAUSAL, VPT, GROUP, THREADS, HG, MINB>(score, qk, ms, batch, heads, q_len, rv, scale, st)
        if (vecs <= 32) ISPORE_SOFTMAX(1, 32, 256, 4, 1);
        if (vecs <= 64) ISPORE_SOFTMAX(2, 32, 256, 2, 4);
        // (launch shapes below were picked by measurement on B200, fp16 and fp32, full and ragged rows)
        if (vecs <= 128) {
            if (vecs == 128 && heads % 2 == 0) ISPORE_SOFTMAX(4, 32, 256, 2, 1);
            ISPORE_SOFTMAX(1, 128, 128, 4, 1);  // ragged rows: one vector per thread, no idle trips
        }
        if (vecs <= 256) ISPORE_SOFTMAX(4, 64, 64, 2, 1);
        // (Few units, e.g. a decode step: one head per group gives four times the CTAs, and the ramp of
        // a launch that is a single wave of them is what such a call costs — [64, 32, 1, 4096] fp16:
        // 8.0 us against 8.75 us replayed from a graph.)
        if (vecs <= 512 && vecs > 256 && tune(kTuneSoftmax, 0) != 40 &&
            batch * q_len * ceil_div(heads, static_cast<int64_t>(4)) <= 4 * static_cast<int64_t>(sm_count()))
            ISPORE_SOFTMAX(4, 128, 128, 1, 4);
        if (vecs <= 512) ISPORE_SOFTMAX(4, 128, 128, 4, 4);
        if (vecs <= 1024) ISPORE_SOFTMAX(4, 256, 256, 1, 1);
        if (vecs <= 2048) {
            if (sizeof(T) == 4) ISPORE_SOFTMAX(4, 512, 512, 1, 1);
            ISPORE_SOFTMAX(4, 512, 512, 2, 1);
        }
        if (vecs <= 4096) ISPORE_SOFTMAX(8, 512, 512, 1, 1);
#undef ISPORE_SOFTMAX
    }
    const int64_t rows_per_batch = heads * q_len;
    {
        // Any row length at least two vectors long: one row per warp or per CTA, mask shifted in registers.
        if (rows_ok) {
#define ISPORE_SOFTMAX_OFFSET(VPT, GROUP, THREADS, rows_per_cta, threads)                                          \
    do {                                                                                                           \
        const unsigned ctas = static_cast<unsigned>(ceil_div(total_rows, static_cast<int64_t>(rows_per_cta)));      \
        launch_chained(softmax_offset_row_kernel<T, VPT, GROUP, THREADS, CAUSAL>, ctas, threads, 0, st,             \
            score, qk, ms.mask, ms.q_lens, ms.k_lens, static_cast<uint32_t>(total_rows), static_cast<int>(batch),  \
            static_cast<int>(q_len), static_cast<int>(k_len), InvariantDivisor(static_cast<uint32_t>(q_len)),      \
            InvariantDivisor(static_cast<uint32_t>(heads)), scale);                                                \
        return check_launch("softmax_offset_row_kernel");                                                          \
    } while (0)
            // a warp per row (the per-row set-up is then paid once, not once per warp): up to 8 vectors
            // per lane for fp32, 6 for fp16 (8 fp16 vectors are 64 live values per lane: measured slower)
            if (whole <= (sizeof(T) == 4 ? 256 : 192)) {
                if (whole <= 32) ISPORE_SOFTMAX_OFFSET(1, 32, 256, 8, 256);
                if (whole <= 64) ISPORE_SOFTMAX_OFFSET(2, 32, 256, 8, 256);
                if (whole <= 96) ISPORE_SOFTMAX_OFFSET(3, 32, 256, 8, 256);
                if (whole <= 128) ISPORE_SOFTMAX_OFFSET(4, 32, 256, 8, 256);
                if (whole <= 160) ISPORE_SOFTMAX_OFFSET(5, 32, 128, 4, 128);
                if (whole <= 192) ISPORE_SOFTMAX_OFFSET(6, 32, 128, 4, 128);
                if (whole <= 224) ISPORE_SOFTMAX_OFFSET(7, 32, 128, 4, 128);
                ISPORE_SOFTMAX_OFFSET(8, 32, 128, 4, 128);
            }
            // A CTA per row: among the (vectors per thread, CTA size) pairs whose trips before the last
            // are full for every row, the one with the fewest thread slots after weighting by how
            // well that many vectors per thread ran on B200 (2047 to 8191-long rows: fp16 best at 3
            // vectors = 24 values per thread, fp32 at 4 to 8 = 16 to 32 values).
            int best_vpt = 0, best_threads = 0;
            double best_cost = 1e30;
            for (int vpt : {3, 4, 8, 6, 2, 1}) {
                const int64_t threads = ceil_div(ceil_div(whole, static_cast<int64_t>(vpt)), static_cast<int64_t>(32)) * 32;
                if (threads < 64 || threads > 512 || (vpt - 1) * threads > whole - 1) continue;
                double weight;  // relative speed at equal slot count
                if (sizeof(T) == 2)
                    weight = vpt == 3 ? 1.0 : vpt == 4 ? 0.87 : vpt == 2 ? 0.85 : vpt == 6 ? 0.8 : vpt == 8 ? 0.75 : 0.55;
                else
                    weight = vpt == 4 ? (whole <= 768 ? 1.0 : 0.93) : vpt == 8 ? 0.97 : vpt == 6 ? 0.85 : vpt == 3 ? 0.72 : vpt == 2 ? 0.7 : 0.55;
                const double cost = static_cast<double>(threads * vpt) / weight;
                if (cost < best_cost) {
                    best_cost = cost;
                    best_vpt = vpt;
                    best_threads = static_cast<int>(threads);
                }
            }
            switch (best_vpt) {
                case 1: ISPORE_SOFTMAX_OFFSET(1, 0, 512, 1, best_threads);
                case 2: ISPORE_SOFTMAX_OFFSET(2, 0, 512, 1, best_threads);
                case 3: ISPORE_SOFTMAX_OFFSET(3, 0, 512, 1, best_threads);
                case 4: ISPORE_SOFTMAX_OFFSET(4, 0, 512, 1, best_threads);
                case 6: ISPORE_SOFTMAX_OFFSET(6, 0, 512, 1, best_threads);
                case 8: ISPORE_SOFTMAX_OFFSET(8, 0, 512, 1, best_threads);
                default: break;  // no shape fits: the kernels below take it
            }
#undef ISPORE_SOFTMAX_OFFSET
        }
    }
    if (k_len <= 256 * 16) {
        const unsigned grid = static_cast<unsigned>(total_rows < (1ll << 30) ? total_rows : (1ll << 30));
        if (k_len <= 128 * 4)
            softmax_row_scalar_kernel<T, 128, 4, CAUSAL><<<grid, 128, 0, st>>>(
                score, qk, ms.mask, ms.q_lens, ms.k_lens, total_rows, rows_per_batch, static_cast<int>(q_len),
                static_cast<int>(k_len), scale);
        else if (k_len <= 256 * 8)
            softmax_row_scalar_kernel<T, 256, 8, CAUSAL><<<grid, 256, 0, st>>>(
                score, qk, ms.mask, ms.q_lens, ms.k_lens, total_rows, rows_per_batch, static_cast<int>(q_len),
                static_cast<int>(k_len), scale);
        else
            softmax_row_scalar_kernel<T, 256, 16, CAUSAL><<<grid, 256, 0, st>>>(
                score, qk, ms.mask, ms.q_lens, ms.k_lens, total_rows, rows_per_batch, static_cast<int>(q_len),
                static_cast<int>(k_len), scale);
        return check_launch("softmax_row_scalar_kernel");
    }
    auto generic = softmax_generic_kernel<T, 256, CAUSAL>;
    generic<<<persistent_grid(generic, 256, 0, total_rows, 8), 256, 0, st>>>(
        score, qk, ms.mask, ms.q_lens, ms.k_lens, total_rows, rows_per_batch, static_cast<int>(q_len), k_len, scale);
    return check_launch("softmax_generic_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {
int ispore_scale_mask_softmax_f32(float* attn_score, const float* qk, const float* mask,
                                  int64_t batch_size, int64_t head_num, int64_t q_len, int64_t k_len,
                                  float scale, ispore_stream_t stream) {
    return ispore::softmax_dispatch<float, false>(attn_score, qk, {mask, nullptr, nullptr}, batch_size, head_num,
                                                  q_len, k_len, scale, static_cast<cudaStream_t>(stream));
}
int ispore_scale_mask_softmax_f16(void* attn_score, const void* qk, const void* mask,
                                  int64_t batch_size, int64_t head_num, int64_t q_len, int64_t k_len,
                                  float scale, ispore_stream_t stream) {
    return ispore::softmax_dispatch<__half, false>(static_cast<__half*>(attn_score), static_cast<const __half*>(qk),
                                                   {static_cast<const __half*>(mask), nullptr, nullptr}, batch_size,
                                                   head_num, q_len, k_len, scale, static_cast<cudaStream_t>(stream));
}
int ispore_scale_causal_softmax_f32(float* attn_score, const float* qk, const int32_t* q_lens, const int32_t* k_lens,
                                    int64_t batch_size, int64_t head_num, int64_t q_len, int64_t k_len, float scale,
                                    ispore_stream_t stream) {
    return ispore::softmax_dispatch<float, true>(attn_score, qk, {nullptr, q_lens, k_lens}, batch_size, head_num,
                                                 q_len, k_len, scale, static_cast<cudaStream_t>(stream));
}
int ispore_scale_causal_softmax_f16(void* attn_score, const void* qk, const int32_t* q_lens, const int32_t* k_lens,
                                    int64_t batch_size, int64_t head_num, int64_t q_len, int64_t k_len, float scale,
                                    ispore_stream_t stream) {
    return ispore::softmax_dispatch<__half, true>(static_cast<__half*>(attn_score), static_cast<const __half*>(qk),
                                                  {nullptr, q_lens, k_lens}, batch_size, head_num, q_len, k_len, scale,
                                                  static_cast<cudaStream_t>(stream));
}
}
