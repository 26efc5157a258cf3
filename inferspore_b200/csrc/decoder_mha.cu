// Decode-time fused masked multi-head attention for sm_100a: one new token per sequence.
//
// Reference: src/kernels/fused_decoder_self_attention.cu:112-250 (fp32 kernel), :251-379 (fp16),
// launcher :381-441.  Per (batch b, q head h), with kv head g = h / (heads / kv_heads):
//   q, k, v  <- the token's rows of qkv_buf [bs, heads + 2*kv_heads, d] (+ bias, :163-188)
//   q, k     <- RoPE on adjacent pairs (2i, 2i+1) with angle t / base^(2i / rot_dim) for
//               2i < rot_dim (:57-110); the reference passes t = step
//   cache[layer, b, g, step-1, :] <- k, v                                  (:206-209, :240-243)
//   logit_i  = rsqrt(d) * <q, K_i>,  i < step                              (:210-221)
//   p        = exp(logit - max) / (sum + 1e-6)                             (:224-238)
//   out[b, h, :] = sum_i p_i V_i                                            (:240-249)
// Where this file departs from the reference kernel, on purpose:
//   * the reference softmax only covers the first blockDim.x = d/vec logits (:224-236); here every
//     one of the `step` logits takes part, which is what the reference's CPU function does
//     (tests/unittests/test_fused_decoder_attention.cu:99-110);
//   * the reference's block max is floored at 0 by the padding of its reduction (:52); here the
//     max is the true maximum (again as in its CPU function);
//   * the reference indexes qkv_buf with a batch stride of heads*d (:132, :141), which is only right
//     for one sequence; here the stride is (heads + 2*kv_heads)*d, the tensor's own layout;
//   * fp16 products are accumulated in fp32 (the reference multiplies in half, :337).
//
// Work split: a CTA owns one (b, kv head), up to eight of the q heads that share it, and one chunk
// of the positions (flash-decoding style split so that small batches still fill 148 SMs); the
// cache rows of the chunk are read once for all heads of the group.  The rows reach the CTA
// through a three-deep ring of 16 KB shared-memory tiles filled by TMA bulk copies (K tiles, then
// V tiles, issued three ahead).  With several q heads on half-precision rows of 128 the q.K
// products run on the tensor cores (mma m16n8k16, a cache tile as the A operand without any
// shuffling); otherwise 16 lanes share a row and a halving butterfly sums the partial products.
// With eight q heads the numerators x V product runs there too (V tiles through ldmatrix), on
// eight warps.
// With more than one chunk per (b, head) the CTAs leave (max, sum, unnormalised output) in a
// workspace and a second kernel combines them.
// Measured and not kept: chunks longer than the logits buffer, worked through in passes of 512
// positions inside one CTA with a running maximum (so that a CTA's start and end are paid once
// per 1024-4096 positions and the number of chunks can be fitted to the rounds of resident CTAs).
// The accumulators and the tile bookkeeping that then live across the passes took the
// eight-head variant from 62 to 123 registers; capped at the 85 that three CTAs per SM allow it
// ran at 0.71 of the copy rate against 0.81 at the same 512-position chunk, and longer chunks
// (0.74 at 1024, 0.60 at 4096) did not make up for it.  A fourth ring stage instead of the third
// CTA: 0.66-0.79 against 0.81.
#include <float.h>

#include <algorithm>
#include <cstdint>
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"

namespace ispore {
namespace {

constexpr int kMhaThreads = 128;
constexpr int kMhaWarps = kMhaThreads / 32;
constexpr int kMaxRotPairs = 128;  // head_size <= 256

struct RopeAngles {
    float denom[kMaxRotPairs];  // powf(base, 2i / rot_dim), evaluated on the host
};

template <typename T>
struct MhaParams {
    T* out;            // [bs, heads, d]
    const T* qkv;      // [bs, heads + 2*kv_heads, d]
    const T* bias;     // [(heads + 2*kv_heads) * d] or NULL
    T* k_cache;        // [bs, kv_heads, max_seq_len, d] of the layer
    T* v_cache;
    float* workspace;  // [bs*heads, splits, d + 2] when splits > 1
    int heads, kv_heads, q_per_kv, head_groups;
    int max_seq_len, step, chunk, splits, rot_pairs;
    float rope_t, scale;
};

__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kMhaWarps; ++w) r = fmaxf(r, red[w]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kMhaWarps; ++w) r += red[w];
    __syncthreads();
    return r;
}

// e^x for the softmax numerators: the library function for fp32 rows, the hardware exp2 for half
// rows (its error, about 2^-21 relative, is far below a half's spacing).
template <typename T>
__device__ __forceinline__ float exp_for(float x) { return std::is_same<T, float>::value ? expf(x) : __expf(x); }

// Rounds through the storage type, as the reference does when it keeps q, k, v in T registers.
template <typename T>
__device__ __forceinline__ float round_to(float x) { return to_float<T>(from_float<T>(x)); }

// Sums N per-lane values across the LPK lanes of a group with a halving butterfly: at each
// level a lane keeps one half of its values and hands the other half to its partner, so N
// values cost about N shuffles in total instead of N * log2(LPK).  On return the lane holds
// max(1, N / LPK) finished sums, v[0..], for the value indices base, base + 1, ...; when
// LPK > N the lanes that differ only in their lowest log2(LPK / N) bits hold duplicates.
template <int N, int O>
struct GroupReduce {
    template <int NMAX>
    static __device__ __forceinline__ void run(float (&v)[NMAX], int lk, int& base) {
        if (N > 1) {
            constexpr int kHalf = N > 1 ? N / 2 : 1;
            const bool upper = (lk & O) != 0;
#pragma unroll
            for (int i = 0; i < kHalf; ++i) {
                const float send = upper ? v[i] : v[i + kHalf];
                const float keep = upper ? v[i + kHalf] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, O);
            }
            if (upper) base += kHalf;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], O);
        }
        GroupReduce<(N > 1 ? N / 2 : 1), O / 2>::run(v, lk, base);
    }
};
template <int N>
struct GroupReduce<N, 0> {
    template <int NMAX>
    static __device__ __forceinline__ void run(float (&)[NMAX], int, int&) {}
};

// D += A * B for one m16n8k16 tile: A 16x16 row-major fp16 (four registers of two halves), B 16x8
// column-major fp16 (two registers), fp32 accumulators.  Lane (g = lane / 4, t = lane % 4) holds
//   a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1], a2 = A[g][2t+8, 2t+9], a3 = A[g+8][2t+8, 2t+9],
//   b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g],  d0, d1 = D[g][2t, 2t+1], d2, d3 = D[g+8][2t, 2t+1].
__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four 8x8 fp16 matrices from shared memory, transposed on the way: lane l gives the address of
// row l % 8 of matrix l / 8; lane (g, t) receives M_i[2t][g], M_i[2t+1][g] in r_i.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// LPK lanes share one cache row (d = LPK * elements per 128-bit vector); a CTA works on
// kMhaThreads / LPK rows at a time.  GT q heads of one kv head per CTA.
// STAGED: the cache rows of the chunk do not go from global memory into registers but through a
// ring of kStages shared-memory tiles of kStageRows rows (16 KB), filled by TMA bulk copies that
// one thread issues kStages tiles ahead — first all K tiles, then all V tiles, so V is already
// arriving while the softmax numerators are computed.  The bytes in flight then do not depend on
// registers or on how many CTAs fit, which is what the wider head groups (more registers, fewer
// CTAs per SM) need to reach the memory roofline.
constexpr int kStages = 3;
constexpr int kPvTensorMinGroup = 8;  // q heads per CTA from which numerators x V runs on the tensor cores

// Both products on the tensor cores: half rows of 128, staged tiles, eight q heads per CTA.  That
// kernel runs eight warps instead of four, so that twice as many warps hide each other's latencies
// (q.K split by rows, numerators x V by rows and by halves of d).
template <typename T, int LPK, int GT, bool STAGED>
constexpr bool mha_both_on_tensor_cores() {
    return std::is_same<T, __half>::value && LPK == 16 && STAGED && GT >= kPvTensorMinGroup;
}
template <typename T, int LPK, int GT, bool STAGED>
constexpr int mha_threads() { return mha_both_on_tensor_cores<T, LPK, GT, STAGED>() ? 2 * kMhaThreads : kMhaThreads; }

template <typename T, int LPK, int GT, int U, bool STAGED>
__global__ void __launch_bounds__((mha_threads<T, LPK, GT, STAGED>()))
decoder_mha_kernel(const MhaParams<T> p, const RopeAngles angles, unsigned* __restrict__ status) {
    constexpr int E = VecTraits<T>::kElems;
    constexpr int D = LPK * E;
    constexpr int kThreads = mha_threads<T, LPK, GT, STAGED>();
    constexpr int kWarps = kThreads / 32;
    constexpr int KPI = kMhaThreads / LPK;  // cache rows per iteration of the FMA paths (four warps)
    constexpr int N = GT * U;               // dot products per thread per iteration (U rows in flight)
    constexpr int kStageRows = KPI * U;     // rows per pass of four warps = rows per shared-memory tile
    constexpr int kStageBytes = kStageRows * D * static_cast<int>(sizeof(T));
    static_assert(!STAGED || kStageBytes == 16384, "a staged tile is one pass of eight rows per thread");
    // Tensor-core paths: q.K needs several heads on half rows of 128; numerators x V needs eight.
    constexpr bool kMmaQK = std::is_same<T, __half>::value && LPK == 16 && GT >= 2;
    constexpr bool kMmaPV = mha_both_on_tensor_cores<T, LPK, GT, STAGED>();
    constexpr int kRowBytes = D * static_cast<int>(sizeof(T));
    // A V tile of the tensor-core path lands as eight groups of eight rows, each group 16 bytes
    // further along than rows alone would put it: the eight rows one ldmatrix phase reads are taken
    // one from each group, so they fall into different banks.
    constexpr int kGroupRows = 8;
    constexpr int kGroupBytes = kGroupRows * kRowBytes + (kMmaPV ? 16 : 0);
    constexpr int kStageStride = kMmaPV ? (kStageRows / kGroupRows) * kGroupBytes : kStageBytes;
    __shared__ float q_s[GT][D];
    __shared__ float knew_s[D], vnew_s[D];
    __shared__ float2 cs_s[kMaxRotPairs];
    __shared__ float red_s[kWarps];
    __shared__ float m_s[GT], l_s[GT];
    __shared__ __align__(8) uint64_t full[kStages];
    chain_begin();
    extern __shared__ __align__(128) unsigned char dyn_raw[];  // [tiles when STAGED][logits / output reduction buffer]
    unsigned char* const stage_base = dyn_raw;
    float* const dyn_s = reinterpret_cast<float*>(dyn_raw + (STAGED ? kStages * kStageStride : 0));
    const int lstride = p.chunk + (kMmaPV ? 8 : 0);  // floats between two heads' logits (bank spread)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lk = tid % LPK, ks = tid / LPK;
    const int hg = blockIdx.x % p.head_groups;
    const int bkv = blockIdx.x / p.head_groups;  // b * kv_heads + kv head
    const int b = bkv / p.kv_heads, kvh = bkv - b * p.kv_heads;
    const int h0 = kvh * p.q_per_kv + hg * GT;   // first q head of this CTA
    const int split = blockIdx.y;
    const int s0 = split * p.chunk;
    const int s1 = min(p.step, s0 + p.chunk);
    const int last = p.step - 1;                  // position of the new token
    const bool has_last = last >= s0 && last < s1;
    const int n = s1 - s0;                        // positions of this chunk
    const int n_cache = (has_last ? last : s1) - s0;  // of which read from the cache
    const int64_t cache_row0 = static_cast<int64_t>(bkv) * p.max_seq_len;

    // Tiles 0 .. nt-1 are K rows, nt .. 2nt-1 the same rows of V.
    const int nt = (n_cache + kStageRows - 1) / kStageRows;
    // K tiles (and V tiles of the FMA path) are one contiguous copy issued by thread 0; a V tile
    // of the tensor-core path is one copy per group of rows, issued by threads 0..7.
    int ring_slot = 0;         // stage of the tile consumed next
    uint32_t ring_phase = 0;   // parity its barrier completes with
    auto issue_tile = [&](int tile, int slot) {
        const bool is_v = tile >= nt;
        const int first_row = (is_v ? tile - nt : tile) * kStageRows;
        const int rows = min(kStageRows, n_cache - first_row);
        const uint32_t bytes = static_cast<uint32_t>(rows) * kRowBytes;
        const T* src = (is_v ? p.v_cache : p.k_cache) + (cache_row0 + s0 + first_row) * D;
        uint64_t* bar = &full[slot];
        unsigned char* dst = stage_base + slot * kStageStride;
        if (tid == 0) tma::mbar_arrive_expect_tx(bar, bytes);
        if (kMmaPV && is_v) {
            const int group_rows = min(kGroupRows, rows - tid * kGroupRows);
            if (group_rows > 0)
                tma::load(dst + tid * kGroupBytes, src + tid * kGroupRows * D, group_rows * kRowBytes, bar);
        } else if (tid == 0) {
            tma::load(dst, src, bytes, bar);
        }
    };
    if (STAGED) {
        if (tid == 0) {
#pragma unroll
            for (int st = 0; st < kStages; ++st) tma::mbar_init(&full[st], 1);
            tma::fence_mbar_init();
        }
        if (kMmaPV) __syncthreads();  // other threads issue copies on these barriers too
        if (tid < (kMmaPV ? kStageRows / kGroupRows : 1))
            for (int tile = 0; tile < kStages && tile < 2 * nt; ++tile) issue_tile(tile, tile);
    }
    // Waits for tile `tile`; false when the copy did not land in time (reported at release).
    auto acquire_tile = [&](int tile) -> bool {
        (void)tile;
        return !STAGED || tma::mbar_wait(&full[ring_slot], ring_phase);
    };
    // Every thread is done with tile `tile`: its stage is refilled with tile + kStages.  Returns
    // false (for the whole CTA) when a copy was lost; the caller leaves the kernel.
    auto release_tile = [&](int tile, bool landed) -> bool {
        if (!STAGED) return true;
        if (__syncthreads_or(!landed)) {
            if (tid == 0) {
                atomicOr(status, ISPORE_DEV_TIMEOUT);
                for (int t2 = tile; t2 < tile + kStages && t2 < 2 * nt; ++t2)  // once more for the copies in flight
                    tma::mbar_wait(&full[t2 % kStages], (t2 / kStages) & 1);
            }
            return false;
        }
        if (tid < (kMmaPV ? kStageRows / kGroupRows : 1) && tile + kStages < 2 * nt) issue_tile(tile + kStages, ring_slot);
        if (++ring_slot == kStages) {
            ring_slot = 0;
            ring_phase ^= 1u;
        }
        return true;
    };

    // ---- the new token: bias, RoPE, rounding through T -------------------------------------------
    for (int i = tid; i < p.rot_pairs; i += kThreads) {
        float sn, cs;
        sincosf(p.rope_t / angles.denom[i], &sn, &cs);
        cs_s[i] = make_float2(cs, sn);
    }
    __syncthreads();
    const int qkv_heads = p.heads + 2 * p.kv_heads;
    const T* tok = p.qkv + static_cast<int64_t>(b) * qkv_heads * D;
    const int rope_rows = GT + (has_last ? 1 : 0);  // q heads, then k
    for (int idx = tid; idx < rope_rows * (D / 2); idx += kThreads) {
        const int r = idx / (D / 2), i = idx - r * (D / 2);
        const int row = r < GT ? h0 + r : p.heads + kvh;
        float x0 = to_float<T>(tok[row * D + 2 * i]), x1 = to_float<T>(tok[row * D + 2 * i + 1]);
        if (p.bias != nullptr) {
            x0 = round_to<T>(x0 + to_float<T>(p.bias[row * D + 2 * i]));
            x1 = round_to<T>(x1 + to_float<T>(p.bias[row * D + 2 * i + 1]));
        }
        float y0 = x0, y1 = x1;
        if (i < p.rot_pairs) {
            const float2 c = cs_s[i];
            y0 = round_to<T>(c.x * x0 - c.y * x1);
            y1 = round_to<T>(c.x * x1 + c.y * x0);
        }
        float* dst = r < GT ? q_s[r] : knew_s;
        dst[2 * i] = y0;
        dst[2 * i + 1] = y1;
    }
    if (has_last) {
        const int row = p.heads + p.kv_heads + kvh;
        for (int i = tid; i < D; i += kThreads) {
            float x = to_float<T>(tok[row * D + i]);
            if (p.bias != nullptr) x = round_to<T>(x + to_float<T>(p.bias[row * D + i]));
            vnew_s[i] = x;
        }
    }
    __syncthreads();
    if (has_last && hg == 0) {  // one writer per (b, kv head)
        T* kd = p.k_cache + (cache_row0 + last) * D;
        T* vd = p.v_cache + (cache_row0 + last) * D;
        for (int i = tid; i < D; i += kThreads) {
            kd[i] = from_float<T>(knew_s[i]);
            vd[i] = from_float<T>(vnew_s[i]);
        }
    }

    // ---- logits of the chunk ------------------------------------------------------------------------
    float* logits = dyn_s;  // [GT][chunk]
    // Several q heads on half-precision rows of 128: the dot products go through the tensor cores.
    // A warp takes 16 cache rows as the A tile; the 16-byte chunk a lane loads from rows g and
    // g + 8 already is its A fragment for two k-steps, because the order in which the 128
    // elements of a row are visited is free as long as q is visited in the same order:
    // k-slot (2t, 2t+1) of step (j, s) stands for elements 8(t+4j) + 4s + (0, 1), slot
    // (2t+8, 2t+9) for elements 8(t+4j) + 4s + (2, 3).  q (already rounded to half) is the B
    // tile, one head per column; columns GT..7 are zero.
    if constexpr (kMmaQK) {
        const int g = lane >> 2, t = lane & 3;
        uint32_t bq[4][2][2];  // [j][s][low / high k half]
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int sft = 0; sft < 2; ++sft) {
                const int d0 = 8 * (t + 4 * j) + 4 * sft;
                const float* qrow = q_s[g < GT ? g : 0];
                bq[j][sft][0] = g < GT ? pack_half2(qrow[d0], qrow[d0 + 1]) : 0u;
                bq[j][sft][1] = g < GT ? pack_half2(qrow[d0 + 2], qrow[d0 + 3]) : 0u;
            }
        const uint4* kbase = reinterpret_cast<const uint4*>(p.k_cache) + (cache_row0 + s0) * LPK;
        // Four warps take 16 rows of a tile each; eight warps take 8 each and leave rows 8..15 of
        // their A tile zero (the tensor pipe has time to spare, the issue slots do not).
        constexpr int kRowsPerWarp = kStageRows / kWarps;
        static_assert(kRowsPerWarp == 16 || kRowsPerWarp == 8, "a warp's share of a tile fills an A tile or half of one");
        constexpr bool kTwoRows = kRowsPerWarp == 16;
        for (int tile_row = 0, tile = 0; tile_row < n_cache; tile_row += kStageRows, ++tile) {
            const bool landed = acquire_tile(tile);
            const int l0 = warp * kRowsPerWarp + g, l1 = l0 + 8;  // rows inside the tile
            const int r0 = tile_row + l0, r1 = kTwoRows ? tile_row + l1 : n_cache;
            const uint4* stage_v = reinterpret_cast<const uint4*>(stage_base + ring_slot * kStageStride);
            uint4 a_lo[4], a_hi[4];  // rows g and g + 8 of this warp's share, chunks t + 4j
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a_hi[j] = make_uint4(0, 0, 0, 0);
                if (STAGED) {
                    a_lo[j] = r0 < n_cache ? stage_v[l0 * LPK + t + 4 * j] : make_uint4(0, 0, 0, 0);
                    if (kTwoRows && r1 < n_cache) a_hi[j] = stage_v[l1 * LPK + t + 4 * j];
                } else {
                    a_lo[j] = r0 < n_cache ? ld_stream(kbase + static_cast<int64_t>(r0) * LPK + t + 4 * j) : make_uint4(0, 0, 0, 0);
                    if (kTwoRows && r1 < n_cache) a_hi[j] = ld_stream(kbase + static_cast<int64_t>(r1) * LPK + t + 4 * j);
                }
            }
            if (!release_tile(tile, landed)) return;  // the tile is in registers: its stage can be refilled
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains: half the latency
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                mma_16x8x16(acc, a_lo[j].x, a_hi[j].x, a_lo[j].y, a_hi[j].y, bq[j][0][0], bq[j][0][1]);
                mma_16x8x16(acc2, a_lo[j].z, a_hi[j].z, a_lo[j].w, a_hi[j].w, bq[j][1][0], bq[j][1][1]);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[c] += acc2[c];
            // acc[0], acc[1]: row g, heads 2t, 2t+1; acc[2], acc[3]: row g + 8
            if (2 * t < GT) {
                if (r0 < n_cache) {
                    logits[(2 * t) * lstride + r0] = acc[0] * p.scale;
                    if (2 * t + 1 < GT) logits[(2 * t + 1) * lstride + r0] = acc[1] * p.scale;
                }
                if (kTwoRows && r1 < n_cache) {
                    logits[(2 * t) * lstride + r1] = acc[2] * p.scale;
                    if (2 * t + 1 < GT) logits[(2 * t + 1) * lstride + r1] = acc[3] * p.scale;
                }
            }
        }
    } else {
        float qreg[GT][E];
#pragma unroll
        for (int g = 0; g < GT; ++g)
#pragma unroll
            for (int e = 0; e < E; ++e) qreg[g][e] = q_s[g][lk * E + e];
        const uint4* krows = reinterpret_cast<const uint4*>(p.k_cache) + (cache_row0 + s0) * LPK + lk;
        for (int base = 0, tile = 0; base < n_cache; base += KPI * U, ++tile) {
            const bool landed = acquire_tile(tile);
            const uint4* stage_v = reinterpret_cast<const uint4*>(stage_base + ring_slot * kStageStride);
            uint4 raw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = base + u * KPI + ks;
                if (STAGED)
                    raw[u] = i < n_cache ? stage_v[(u * KPI + ks) * LPK + lk] : make_uint4(0, 0, 0, 0);
                else
                    raw[u] = i < n_cache ? ld_stream(krows + static_cast<int64_t>(i) * LPK) : make_uint4(0, 0, 0, 0);
            }
            if (!release_tile(tile, landed)) return;  // the tile is in registers: its stage can be refilled
            float dots[N];  // index g * U + u
#pragma unroll
            for (int u = 0; u < U; ++u) {
                Unpacked<T> kf;
                unpack(raw[u], kf);
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    float dot = 0.f;
#pragma unroll
                    for (int e = 0; e < E; ++e) dot = fmaf(qreg[g][e], kf.v[e], dot);
                    dots[g * U + u] = dot;
                }
            }
            int first = 0;
            GroupReduce<N, LPK / 2>::run(dots, lk, first);
            constexpr int kHeld = N > LPK ? N / LPK : 1;   // finished sums per lane
            constexpr int kDup = LPK > N ? LPK / N : 1;    // lanes holding the same sum
            if ((lk & (kDup - 1)) == 0) {
#pragma unroll
                for (int j = 0; j < kHeld; ++j) {
                    const int idx = first + j, g = idx / U, u = idx % U;
                    const int i = base + u * KPI + ks;
                    if (i < n_cache) logits[g * lstride + i] = dots[j] * p.scale;
                }
            }
        }
    }
    if (has_last && warp == 0) {  // the new token's own logit, from shared memory
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float dot = 0.f;
            for (int i = lane; i < D; i += 32) dot = fmaf(q_s[g][i], knew_s[i], dot);
            dot = warp_sum(dot);
            if (lane == 0) logits[g * lstride + (last - s0)] = dot * p.scale;
        }
    }
    __syncthreads();

    // ---- softmax numerators over the chunk ----------------------------------------------------------
    if constexpr (GT % kWarps == 0) {
        // a warp per head (two when eight heads share the rows): warp reductions only, no block
        // barrier until all heads are done
        for (int hh = warp; hh < GT; hh += kWarps) {
            float* row = logits + hh * lstride;  // 16-byte aligned: chunk and the row pad are multiples of 4 floats
            const int n4 = n & ~3;
            float mx = -FLT_MAX;
            for (int i = 4 * lane; i < n4; i += 128) {
                const float4 v = *reinterpret_cast<const float4*>(row + i);
                mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
            }
            for (int i = n4 + lane; i < n; i += 32) mx = fmaxf(mx, row[i]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int i = 4 * lane; i < n4; i += 128) {
                float4 v = *reinterpret_cast<const float4*>(row + i);
                v.x = exp_for<T>(v.x - mx);
                v.y = exp_for<T>(v.y - mx);
                v.z = exp_for<T>(v.z - mx);
                v.w = exp_for<T>(v.w - mx);
                *reinterpret_cast<float4*>(row + i) = v;
                sum += (v.x + v.y) + (v.z + v.w);
            }
            for (int i = n4 + lane; i < n; i += 32) {
                const float e = exp_for<T>(row[i] - mx);
                row[i] = e;
                sum += e;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                m_s[hh] = mx;
                l_s[hh] = sum;
            }
        }
    } else {
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float* row = logits + g * lstride;
            float mx = -FLT_MAX;
            for (int i = tid; i < n; i += kThreads) mx = fmaxf(mx, row[i]);
            mx = block_max(mx, red_s);
            float sum = 0.f;
            for (int i = tid; i < n; i += kThreads) {
                const float e = exp_for<T>(row[i] - mx);
                row[i] = e;
                sum += e;
            }
            sum = block_sum(sum, red_s);  // its barriers also publish the numerators
            if (tid == 0) {
                m_s[g] = mx;
                l_s[g] = sum;
            }
        }
    }
    __syncthreads();

    // ---- numerators x V ----------------------------------------------------------------------------------
    float* part = dyn_s;  // [four partial sums][GT][D] once every thread is done with the numerators
    if constexpr (kMmaPV) {
        // out^T [d x heads] = V^T [d x keys] * P^T [keys x heads] on the tensor cores.  Warp w takes
        // the 16 rows of key group w % 4 and half w / 4 of d: ldmatrix (transposing) turns the rows
        // into the A fragments of its four 16-wide blocks of d.  The numerators (fp32, at most 1)
        // go in as the B operand split into a half and the half of the remainder, so the products
        // carry about 22 bits of p.
        static_assert(kWarps == 8, "two warps per key group");
        constexpr int kBlocks = 4;  // 16-wide blocks of d per warp
        const int g = lane >> 2, t = lane & 3;
        const int kg = warp & 3, dh = warp >> 2;
        float acc[kBlocks][4];
#pragma unroll
        for (int blk = 0; blk < kBlocks; ++blk)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[blk][c] = 0.f;
        // Which rows of the tile a key group takes is free as long as the numerators follow: k-slot
        // s (0..7) stands for tile row 8s + 2 kg, slot 8 + s for row 8s + 2 kg + 1, so the eight
        // rows of every 8x8 matrix come from the eight groups of the tile.
        auto tile_offset = [&](int row) { return (row >> 3) * kGroupBytes + (row & 7) * kRowBytes; };
        const int ld_row = 8 * (lane & 7) + 2 * kg + ((lane >> 4) & 1);                          // the row this lane addresses
        const int ld_off = tile_offset(ld_row) + ((lane >> 3) & 1) * 16 + dh * kBlocks * 32;     // and its columns
        const int p_row = 16 * t + 2 * kg;  // rows p_row, +1 (slots 2t, 2t+8) and p_row + 8, +9 (slots 2t+1, 2t+9)
        for (int base = 0, tile = nt; base < n_cache; base += kStageRows, ++tile) {
            const bool landed = acquire_tile(tile);
            unsigned char* stage = stage_base + ring_slot * kStageStride;
            const int rows_valid = min(kStageRows, n_cache - base);
            const bool compute = landed && 2 * kg < rows_valid;
            uint32_t a[kBlocks][4], bh[2] = {0u, 0u}, bl[2] = {0u, 0u};
            if (compute) {
                if (rows_valid < kStageRows) {  // this warp's rows and columns past the end of the chunk hold stale bytes
                    for (int idx = lane; idx < 16 * (LPK / 2); idx += 32) {
                        const int slot = idx / (LPK / 2), r = 8 * (slot & 7) + 2 * kg + (slot >> 3);
                        if (r >= rows_valid)
                            *reinterpret_cast<uint4*>(stage + tile_offset(r) + (dh * (LPK / 2) + idx % (LPK / 2)) * 16) =
                                make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
                if (g < GT) {
                    const float* prow = logits + g * lstride + base + p_row;
                    const bool full = p_row + 9 < rows_valid;
                    float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);  // rows (p_row, +1), (p_row + 8, +9)
                    if (full) {
                        lo = *reinterpret_cast<const float2*>(prow);
                        hi = *reinterpret_cast<const float2*>(prow + 8);
                    } else {
                        if (p_row < rows_valid) lo.x = prow[0];
                        if (p_row + 1 < rows_valid) lo.y = prow[1];
                        if (p_row + 8 < rows_valid) hi.x = prow[8];
                        if (p_row + 9 < rows_valid) hi.y = prow[9];
                    }
                    // register 0: slots 2t, 2t+1 = rows p_row, p_row + 8; register 1: slots 2t+8, 2t+9
                    const __half2 h0 = __floats2half2_rn(lo.x, hi.x), h1 = __floats2half2_rn(lo.y, hi.y);
                    const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
                    bh[0] = *reinterpret_cast<const uint32_t*>(&h0);
                    bh[1] = *reinterpret_cast<const uint32_t*>(&h1);
                    bl[0] = pack_half2(lo.x - b0.x, hi.x - b0.y);
                    bl[1] = pack_half2(lo.y - b1.x, hi.y - b1.y);
                }
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk) ldmatrix_x4_trans(a[blk], stage + ld_off + blk * 32);
            }
            if (!release_tile(tile, landed)) return;  // the tile is in registers: its stage can be refilled
            if (compute) {
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk)
                    mma_16x8x16(acc[blk], a[blk][0], a[blk][1], a[blk][2], a[blk][3], bh[0], bh[1]);
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk)
                    mma_16x8x16(acc[blk], a[blk][0], a[blk][1], a[blk][2], a[blk][3], bl[0], bl[1]);
            }
        }
        // acc[blk][0], [1]: d = d_first + 16 blk + g, heads 2t, 2t+1; [2], [3]: the same d + 8
        const int ha = 2 * t, hb = 2 * t + 1;
        const int d_first = dh * kBlocks * 16;
        if (has_last && kg == 0) {
            const float wa = ha < GT ? logits[ha * lstride + (last - s0)] : 0.f;
            const float wb = hb < GT ? logits[hb * lstride + (last - s0)] : 0.f;
#pragma unroll
            for (int blk = 0; blk < kBlocks; ++blk) {
                const float v0 = vnew_s[d_first + 16 * blk + g], v1 = vnew_s[d_first + 16 * blk + g + 8];
                acc[blk][0] = fmaf(wa, v0, acc[blk][0]);
                acc[blk][1] = fmaf(wb, v0, acc[blk][1]);
                acc[blk][2] = fmaf(wa, v1, acc[blk][2]);
                acc[blk][3] = fmaf(wb, v1, acc[blk][3]);
            }
        }
        __syncthreads();  // every thread is done with the numerators: the buffer becomes [key groups][GT][D]
#pragma unroll
        for (int blk = 0; blk < kBlocks; ++blk) {
            const int dd = d_first + 16 * blk + g;
            if (ha < GT) {
                part[(kg * GT + ha) * D + dd] = acc[blk][0];
                part[(kg * GT + ha) * D + dd + 8] = acc[blk][2];
            }
            if (hb < GT) {
                part[(kg * GT + hb) * D + dd] = acc[blk][1];
                part[(kg * GT + hb) * D + dd + 8] = acc[blk][3];
            }
        }
    } else {
        float acc[GT][E];
#pragma unroll
        for (int g = 0; g < GT; ++g)
#pragma unroll
            for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
        const uint4* vrows = reinterpret_cast<const uint4*>(p.v_cache) + (cache_row0 + s0) * LPK + lk;
        for (int base = 0, tile = nt; base < n_cache; base += KPI * U, ++tile) {
            const bool landed = acquire_tile(tile);
            const uint4* stage_v = reinterpret_cast<const uint4*>(stage_base + ring_slot * kStageStride);
            uint4 raw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = base + u * KPI + ks;
                if (STAGED)
                    raw[u] = i < n_cache ? stage_v[(u * KPI + ks) * LPK + lk] : make_uint4(0, 0, 0, 0);
                else
                    raw[u] = i < n_cache ? ld_stream(vrows + static_cast<int64_t>(i) * LPK) : make_uint4(0, 0, 0, 0);
            }
            if (!release_tile(tile, landed)) return;  // the tile is in registers: its stage can be refilled
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = base + u * KPI + ks;
                Unpacked<T> vf;
                unpack(raw[u], vf);
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    const float w = i < n_cache ? logits[g * lstride + i] : 0.f;
#pragma unroll
                    for (int e = 0; e < E; ++e) acc[g][e] = fmaf(w, vf.v[e], acc[g][e]);
                }
            }
        }
        if (has_last && ks == 0) {
#pragma unroll
            for (int g = 0; g < GT; ++g) {
                const float w = logits[g * lstride + (last - s0)];
#pragma unroll
                for (int e = 0; e < E; ++e) acc[g][e] = fmaf(w, vnew_s[lk * E + e], acc[g][e]);
            }
        }
        // rows held by the other lane groups of this warp, then by the other warps
#pragma unroll
        for (int g = 0; g < GT; ++g)
#pragma unroll
            for (int e = 0; e < E; ++e)
#pragma unroll
                for (int o = LPK; o < 32; o <<= 1) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        __syncthreads();  // every thread is done with the numerators: the buffer becomes [warps][GT][D]
        constexpr int kLanesUsed = LPK < 32 ? LPK : 32;  // lanes 0..LPK-1 of a warp hold its sums
        if (lane < kLanesUsed) {
#pragma unroll
            for (int g = 0; g < GT; ++g)
#pragma unroll
                for (int e = 0; e < E; ++e) part[(warp * GT + g) * D + lane * E + e] = acc[g][e];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < GT * D; idx += kThreads) {
        const int g = idx / D, dd = idx - g * D;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kMhaWarps; ++w) o += part[(w * GT + g) * D + dd];  // four partial sums in either variant
        const int64_t bh = static_cast<int64_t>(b) * p.heads + h0 + g;
        if (p.splits == 1) {
            p.out[bh * D + dd] = from_float<T>(o / (l_s[g] + 1e-6f));
        } else {
            float* ws = p.workspace + (bh * p.splits + split) * (D + 2);
            ws[2 + dd] = o;
            if (dd == 0) {
                ws[0] = m_s[g];
                ws[1] = l_s[g];
            }
        }
    }
}

// Merges the chunks of one (b, head): out = sum_s e^(m_s - M) O_s / (sum_s e^(m_s - M) l_s + 1e-6).
template <typename T>
__global__ void __launch_bounds__(128)
decoder_mha_combine_kernel(T* __restrict__ out, const float* __restrict__ workspace, int splits, int head_size) {
    chain_begin();
    const int64_t bh = blockIdx.x;
    const float* ws = workspace + bh * splits * (head_size + 2);
    float mx = -FLT_MAX;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, ws[s * (head_size + 2)]);
    float denom = 0.f;
    for (int s = 0; s < splits; ++s) denom += expf(ws[s * (head_size + 2)] - mx) * ws[s * (head_size + 2) + 1];
    const float inv = 1.0f / (denom + 1e-6f);
    for (int dd = threadIdx.x; dd < head_size; dd += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s)
            o = fmaf(expf(ws[s * (head_size + 2)] - mx), ws[s * (head_size + 2) + 2 + dd], o);
        out[bh * head_size + dd] = from_float<T>(o * inv);
    }
}

constexpr int kChunkFloatsDefault = 8192;    // logits floats per CTA without opting in to large shared memory
constexpr int kChunkFloatsMax = 40960;       // with the opt-in (160 KB)

// q heads of one kv head per CTA.  Eight only where both products run on the tensor cores (half
// rows of 128); with FMA products a group of eight is bound by instruction issue.
int pick_group(int64_t q_per_kv, bool tensor_cores) {
    int cap = tune(kTuneMhaGroup, 8);
    if (tune(kTuneMhaStaged, 1) == 0 && cap > 4) cap = 4;  // the register-staged comparison variant has no group of eight
    for (int g : {8, 4, 2})
        if (g <= cap && q_per_kv % g == 0 && (g < 8 || tensor_cores)) return g;
    return 1;
}

// Positions per chunk and number of chunks for one (b, kv head, head group).
void plan_chunks(int64_t batch, int64_t heads, int64_t kv_heads, int64_t step, bool have_workspace, int gt,
                 int* chunk, int* splits) {
    const int64_t base_ctas = batch * kv_heads * (heads / kv_heads / gt);
    int64_t want = 1;
    if (have_workspace) {
        // The tile ring keeps every CTA's reads in flight on its own, so a CTA takes a long chunk
        // (1024 positions) whenever that still gives every SM one; smaller batches get as many
        // chunks as reach two CTAs per SM, down to 128 positions each.
        const int sms = sm_count() > 0 ? sm_count() : 148;
        const int64_t enough = static_cast<int64_t>(tune(kTuneMhaCtasPerSm, 1)) * sms;
        // (512 with eight heads per CTA: their numerators then leave room for three CTAs per SM)
        const int64_t big = tune(kTuneMhaChunk, gt >= 8 ? 512 : 1024), small = 128;
        want = ceil_div(step, big);
        if (base_ctas * want < enough) want = std::min(ceil_div(2 * enough, base_ctas), std::max<int64_t>(1, step / small));
        want = std::max<int64_t>(want, ceil_div(step, static_cast<int64_t>(kChunkFloatsDefault / gt)));
    }
    int64_t c = ceil_div(step, want);
    c = ceil_div(c, static_cast<int64_t>(32)) * 32;
    *chunk = static_cast<int>(c);
    *splits = static_cast<int>(ceil_div(step, c));
}

template <typename T, int LPK, int GT, int U, bool STAGED>
int launch_mha(const MhaParams<T>& p, const RopeAngles& angles, int64_t batch, cudaStream_t st) {
    constexpr int D = LPK * VecTraits<T>::kElems;
    auto kernel = decoder_mha_kernel<T, LPK, GT, U, STAGED>;
    constexpr bool kPadded = STAGED && std::is_same<T, __half>::value && LPK == 16 && GT >= kPvTensorMinGroup;  // the kernel's kMmaPV
    const size_t floats = std::max<size_t>(static_cast<size_t>(GT) * (p.chunk + (kPadded ? 8 : 0)),
                                           static_cast<size_t>(kMhaWarps) * GT * D);
    const size_t stage = 16384 + (kPadded ? 8 * 16 : 0);
    const size_t smem = floats * sizeof(float) + (STAGED ? static_cast<size_t>(kStages) * stage : 0);
    if (!allow_dynamic_smem(kernel, smem))
        return fail(ISPORE_ELAUNCH, "decoder_masked_mha: %zu bytes of shared memory refused", smem);
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "decoder_masked_mha: no device status word");
    dim3 grid(static_cast<unsigned>(batch * p.kv_heads * p.head_groups), static_cast<unsigned>(p.splits));
    launch_chained(kernel, grid, mha_threads<T, LPK, GT, STAGED>(), smem, st, p, angles, status);
    int rc = check_launch("decoder_mha_kernel");
    if (rc != ISPORE_OK || p.splits == 1) return rc;
    launch_chained(decoder_mha_combine_kernel<T>, static_cast<unsigned>(batch * p.heads), 128, 0, st, p.out, p.workspace,
                   p.splits, D);
    return check_launch("decoder_mha_combine_kernel");
}

template <typename T, int LPK>
int launch_mha_group(const MhaParams<T>& p, const RopeAngles& angles, int gt, int64_t batch, cudaStream_t st) {
#ifdef ISPORE_TUNING
    if (tune(kTuneMhaStaged, 1) == 0) {  // the register-staged variant, kept for comparison
        switch (gt) {
            case 4: return launch_mha<T, LPK, 4, 8, false>(p, angles, batch, st);
            case 2: return launch_mha<T, LPK, 2, 8, false>(p, angles, batch, st);
            default: return launch_mha<T, LPK, 1, 8, false>(p, angles, batch, st);
        }
    }
#endif
    if constexpr (std::is_same<T, __half>::value && LPK == 16)
        if (gt == 8) return launch_mha<T, LPK, 8, 8, true>(p, angles, batch, st);
    switch (gt) {
        case 4: return launch_mha<T, LPK, 4, 8, true>(p, angles, batch, st);
        case 2: return launch_mha<T, LPK, 2, 8, true>(p, angles, batch, st);
        default: return launch_mha<T, LPK, 1, 8, true>(p, angles, batch, st);
    }
}

template <typename T>
int mha_dispatch(T* out, const T* qkv, const T* bias, T* k_cache, T* v_cache, int64_t layer, int64_t num_layers,
                 int64_t batch, int64_t heads, int64_t kv_heads, int64_t max_seq_len, int64_t head_size, int64_t step,
                 int32_t rot_dim, float rope_base, float rope_timestep, void* workspace, int64_t workspace_bytes,
                 cudaStream_t st) {
    constexpr int E = VecTraits<T>::kElems;
    if (batch < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || max_seq_len <= 0 || head_size <= 0 ||
        step <= 0 || step > max_seq_len || layer < 0 || (num_layers > 0 && layer >= num_layers) ||
        batch * heads > INT32_MAX || max_seq_len > INT32_MAX)
        return fail(ISPORE_ESHAPE, "decoder_masked_mha: bad shape bs=%lld heads=%lld/%lld step=%lld/%lld layer=%lld/%lld",
                    (long long)batch, (long long)heads, (long long)kv_heads, (long long)step, (long long)max_seq_len,
                    (long long)layer, (long long)num_layers);
    const int64_t lpk = head_size / E;
    if (head_size % E != 0 || lpk > 32 || (lpk & (lpk - 1)) != 0)
        return fail(ISPORE_ESHAPE, "decoder_masked_mha: head size %lld must be %d x a power of two up to 32",
                    (long long)head_size, E);
    if (rot_dim < 0 || rot_dim % 2 != 0 || rot_dim / 2 > kMaxRotPairs)
        return fail(ISPORE_ESHAPE, "decoder_masked_mha: rotary dim %d", rot_dim);
    if (batch == 0) return ISPORE_OK;
    if (!out || !qkv || !k_cache || !v_cache) return fail(ISPORE_ENULL, "decoder_masked_mha: NULL buffer");
    if (!aligned16(k_cache) || !aligned16(v_cache)) return fail(ISPORE_EALIGN, "decoder_masked_mha: caches must be 16-byte aligned");

    MhaParams<T> p;
    const int gt = pick_group(heads / kv_heads, std::is_same<T, __half>::value && lpk == 16);
    int chunk = 0, splits = 1;
    plan_chunks(batch, heads, kv_heads, step, workspace != nullptr, gt, &chunk, &splits);
    const int64_t need = splits > 1 ? batch * heads * splits * (head_size + 2) * static_cast<int64_t>(sizeof(float)) : 0;
    if (need > workspace_bytes || (splits > 1 && (reinterpret_cast<uintptr_t>(workspace) & 3) != 0)) {
        // workspace too small for the plan: fall back to one chunk per (b, head) if shared memory can hold it
        plan_chunks(batch, heads, kv_heads, step, false, gt, &chunk, &splits);
    }
    if (static_cast<int64_t>(chunk) * gt > kChunkFloatsMax)
        return fail(ISPORE_ESCRATCH, "decoder_masked_mha: step %lld needs a workspace of %lld bytes",
                    (long long)step, (long long)ispore_decoder_masked_mha_workspace_bytes(batch, heads, kv_heads, head_size, step));
    const int64_t layer_offset = layer * batch * kv_heads * max_seq_len * head_size;
    p.out = out;
    p.qkv = qkv;
    p.bias = bias;
    p.k_cache = k_cache + layer_offset;
    p.v_cache = v_cache + layer_offset;
    p.workspace = static_cast<float*>(workspace);
    p.heads = static_cast<int>(heads);
    p.kv_heads = static_cast<int>(kv_heads);
    p.q_per_kv = static_cast<int>(heads / kv_heads);
    p.head_groups = p.q_per_kv / gt;
    p.max_seq_len = static_cast<int>(max_seq_len);
    p.step = static_cast<int>(step);
    p.chunk = chunk;
    p.splits = splits;
    p.rot_pairs = static_cast<int>(std::min<int64_t>(rot_dim, head_size) / 2);
    p.rope_t = rope_timestep;
    p.scale = 1.0f / sqrtf(static_cast<float>(head_size));
    RopeAngles angles;
    for (int i = 0; i < p.rot_pairs; ++i)
        angles.denom[i] = powf(rope_base, static_cast<float>(2 * i) / static_cast<float>(rot_dim));
    switch (lpk) {
        case 32: return launch_mha_group<T, 32>(p, angles, gt, batch, st);
        case 16: return launch_mha_group<T, 16>(p, angles, gt, batch, st);
        case 8: return launch_mha_group<T, 8>(p, angles, gt, batch, st);
        case 4: return launch_mha_group<T, 4>(p, angles, gt, batch, st);
        case 2: return launch_mha_group<T, 2>(p, angles, gt, batch, st);
        default: return launch_mha_group<T, 1>(p, angles, gt, batch, st);
    }
}

}  // namespace
}  // namespace ispore

extern "C" {

int64_t ispore_decoder_masked_mha_workspace_bytes(int64_t batch_size, int64_t head_num, int64_t kv_head_num,
                                                  int64_t head_size, int64_t step) {
    if (batch_size <= 0 || head_num <= 0 || kv_head_num <= 0 || head_num % kv_head_num != 0 || head_size <= 0 || step <= 0)
        return 0;
    // The plan depends on the head group, which depends on the element type: enough for either.
    int64_t bytes = 0;
    for (bool tensor_cores : {false, true}) {
        int chunk = 0, splits = 1;
        const int gt = ispore::pick_group(head_num / kv_head_num, tensor_cores && head_size == 128);
        ispore::plan_chunks(batch_size, head_num, kv_head_num, step, true, gt, &chunk, &splits);
        if (splits > 1)
            bytes = std::max(bytes, batch_size * head_num * splits * (head_size + 2) * static_cast<int64_t>(sizeof(float)));
    }
    return bytes;
}

int ispore_decoder_masked_mha_f32(float* mha_output, const float* qkv_buf, const float* qkv_bias, float* k_cache,
                                  float* v_cache, int64_t layer, int64_t num_layers, int64_t batch_size,
                                  int64_t head_num, int64_t kv_head_num, int64_t max_seq_len, int64_t head_size,
                                  int64_t step, int32_t rotary_embedding_dim, float rotary_embedding_base,
                                  float rope_timestep, void* workspace, int64_t workspace_bytes,
                                  ispore_stream_t stream) {
    return ispore::mha_dispatch<float>(mha_output, qkv_buf, qkv_bias, k_cache, v_cache, layer, num_layers, batch_size,
                                       head_num, kv_head_num, max_seq_len, head_size, step, rotary_embedding_dim,
                                       rotary_embedding_base, rope_timestep, workspace, workspace_bytes,
                                       static_cast<cudaStream_t>(stream));
}

int ispore_decoder_masked_mha_f16(void* mha_output, const void* qkv_buf, const void* qkv_bias, void* k_cache,
                                  void* v_cache, int64_t layer, int64_t num_layers, int64_t batch_size,
                                  int64_t head_num, int64_t kv_head_num, int64_t max_seq_len, int64_t head_size,
                                  int64_t step, int32_t rotary_embedding_dim, float rotary_embedding_base,
                                  float rope_timestep, void* workspace, int64_t workspace_bytes,
                                  ispore_stream_t stream) {
    return ispore::mha_dispatch<__half>(static_cast<__half*>(mha_output), static_cast<const __half*>(qkv_buf),
                                        static_cast<const __half*>(qkv_bias), static_cast<__half*>(k_cache),
                                        static_cast<__half*>(v_cache), layer, num_layers, batch_size, head_num,
                                        kv_head_num, max_seq_len, head_size, step, rotary_embedding_dim,
                                        rotary_embedding_base, rope_timestep, workspace, workspace_bytes,
                                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
