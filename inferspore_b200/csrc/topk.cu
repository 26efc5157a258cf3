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
// Round 1 (one CTA per row slice) streams its slice from HBM once, in passes of 64 KB
// — two tiles of 8192 fp32 elements or four of fp16, 64 or 128 elements per
// thread (TMA bulk copies into a shared-memory ring that holds a pass, the next
// tiles requested as soon as every thread has read this pass's).  First pass: a threshold that is
// guaranteed to keep at least K elements comes from one representative per
// thread: every warp sorts its 32 with a shuffle network and contributes its
// best few, and the K-th largest contribution is the threshold.  The few
// survivors are compacted into shared memory, a warp at a time, and ranked by
// counting against each other, which yields the running top-K already sorted.
// Every later pass only has to beat the running K-th best: while that is a
// positive value the test is one integer compare of the thread's maximum and
// one vote per warp; the few survivors are parked behind the running best and
// ranked before the next pass is touched, so the bar rises as early as
// possible.  A later pass costs one block barrier, plus one for its ranking
// when it had survivors.  (The code calls a pass a "round".)
// Adversarial tiles (e.g. constant data, where the threshold keeps everything)
// fall back to an exact radix select over the tile, ties resolved by an
// index-ordered block scan.  Round 2 (one CTA per row) merges the slices' sorted
// lists by binary search and can draw the sampled token in its epilogue.
#include <float.h>
#include <limits.h>
#include <math.h>

#include <mutex>

#include "common.cuh"
#include "tma.cuh"

namespace ispore {
namespace {

#ifdef ISPORE_TUNING
__device__ int g_topk_debug = 0;  // ablation switches, tuning builds only
__device__ long long g_topk_ts[64];  // clock64() of CTA 0 at marked points, tuning builds only
#define TOPK_DEBUG(bit) (g_topk_debug & (bit))
#define TOPK_MARK(i) do { if (blockIdx.x == 0 && threadIdx.x == 0 && (i) < 64) g_topk_ts[i] = clock64(); } while (0)
#else
#define TOPK_DEBUG(bit) false
#define TOPK_MARK(i) do { } while (0)
#endif

constexpr int kTopkThreads = 256;  // measured: 512 threads x 16 keys is 1.5x slower (barriers over 16 warps)
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kElemsPerThread = 32;                          // elements of a tile a thread looks at
constexpr int kTileElems = kTopkThreads * kElemsPerThread;   // 8192
constexpr int kMaxStages = 8;                                // tiles of the shared-memory ring
// Tiles a CTA thresholds, compacts and ranks together: 64 KB of the row, i.e. 64 fp32 or 128 fp16
// elements per thread (measured for fp16 against two tiles per round: [256, 32000] 12.2 -> 9.5 us,
// 4096 rows 100 -> 89 us, [256, 128256] 31.7 -> 26.3 us).
template <typename T>
constexpr int round_tiles() { return sizeof(T) == 2 ? 4 : 2; }
constexpr int kTileCap = 256;                                // survivors a round may add on the fast path
constexpr int kCandSlots = ISPORE_TOPK_MAX_K + kTileCap;     // running best + a round's survivors
constexpr int kWarpVecCap = 64;                              // vectors with survivors a warp lists per round
constexpr int kMergeCap = 4096;                              // lists*K candidates the merge kernel holds

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

// Bitonic networks over one warp.  Element i of a sequence of 32 R values sits in register i / 32
// of lane i % 32; exchanges across a distance below 32 are shuffles, the others stay inside a lane.
// Every loop unrolls, so the network is straight-line code.
// (Measured and not kept: ranking the candidates of a tile — 64-bit composites, up to 128 — with
// these networks in a single warp instead of the counting rank of the whole CTA below.  It
// executes a fifth fewer instructions over the kernel and is slower at every row count, 8 to 25 %:
// two dozen dependent exchanges in one warp against independent counting loops in eight.)
template <typename V, int R>
__device__ __forceinline__ void bitonic_phase(V (&a)[R], int k) {  // merges runs of k / 2 into runs of k
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 16 * R; j > 0; j >>= 1) {
        if (j >= k) continue;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const bool desc = ((r * 32 + lane) & k) == 0;  // the last phase (k = 32 R) is descending everywhere
            if (j >= 32) {
                const int rp = r ^ (j >> 5);
                if (rp > r && ((a[r] < a[rp]) == desc)) {
                    const V t = a[r];
                    a[r] = a[rp];
                    a[rp] = t;
                }
            } else {
                const V p = __shfl_xor_sync(0xffffffffu, a[r], j);
                const bool take_max = ((lane & j) == 0) == desc;
                a[r] = ((a[r] > p) == take_max) ? a[r] : p;
            }
        }
    }
}
// Sorts the 32 R values best (largest) first.
template <typename V, int R>
__device__ __forceinline__ void warp_sort_desc(V (&a)[R]) {
#pragma unroll
    for (int k = 2; k <= 32 * R; k <<= 1) bitonic_phase<V, R>(a, k);
}

// The q largest (q <= 32) of the 32 lane values, best first, to out[0..q) (0 where fewer than q
// lanes are non-empty): one 32-value sorting network, 15 exchanges whatever q.  Returns the q-th
// largest to every lane.
__device__ __forceinline__ uint32_t warp_top_q(uint32_t v, int q, uint32_t* out) {
    const int lane = threadIdx.x & 31;
    uint32_t a[1] = {v};
    warp_sort_desc<uint32_t, 1>(a);
    if (lane < q) out[lane] = a[0];
    return __shfl_sync(0xffffffffu, a[0], q - 1);
}

// Number of entries of a descending-sorted composite list that are greater than x.
__device__ __forceinline__ int count_greater(const unsigned long long* list, int len, unsigned long long x) {
    int lo = 0, hi = len;  // invariant: list[0..lo) > x, list[hi..len) <= x
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (list[mid] > x) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// Ranks the `total` distinct composites in `in` against each other; those with rank < K land
// at out[rank].  in[0..nsorted) is already sorted (best first): an entry of that prefix starts
// from its own position, any other entry from a binary search in the prefix, and only the
// unsorted tail in[nsorted..total) is compared one by one.  Threads are split P per candidate
// (P a power of two) so that short lists still use the whole CTA.
__device__ __forceinline__ void rank_into(const unsigned long long* in, int nsorted, int total, int K,
                                          unsigned long long* out) {
    int P = 1, shift = 0;
    while (P < 32 && total * (P * 2) <= kTopkThreads) {
        P *= 2;
        ++shift;
    }
    const int part = threadIdx.x & (P - 1);
    for (int c0 = 0; c0 < total; c0 += kTopkThreads >> shift) {
        const int c = c0 + (threadIdx.x >> shift);
        const bool live = c < total;
        const unsigned long long mine = live ? in[c] : 0ull;
        int rank = 0;
        if (live) {
            if (part == 0) rank = c < nsorted ? c : count_greater(in, nsorted, mine);
#pragma unroll 4
            for (int j = nsorted + part; j < total; j += P) rank += in[j] > mine;
        }
        for (int o = 1; o < P; o <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
        if (live && part == 0 && rank < K) out[rank] = mine;
    }
}

// A thread looks at 32 elements of a tile, as kElemsPerThread / E groups of E consecutive ones
// (one 128-bit vector each): group k of thread t is vector (t + k*256) of the tile.  It keeps
// only the maximum of every group, as raw fp32 bit patterns viewed as signed ints, and their
// maximum pmax; a slot beyond the slice counts as INT_MIN.  For non-negative floats (NaNs
// included) signed-int order of the bits IS the output order, so as long as the threshold is a
// positive float "does this group hold a survivor" is one integer compare, and only the (rare)
// groups that do are read again — from the shared-memory stage or the cache — to be pushed.
// pmax is a real element of the thread (the true maximum whenever the thread holds a
// non-negative value), which is all the threshold derivation of the first tile needs.
template <typename T>
__device__ __forceinline__ void group_maxima_from_global(const T* src, int n, int tile_begin, bool vec_loads,
                                                         int (&gmax)[kElemsPerThread / VecTraits<T>::kElems], int& pmax) {
    constexpr int E = VecTraits<T>::kElems;
    constexpr int kVecs = kElemsPerThread / E;
    pmax = INT_MIN;
    if (vec_loads) {
        uint4 raw[kVecs];
        const uint4* src_v = reinterpret_cast<const uint4*>(src + tile_begin);
#pragma unroll
        for (int k = 0; k < kVecs; ++k) {
            const int v = threadIdx.x + k * kTopkThreads;
            // L1-allocating load: the few survivors are re-read below and should hit L1.
            if (tile_begin + v * E < n) raw[k] = ld_keep(src_v + v);  // n % E == 0 on this path
        }
#pragma unroll
        for (int k = 0; k < kVecs; ++k) {
            const int v = threadIdx.x + k * kTopkThreads;
            gmax[k] = INT_MIN;
            if (tile_begin + v * E < n) {
                Unpacked<T> x;
                unpack(raw[k], x);
#pragma unroll
                for (int e = 0; e < E; ++e) gmax[k] = max(gmax[k], __float_as_int(x.v[e]));
            }
            pmax = max(pmax, gmax[k]);
        }
    } else {
#pragma unroll
        for (int k = 0; k < kVecs; ++k) {
            const int v = threadIdx.x + k * kTopkThreads;
            gmax[k] = INT_MIN;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const int i = tile_begin + v * E + e;
                if (i < n) gmax[k] = max(gmax[k], __float_as_int(to_float<T>(src[i])));
            }
            pmax = max(pmax, gmax[k]);
        }
    }
}

// Exact selection of a tile's K largest keys, for tiles the threshold cannot thin out
// (constant data, K close to the tile size): radix select, 8 bits per pass, then an
// index-ordered block scan that hands the tied key to the lowest indices.  Writes the tile's
// min(K, elements) best composites to `mine` and returns how many.  Kept out of line, and re-reading the tile from global memory (it is
// cache-resident) instead of taking the caller's registers, so that it costs the fast path
// neither registers nor stack traffic.
struct SelectScratch {
    int* hist;      // [256]
    int* warp_cnt;  // [kTopkWarps]
    int* s_count;
    int* s_digit;
    int* s_need;
};
template <typename T>
__device__ __noinline__ int exact_select_tile(const T* src, int tile_begin, int n, long long begin, int K,
                                              unsigned long long* mine, SelectScratch sm) {
    const int tid = threadIdx.x;
    int* hist = sm.hist;
    int* warp_cnt = sm.warp_cnt;
    int& s_count = *sm.s_count;
    int& s_digit = *sm.s_digit;
    int& s_need = *sm.s_need;
    int tile_end = tile_begin + kTileElems;
    if (tile_end > n) tile_end = n;
    auto key_at = [&](int el) { return order_key(to_float<T>(src[el])); };

    uint32_t prefix = 0, prefix_mask = 0;
    const int wanted = tile_end - tile_begin < K ? tile_end - tile_begin : K;
    int need = wanted;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int el = tile_begin + tid; el < tile_end; el += kTopkThreads) {
            const uint32_t key = key_at(el);
            if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
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
    // keys > prefix: all of them (fewer than K); keys == prefix: the `need` lowest indices.
    if (tid == 0) s_count = 0;
    __syncthreads();
    for (int el = tile_begin + tid; el < tile_end; el += kTopkThreads) {
        const uint32_t key = key_at(el);
        if (key > prefix) mine[atomicAdd(&s_count, 1)] = composite(key, static_cast<uint32_t>(begin + el));
    }
    __syncthreads();
    const int greater = s_count;
    int taken = 0;
    for (int base = tile_begin; base < tile_end && taken < need; base += kTopkThreads) {  // uniform trip count
        const int el = base + tid;
        const bool tie = el < tile_end && key_at(el) == prefix;
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
        if (tie && ordinal < need) mine[greater + ordinal] = composite(prefix, static_cast<uint32_t>(begin + el));
        taken += total;
        __syncthreads();
    }
    return wanted;
}

// exp((v - v0)/T) in index order, inverse CDF on a caller-drawn uniform.  One warp; `cum` is K
// floats of shared memory.  The lanes evaluate the exponentials, lane 0 turns them into running
// sums one after the other — the sequential fp32 sums of the definition, p_0 + p_1 + ... in index
// order (an empty slot contributes an exact zero) — and the lanes then look for the smallest valid
// index whose running sum reaches u * total.
template <typename T>
__device__ __forceinline__ void sample_row(const int32_t* ids, const T* vals, int K, float u,
                                           float temperature, float* cum, int32_t* out) {
    const int lane = threadIdx.x & 31;
    const float v0 = to_float<T>(vals[0]);
    for (int i = lane; i < K; i += 32)
        cum[i] = ids[i] < 0 ? 0.f : expf((to_float<T>(vals[i]) - v0) / temperature);
    __syncwarp();
    if (lane == 0) {
        float run = 0.f;
        for (int i = 0; i < K; ++i) {
            run += cum[i];
            cum[i] = run;
        }
    }
    __syncwarp();
    const float target = u * cum[K - 1];
    int pick = INT_MAX, last = -1;
    for (int i = lane; i < K; i += 32) {
        if (ids[i] >= 0) {
            last = i;
            if (cum[i] >= target && i < pick) pick = i;
        }
    }
    pick = __reduce_min_sync(0xffffffffu, pick);
    last = __reduce_max_sync(0xffffffffu, last);
    if (pick == INT_MAX) pick = last;  // nothing reached the target (rounding): the last valid slot
    if (lane == 0) *out = pick >= 0 ? ids[pick] : -1;
}

// TMA: the tiles arrive through the copy engine (cp.async.bulk into a ring of `nstages`
// shared-memory stages, completion on one mbarrier per stage).  The whole ring is requested at
// the start, and once every thread has read the tiles of a round their stages are refilled, so
// the next tiles are on their way while this round is ranked.  The registers are filled from
// shared memory.  Needs the vector-load conditions (16-byte aligned rows, slice length a multiple
// of the vector) and a ring that holds a round.  Without TMA the tiles are loaded straight into
// registers.
template <typename T, int MIN_BLOCKS, bool TMA>
__global__ void __launch_bounds__(kTopkThreads, MIN_BLOCKS)
topk_slice_kernel(const T* __restrict__ probs, int64_t vocab, int slice_len, int slices, int K,
                  int32_t* __restrict__ out_ids_base, T* __restrict__ out_vals_base, int out_lists,
                  int32_t index_offset, int vec_loads, int nstages, unsigned* __restrict__ status,
                  const float* __restrict__ uniform, float temperature, int32_t* __restrict__ sampled_ids) {
    constexpr int E = VecTraits<T>::kElems;
    constexpr int kVecs = kElemsPerThread / E;
    constexpr int kRoundTiles = round_tiles<T>();
    extern __shared__ __align__(128) unsigned char stage_raw[];  // TMA: [nstages][kTileElems * sizeof(T)]
    __shared__ __align__(8) uint64_t full[kMaxStages];
    __shared__ unsigned long long cand[2][kCandSlots];  // [cur]: running best, then the round's survivors
    __shared__ uint32_t warp_thr[kTopkWarps];
    __shared__ int s_count;
    __shared__ int s_push[4];
    __shared__ int s_timeout;
    __shared__ int hist[256];
    __shared__ int s_digit, s_need;
    __shared__ int warp_cnt[kTopkWarps];
    chain_begin();
    TOPK_MARK(0);

    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x / slices;
    const int slice = static_cast<int>(blockIdx.x - row * slices);
    const int64_t begin = static_cast<int64_t>(slice) * slice_len;
    int64_t n64 = vocab - begin;
    if (n64 > slice_len) n64 = slice_len;
    const int n = n64 > 0 ? static_cast<int>(n64) : 0;
    const T* src = probs + row * vocab + begin;
    // (requested now, needed at the very end: its DRAM latency would otherwise sit on the row's critical path)
    const float u_row = (uniform != nullptr && tid < 32) ? __ldg(uniform + row) : 0.f;

    if (tid < 4) s_push[tid] = 0;  // visible before its first use: every kind of round has a barrier before the next round

    int cur = 0;    // which cand[] buffer holds the running best
    int nbest = 0;  // entries of the running best (sorted, best first)
    const int q = (K + kTopkWarps - 1) / kTopkWarps;
    const int ntiles = (n + kTileElems - 1) / kTileElems;
    const int nrounds = (ntiles + kRoundTiles - 1) / kRoundTiles;

    constexpr uint32_t kStageBytes = kTileElems * sizeof(T);
    auto tile_bytes = [&](int tile_begin) {
        const int left = n - tile_begin;
        return static_cast<uint32_t>(left < kTileElems ? left : kTileElems) * static_cast<uint32_t>(sizeof(T));
    };
    // Tile t lives in stage t % nstages and completes its barrier with parity (t / nstages) & 1.
    auto stage_of = [&](int tile) {
        return reinterpret_cast<const T*>(stage_raw + static_cast<size_t>(tile % nstages) * kStageBytes);
    };
    auto issue_tile = [&](int tile) {  // thread 0 only
        const int stage = tile % nstages;
        const int tile_begin = tile * kTileElems;
        tma::mbar_arrive_expect_tx(&full[stage], tile_bytes(tile_begin));
        tma::load(stage_raw + static_cast<size_t>(stage) * kStageBytes, src + tile_begin, tile_bytes(tile_begin), &full[stage]);
    };
    if (TMA) {
        if (tid == 0) {
            // The whole ring is requested before the other threads have even arrived: the wait for
            // the first tiles is the longest stall of a row.
            for (int st = 0; st < nstages; ++st) tma::mbar_init(&full[st], 1);
            tma::fence_mbar_init();
            s_timeout = 0;
            for (int tile = 0; tile < nstages && tile < ntiles; ++tile) issue_tile(tile);
        }
        __syncthreads();  // the barriers' initialisation is visible to every thread that will wait on them
    }

    // A round takes kRoundTiles tiles at once — 64 KB of the row — through threshold,
    // compaction and ranking: those steps depend on each other and on two block barriers, and a row
    // is a chain of them, so half as many rounds is what shortens a row (measured at 256 and 4096
    // rows x 32000 against one tile per round: see the dispatcher).
    // Streamed rounds count their survivors in s_push[round & 3]: the count of round r is read by
    // everyone after the barrier of round r+1 while round r+1 already counts in the next slot, and
    // the slot is cleared again two rounds later, so no thread reads a counter that another is
    // still adding to.
    bool streamed_prev = false;  // the previous round's survivors are parked behind the running best, not yet ranked
    uint32_t thr = 0;
    // A bounded wait on a tile ran out somewhere in the CTA: record it, wait once more for the copies
    // in flight (shared memory must not be released under them) and leave; every thread comes here.
    auto timed_out = [&](int first_tile) {
        if (tid == 0) {
            atomicOr(status, ISPORE_DEV_TIMEOUT);
            for (int t2 = first_tile; t2 < first_tile + nstages && t2 < ntiles; ++t2)  // the round's tiles and those already requested
                tma::mbar_wait(&full[t2 % nstages], static_cast<uint32_t>(t2 / nstages) & 1u);
        }
    };
    // Every thread has read the tiles of the round that starts at `first_tile` (a barrier has
    // passed): their stages take the tiles one ring further on.
    auto refill = [&](int first_tile) {
        if (TMA && tid == 0) {
            for (int t2 = first_tile + nstages; t2 < first_tile + kRoundTiles + nstages && t2 < ntiles; ++t2) issue_tile(t2);
        }
    };
    // Ranks the running best together with the first `count` entries behind it; afterwards the
    // (sorted) best is in the other buffer.  Called by every thread; ends with a barrier.
    auto rank_pending = [&](int count) {
        const int total = nbest + count;
        rank_into(cand[cur], nbest, total, K, cand[cur ^ 1]);
        cur ^= 1;
        nbest = total < K ? total : K;
        __syncthreads();
        if (nbest == K) {
            const uint32_t kth = static_cast<uint32_t>(cand[cur][K - 1] >> 32);
            thr = kth == 0xffffffffu ? kth : kth + 1u;  // a later element must beat the K-th best outright
        }
    };
    // The survivors of the round that starts at `first_tile` did not fit behind the running best:
    // each of its tiles is selected exactly (from global memory: the stages may be refilled by now)
    // and ranked.
    auto overflow_round = [&](int first_tile) {
        for (int t2 = first_tile; t2 < first_tile + kRoundTiles && t2 < ntiles; ++t2) {
            const int got = exact_select_tile<T>(src, t2 * kTileElems, n, begin, K, cand[cur] + nbest,
                                                 SelectScratch{hist, warp_cnt, &s_count, &s_digit, &s_need});
            __syncthreads();
            rank_pending(got);
        }
    };

    // Takes in the survivors the previous (streamed) round parked behind the running best and ranks
    // them at once: the sooner the K-th best rises, the fewer elements of the following rounds
    // survive, and a ranking costs (K + survivors) x survivors comparisons.  Measured and not kept:
    // parking the survivors of several rounds and ranking them together (5x the comparisons), and
    // taking a fixed threshold from the first tile with ONE ranking at the end of the row (a row
    // whose first tile misleads needs a second pass, and with hundreds of rows per launch some row
    // always does).  A round that overflowed its room is selected exactly.  Runs at the top of an
    // iteration, after the barrier that ended the previous one, while no tile is held in registers.
    auto settle_previous = [&](int prev_round) {
        const int added = s_push[prev_round & 3];
        if (added > kTileCap) {
            overflow_round(prev_round * kRoundTiles);
        } else if (added > 0) {
            rank_pending(added);
        }
    };

    for (int round = 0; round < nrounds; ++round) {
        const int t0 = round * kRoundTiles;
        TOPK_MARK(1 + round * 6);  // top of the iteration
        if (tid == 0) s_push[(round + 1) & 3] = 0;  // that slot was read for the last time two rounds ago
        if (streamed_prev) settle_previous(round - 1);
        streamed_prev = false;
        TOPK_MARK(2 + round * 6);  // previous round settled

        // Group maxima: gmax[h * kVecs + k] covers vector tid + k * 256 of tile t0 + h.
        int gmax[kRoundTiles * kVecs];
        int pmax = INT_MIN;
#pragma unroll
        for (int h = 0; h < kRoundTiles; ++h) {
            const int tile = t0 + h;
            const int tile_begin = tile * kTileElems;
            if (tile >= ntiles) {  // uniform: the slice ends with half a round
#pragma unroll
                for (int k = 0; k < kVecs; ++k) gmax[h * kVecs + k] = INT_MIN;
                continue;
            }
            if (TMA) {
                // A wait that runs out is recorded here and acted on by the whole CTA after the next
                // barrier (whatever was read meanwhile is discarded).
                if (!tma::mbar_wait(&full[tile % nstages], static_cast<uint32_t>(tile / nstages) & 1u)) s_timeout = 1;
                const uint4* stage_v = reinterpret_cast<const uint4*>(stage_of(tile));
                const bool whole_tile = tile_begin + kTileElems <= n;  // uniform: no per-vector guards then
#pragma unroll
                for (int k = 0; k < kVecs; ++k) {
                    const int v = tid + k * kTopkThreads;
                    int g = INT_MIN;
                    if (whole_tile || tile_begin + v * E < n) {
                        Unpacked<T> x;
                        unpack(stage_v[v], x);
#pragma unroll
                        for (int e = 0; e < E; ++e) g = max(g, __float_as_int(x.v[e]));
                    }
                    gmax[h * kVecs + k] = g;
                    pmax = max(pmax, g);
                }
            } else {
                int part[kVecs];
                int part_max;
                group_maxima_from_global<T>(src, n, tile_begin, vec_loads != 0, part, part_max);
#pragma unroll
                for (int k = 0; k < kVecs; ++k) gmax[h * kVecs + k] = part[k];
                pmax = max(pmax, part_max);
            }
        }
        TOPK_MARK(3 + round * 6);  // tiles landed and read
        // Survivors: the elements whose key reaches `limit`, pushed behind the running best from
        // position base + (their share of `counter`), dropped beyond kTileCap (the counter still
        // counts them, which is how the overflow is noticed).
        auto push_survivors = [&](uint32_t limit, int base, int* counter) {
            unsigned long long* mine = cand[cur] + nbest;
            if (TOPK_DEBUG(16)) return;
            if (limit > 0x80000000u) {
                // A positive limit: survivors are exactly the elements whose raw bits, as signed ints,
                // reach its bits.  pmax and one vote clear a warp without survivors.  Otherwise the
                // warp works as one: the lanes note which of their vectors hold a survivor in a
                // short per-warp list (positions from votes, no atomics), then lane l looks at
                // element l % E of listed vector l / E — 32 elements per trip, read again from the
                // stage — and the survivors among them take consecutive slots behind the running
                // best through one shared-memory atomic per trip.  (A thread walking its own groups
                // instead costs the warp the union of all its lanes' walks, with an atomic in each;
                // a warp walking its holder threads one by one, 32 elements each, was measured 25 %
                // slower over the whole kernel: a dozen dependent trips instead of one or two.)
                const int limit_bits = static_cast<int>(limit & 0x7fffffffu);
                if (__ballot_sync(0xffffffffu, pmax >= limit_bits) == 0) return;
                const int lane = tid & 31;
                const uint32_t below = (1u << lane) - 1u;
                uint16_t* wlist = reinterpret_cast<uint16_t*>(hist) + (tid >> 5) * kWarpVecCap;
                int nv = 0;
#pragma unroll
                for (int g = 0; g < kRoundTiles * kVecs; ++g) {
                    const bool holds = gmax[g] >= limit_bits;  // a group beyond the slice is INT_MIN
                    const uint32_t votes = __ballot_sync(0xffffffffu, holds);
                    const int at = nv + __popc(votes & below);
                    // (which tile of the round) << 11 | vector within the tile
                    if (holds && at < kWarpVecCap)
                        wlist[at] = static_cast<uint16_t>(((g / kVecs) << 11) | (tid + (g % kVecs) * kTopkThreads));
                    nv += __popc(votes);
                }
                if (nv > kWarpVecCap) {  // more than the list holds: the round is selected exactly
                    if (lane == 0) atomicAdd(counter, kTileCap + 1);
                    return;
                }
                __syncwarp();
                const int sub = lane / E, e = lane % E;
                for (int j0 = 0; j0 < nv; j0 += 32 / E) {
                    const int j = j0 + sub;
                    int bits = INT_MIN, el = 0;
                    if (j < nv) {
                        const int entry = wlist[j];
                        const int tile = t0 + (entry >> 11);
                        el = tile * kTileElems + (entry & 2047) * E + e;  // within the slice
                        if (TMA) bits = __float_as_int(to_float<T>(stage_of(tile)[el - tile * kTileElems]));
                        else if (el < n) bits = __float_as_int(to_float<T>(__ldg(src + el)));
                    }
                    const bool in = bits >= limit_bits;
                    const uint32_t votes = __ballot_sync(0xffffffffu, in);
                    if (votes == 0) continue;
                    int first = 0;
                    if (lane == 0) first = atomicAdd(counter, __popc(votes));
                    first = __shfl_sync(0xffffffffu, first, 0);
                    const int pos = base + first + __popc(votes & below);
                    if (in && pos < kTileCap)
                        mine[pos] = composite(static_cast<uint32_t>(bits) | 0x80000000u, static_cast<uint32_t>(begin + el));
                }
                return;
            }
            // Zero or negative limit (fewer than K positive values so far): every group is read
            // again by its own thread and compared through the order key.
#pragma unroll 1
            for (int g = 0; g < kRoundTiles * kVecs; ++g) {
                const int tile = t0 + g / kVecs;
                const int v = tid + (g % kVecs) * kTopkThreads;
                const int el0 = tile * kTileElems + v * E;
                if (el0 >= n) continue;
                float val[E];
                uint32_t live = 0;  // which of the group's elements exist
                if (TMA || vec_loads) {  // whole vectors only on these paths (n % E == 0)
                    Unpacked<T> x;
                    unpack(TMA ? reinterpret_cast<const uint4*>(stage_of(tile))[v] : ld_keep(reinterpret_cast<const uint4*>(src + el0)), x);
#pragma unroll
                    for (int e = 0; e < E; ++e) val[e] = x.v[e];
                    live = (1u << E) - 1u;
                } else {
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        val[e] = 0.f;
                        if (el0 + e < n) {
                            val[e] = to_float<T>(src[el0 + e]);
                            live |= 1u << e;
                        }
                    }
                }
                uint32_t m = 0;
#pragma unroll
                for (int e = 0; e < E; ++e) m |= (order_key(val[e]) >= limit ? 1u : 0u) << e;
                m &= live;
                if (m != 0) {
                    int pos = base + atomicAdd(counter, __popc(m));
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        if ((m >> e) & 1u) {
                            if (pos < kTileCap) mine[pos] = composite(order_key(val[e]), static_cast<uint32_t>(begin + el0 + e));
                            ++pos;
                        }
                    }
                }
            }
        };

        if (nbest < K) {
            // Fewer than K entries are held (the first round; later ones only in tiny slices).  Every
            // warp contributes its q = ceil(K / 8) largest thread representatives: 8q distinct elements
            // of the round, of which the K-th largest is the threshold — at least K elements have a
            // key >= it, and it sits far higher than the smallest of the 8q (the q-th best of the
            // weakest warp), and the ranking that follows costs survivors squared.  The survivors
            // are ranked at once.
            const bool any_live = t0 * kTileElems + tid * E < n;  // the thread's first group exists
            uint32_t* reps = reinterpret_cast<uint32_t*>(hist);  // [8][q] best first per warp
            const uint32_t wq = warp_top_q(any_live ? order_key(__int_as_float(pmax)) : 0u, q, reps + (tid >> 5) * q);
            if ((tid & 31) == 0) warp_thr[tid >> 5] = wq;
            if (tid == 0) s_count = 0;
            __syncthreads();
            if (TMA && s_timeout) return timed_out(t0);
            const int nreps = kTopkWarps * q;
            if (nreps > K) {
                // (uniform) The K-th largest representative, ties by position: every representative
                // is ranked by as many threads as the CTA affords, each counting a share of the others.
                int P = 1, shift = 0;
                while (P < 32 && nreps * (P * 2) <= kTopkThreads) {
                    P *= 2;
                    ++shift;
                }
                const int r = tid >> shift, part = tid & (P - 1);
                const bool live = r < nreps;  // nreps <= 256: one trip
                const uint32_t mine = live ? reps[r] : 0u;
                int rank = 0;
                if (live) {
#pragma unroll 4
                    for (int j = part; j < nreps; j += P) {
                        const uint32_t other = reps[j];
                        rank += (other > mine || (other == mine && j < r)) ? 1 : 0;
                    }
                }
                for (int o = 1; o < P; o <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
                if (live && part == 0 && rank == K - 1) warp_thr[0] = mine;
                __syncthreads();
            }
            uint32_t first_thr = warp_thr[0];
            if (nreps <= K) {  // every representative is needed: the smallest one
#pragma unroll
                for (int w = 1; w < kTopkWarps; ++w) first_thr = min(first_thr, warp_thr[w]);
            }
            TOPK_MARK(4 + round * 6);  // threshold known
            push_survivors(first_thr, 0, &s_count);
            __syncthreads();
            TOPK_MARK(5 + round * 6);  // survivors pushed
            refill(t0);
            const int count = s_count;
            if (count > kTileCap) {
                overflow_round(t0);
            } else {
                rank_pending(count);
            }
            TOPK_MARK(6 + round * 6);  // first round ranked
            continue;
        }

        // Streamed round: K entries are held, an element only matters if it beats the current K-th
        // best outright (on a tie the earlier index, already held, wins).  Survivors are parked
        // behind the running best and ranked at the top of the next iteration.
        push_survivors(thr, 0, &s_push[round & 3]);
        streamed_prev = true;
        __syncthreads();  // the tiles have been read and their survivors counted by every thread
        TOPK_MARK(5 + round * 6);  // survivors pushed
        if (TMA && s_timeout) return timed_out(t0);
        refill(t0);
    }
    const int tile_no = nrounds;
    TOPK_MARK(40);
    if (streamed_prev) settle_previous(tile_no - 1);
    TOPK_MARK(41);
    // The lists come straight from the sorted composites in shared memory: the id is the low word,
    // the value's bits follow from the order key (exactly, except that both zeros share a key — a
    // zero is read again from the row so that -0.0 keeps its sign).
    int32_t* out_ids = out_ids_base + (row * out_lists + slice) * K;
    T* out_vals = out_vals_base + (row * out_lists + slice) * K;
    const unsigned long long* best = cand[cur];
    auto value_of = [&](unsigned long long c) {  // the float whose order key is the composite's high word
        const uint32_t key = static_cast<uint32_t>(c >> 32);
        return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
    };
    // (Written by the last warps first: the first warp goes straight on to the sampling.)
    for (int s = kTopkThreads - 1 - tid; s < K; s += kTopkThreads) {
        if (s < nbest) {
            const uint32_t idx = ~static_cast<uint32_t>(best[s]);
            out_ids[s] = static_cast<int32_t>(idx) + index_offset;
            const float v = value_of(best[s]);
            out_vals[s] = v == 0.0f ? src[static_cast<int64_t>(idx) - begin] : from_float<T>(v);
        } else {
            out_ids[s] = -1;
            out_vals[s] = neg_inf<T>();
        }
    }
    TOPK_MARK(42);  // lists written
    // With one slice per row the list just written is the final one: sample from it here instead
    // of in a launch of its own (uniform is NULL whenever there are several slices).  Same
    // arithmetic as sample_row, on the values recovered from the keys.
    if (uniform != nullptr && tid < 32) {
        const int lane = tid;
        const int valid = nbest;  // slots nbest..K-1 are empty
        const float v0 = valid > 0 ? value_of(best[0]) : 0.f;
        int pick = INT_MAX;
        if (valid <= 64) {
            // Two terms per lane in registers; the running sum is carried by every lane and fed one
            // term at a time by a shuffle from the lane that holds it (the sequential fp32 sums of the
            // definition, without a chain of dependent shared-memory accesses); lane i % 32 keeps the
            // sum after term i.
            const float p0 = lane < valid ? expf((value_of(best[lane]) - v0) / temperature) : 0.f;
            const float p1 = lane + 32 < valid ? expf((value_of(best[lane + 32]) - v0) / temperature) : 0.f;
            float c0 = 0.f, c1 = 0.f, run = 0.f;
            const int first = valid < 32 ? valid : 32;
#pragma unroll 8
            for (int i = 0; i < first; ++i) {
                run += __shfl_sync(0xffffffffu, p0, i);
                if (lane == i) c0 = run;
            }
#pragma unroll 8
            for (int i = 0; i < valid - 32; ++i) {
                run += __shfl_sync(0xffffffffu, p1, i);
                if (lane == i) c1 = run;
            }
            const float target = u_row * run;  // every valid term has been added: run is the total
            if (lane < valid && c0 >= target) pick = lane;
            else if (lane + 32 < valid && c1 >= target) pick = lane + 32;
        } else {
            float* cum = reinterpret_cast<float*>(hist);
            for (int i = lane; i < valid; i += 32) cum[i] = expf((value_of(best[i]) - v0) / temperature);
            __syncwarp();
            if (lane == 0) {
                float run = 0.f;
#pragma unroll 8
                for (int i = 0; i < valid; ++i) {
                    run += cum[i];
                    cum[i] = run;
                }
            }
            __syncwarp();
            const float target = u_row * cum[valid - 1];
            for (int i = lane; i < valid; i += 32)
                if (cum[i] >= target && i < pick) pick = i;
        }
        pick = __reduce_min_sync(0xffffffffu, pick);
        if (pick == INT_MAX) pick = valid - 1;  // nothing reached the target (rounding): the last valid slot
        if (lane == 0)
            sampled_ids[row] = pick >= 0 ? static_cast<int32_t>(~static_cast<uint32_t>(best[pick])) + index_offset : -1;
    }
    TOPK_MARK(43);  // sampled
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
topk_merge_kernel(const int32_t* __restrict__ cand_ids, const T* __restrict__ cand_vals, int lists, int K,
                  int64_t id_list_stride, int64_t id_row_stride, int64_t val_list_stride, int64_t val_row_stride,
                  int32_t* __restrict__ final_ids, T* __restrict__ final_vals, const float* __restrict__ uniform,
                  float temperature, int32_t* __restrict__ sampled_ids) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* comp = reinterpret_cast<unsigned long long*>(smem_raw);  // [lists*K]
    __shared__ int32_t fin_ids[ISPORE_TOPK_MAX_K];
    __shared__ T fin_vals[ISPORE_TOPK_MAX_K];
    __shared__ float p_smem[ISPORE_TOPK_MAX_K];
    chain_begin();

    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x;
    const int total = lists * K;
    // Entry k of list a of this row sits at a * list_stride + k behind the row's base: lists of a
    // row next to each other ([rows, lists, K], the slice kernel's scratch) or one block per list
    // ([lists, rows, K], what an all-gather of per-rank results leaves behind).
    const int32_t* ids = cand_ids + row * id_row_stride;
    const T* vals = cand_vals + row * val_row_stride;
    auto id_at = [&](int c) { const int a = c / K; return ids[a * id_list_stride + (c - a * K)]; };
    auto val_at = [&](int c) { const int a = c / K; return vals[a * val_list_stride + (c - a * K)]; };

    for (int c = tid; c < total; c += kTopkThreads) {
        const int32_t id = id_at(c);
        comp[c] = id < 0 ? 0ull : composite(order_key(to_float<T>(val_at(c))), static_cast<uint32_t>(id));
    }
    for (int s = tid; s < K; s += kTopkThreads) {
        fin_ids[s] = -1;
        fin_vals[s] = neg_inf<T>();
    }
    __syncthreads();
    // Lists produced by the slice kernel are sorted (best first, empties last).  Check it
    // rather than trust it: unsorted input takes the all-pairs ranking instead.
    int unsorted = 0;
    for (int c = tid; c < total; c += kTopkThreads)
        if (c % K != 0 && comp[c] > comp[c - 1]) unsorted = 1;
    unsorted = __syncthreads_or(unsorted);

    for (int c = tid; c < total; c += kTopkThreads) {
        const unsigned long long mine = comp[c];
        if (mine == 0ull) continue;
        int rank = 0;
        if (!unsorted) {
            const int a = c / K;
            rank = c - a * K;  // entries ahead of it in its own list
            for (int b = 0; b < lists; ++b)
                if (b != a) rank += count_greater(comp + b * K, K, mine);
        } else {
            for (int j = 0; j < total; ++j) rank += comp[j] > mine;
        }
        if (rank < K) {
            fin_ids[rank] = id_at(c);
            fin_vals[rank] = val_at(c);
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
    chain_begin();
    const int warp = threadIdx.x >> 5;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTopkWarps + warp;
    if (row >= rows) return;  // whole warps leave; no block barrier follows
    sample_row<T>(topk_ids + row * K, topk_vals + row * K, K, uniform[row], temperature, p_smem[warp], output_ids + row);
}

int check_k(const char* who, int32_t K) {
    if (K < 1 || K > ISPORE_TOPK_MAX_K) return fail(ISPORE_ELIMIT, "%s: K=%d outside [1,%d]", who, K, ISPORE_TOPK_MAX_K);
    return ISPORE_OK;
}

template <typename T>
int sampling_dispatch(const int32_t* ids, const T* vals, const float* uniform, int32_t* out, int64_t rows,
                      int32_t K, float temperature, cudaStream_t st) {
    if (int rc = check_k("sampling", K)) return rc;
    if (rows < 0) return fail(ISPORE_ESHAPE, "sampling: rows=%lld", (long long)rows);
    if (!(temperature > 0.f)) return fail(ISPORE_ESHAPE, "sampling: temperature must be > 0");
    if (rows == 0) return ISPORE_OK;
    if (!ids || !vals || !uniform || !out) return fail(ISPORE_ENULL, "sampling: NULL buffer");
    launch_chained(sampling_kernel<T>, static_cast<int>(ceil_div(rows, kTopkWarps)), kTopkThreads, 0, st,
        ids, vals, uniform, out, rows, K, temperature);
    return check_launch("sampling_kernel");
}

template <typename T>
int merge_dispatch(const int32_t* cand_ids, const T* cand_vals, int64_t rows, int32_t lists, int32_t K,
                   int64_t id_list_stride, int64_t id_row_stride, int64_t val_list_stride, int64_t val_row_stride,
                   int32_t* final_ids, T* final_vals, const float* uniform, float temperature, int32_t* sampled_ids,
                   cudaStream_t st) {
    if (int rc = check_k("topk_merge", K)) return rc;
    if (rows < 0 || lists < 1 || rows > INT32_MAX) return fail(ISPORE_ESHAPE, "topk_merge: rows=%lld lists=%d", (long long)rows, lists);
    if (id_list_stride < 0 || id_row_stride < 0 || val_list_stride < 0 || val_row_stride < 0)
        return fail(ISPORE_ESHAPE, "topk_merge: negative stride");
    if (static_cast<int64_t>(lists) * K > kMergeCap)
        return fail(ISPORE_ELIMIT, "topk_merge: lists*K=%lld > %d", (long long)lists * K, kMergeCap);
    if (uniform != nullptr && !(temperature > 0.f)) return fail(ISPORE_ESHAPE, "topk_merge: temperature must be > 0");
    if (rows == 0) return ISPORE_OK;
    if (!cand_ids || !cand_vals || !final_ids || !final_vals) return fail(ISPORE_ENULL, "topk_merge: NULL buffer");
    if (uniform != nullptr && sampled_ids == nullptr) return fail(ISPORE_ENULL, "topk_merge: uniform given without sampled_ids");
    const size_t smem = static_cast<size_t>(lists) * K * sizeof(unsigned long long);
    launch_chained(topk_merge_kernel<T>, static_cast<int>(rows), kTopkThreads, smem, st, cand_ids, cand_vals, lists, K,
                   id_list_stride, id_row_stride, val_list_stride, val_row_stride, final_ids, final_vals, uniform,
                   temperature, sampled_ids);
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
    if (uniform != nullptr && !(temperature > 0.f)) return fail(ISPORE_ESHAPE, "topk: temperature must be > 0");
    if (rows == 0) return ISPORE_OK;
    if (!probs || !final_ids || !final_vals) return fail(ISPORE_ENULL, "topk: NULL buffer");
    if (uniform != nullptr && sampled_ids == nullptr) return fail(ISPORE_ENULL, "topk: uniform given without sampled_ids");

    constexpr int E = VecTraits<T>::kElems;
    const int variant = tune(kTuneTopk, 0);
    const bool have_scratch = scratch_ids != nullptr && scratch_vals != nullptr && scratch_slices >= 1;
    const int vec_loads = (vocab % E == 0) && aligned16(probs);
    const bool use_tma = vec_loads && !(variant & 1);
    // The tile ring: 64 KB, one round, three CTAs per SM.  A row is a chain of dependent steps
    // (tiles, threshold, survivors, rank, next tiles ...): what shortens it is fewer, larger rounds,
    // and what a launch of more rows than the GPU holds at once needs is rows in flight.  Measured
    // and not kept: deeper rings at fewer CTAs per SM, slower at every row count; four CTAs per SM
    // on a 32 KB ring (a gain while a round was one tile, none against 64 KB rounds); and one
    // CTA per resident slot walking the rows
    // b, b + grid, ... with the next row's first tiles requested during the current row's last
    // ranking (4096 rows: 124 us against 115 us — the rows a static stride hands the slowest CTA
    // set the time, and with three rows per SM in flight the wait it hides was not exposed).
    constexpr size_t kStage = static_cast<size_t>(kTileElems) * sizeof(T);
    constexpr size_t kRingBytes = 64 * 1024;
    constexpr int kRoundTiles = round_tiles<T>();
    static_assert(kRoundTiles * kStage == kRingBytes, "the ring holds one round");
    auto kernel = use_tma ? topk_slice_kernel<T, 3, true> : topk_slice_kernel<T, 4, false>;
    const size_t ring_bytes = (variant >> 8) ? static_cast<size_t>(variant >> 8) * kStage : kRingBytes;  // (tuning builds: stages from the variant's high byte)
    if (use_tma && !allow_dynamic_smem(kernel, ring_bytes))
        return fail(ISPORE_ELAUNCH, "topk: %zu bytes of dynamic shared memory refused", ring_bytes);
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "topk: no device status word");
    const int64_t resident = resident_ctas(reinterpret_cast<const void*>(kernel), kTopkThreads, use_tma ? ring_bytes : 0);
    // Slices per row.  A row of up to four rounds is one slice: a CTA walks it in 9-10 us at any
    // row count that fits the GPU, where cutting it costs the merge launch (measured at 8-128
    // rows x 32000: 9-10 us against 11-17 us with 2-8 slices).  Longer rows are cut into slices of
    // two rounds, as far as the resident slots, the scratch and the merge kernel allow.
    constexpr int64_t kRoundElems = static_cast<int64_t>(kRoundTiles) * kTileElems;
    int64_t slices;
    switch ((variant & 0xff) >> 1) {
        case 1: slices = resident / rows; break;  // (tuning builds: as many slices as fill the GPU once)
        case 2: slices = 8; break;
        case 3: slices = 2; break;
        case 4: slices = 3; break;
        default:
            slices = vocab <= 4 * kRoundElems ? 1 : ceil_div(vocab, 2 * kRoundElems);
            if (slices > resident / rows) slices = resident / rows;
            break;
    }
    if (slices < 1) slices = 1;
    if (slices > ceil_div(vocab, 1024)) slices = ceil_div(vocab, 1024);
    if (slices * K > kMergeCap) slices = kMergeCap / K;
    if (slices > (have_scratch ? scratch_slices : 1)) slices = have_scratch ? scratch_slices : 1;
    if (slices < 1) slices = 1;
    int64_t slice_len = ceil_div(ceil_div(vocab, slices), E) * E;
    slices = ceil_div(vocab, slice_len);
    if (rows * slices > INT32_MAX) return fail(ISPORE_ELIMIT, "topk: rows*slices too large");
    int nstages = 0;
    size_t smem = 0;
    if (use_tma) {
        int64_t st_n = static_cast<int64_t>(ring_bytes / kStage);
        const int64_t tiles = ceil_div(slice_len, kTileElems);
        if (st_n > tiles) st_n = tiles;  // a short slice needs no more stages than it has tiles
        if (st_n > kMaxStages) st_n = kMaxStages;
        if (st_n < 1) st_n = 1;
        nstages = static_cast<int>(st_n);
        smem = static_cast<size_t>(nstages) * kStage;
    }

    if (slices == 1) {
        // The slice kernel's sorted list is already the answer.
        launch_chained(kernel, static_cast<int>(rows), kTopkThreads, smem, st, probs, vocab, static_cast<int>(slice_len), 1, K,
                       final_ids, final_vals, 1, index_offset, vec_loads, nstages, status, uniform, temperature, sampled_ids);
        return check_launch("topk_slice_kernel");
    }
    launch_chained(kernel, static_cast<int>(rows * slices), kTopkThreads, smem, st, probs, vocab,
                   static_cast<int>(slice_len), static_cast<int>(slices), K, scratch_ids, scratch_vals, scratch_slices,
                   index_offset, vec_loads, nstages, status, nullptr, 1.0f, nullptr);
    if (int rc = check_launch("topk_slice_kernel")) return rc;
    const int64_t row_stride = static_cast<int64_t>(scratch_slices) * K;
    return merge_dispatch<T>(scratch_ids, scratch_vals, rows, static_cast<int32_t>(slices), K, K, row_stride, K,
                             row_stride, final_ids, final_vals, uniform, temperature, sampled_ids, st);
}

}  // namespace
}  // namespace ispore

// ---- top-K for callers that cannot allocate ------------------------------------------------
//
// Round 1 needs a place for the per-slice candidate lists.  ispore_topk_* takes it from the
// caller; ispore_topk_static_f32 takes it from this array instead, which is part of the
// library image: every GPU that loads the library holds these kStaticScratchBytes until the
// process exits.  First kStaticScratchEntries int32 ids, then as many fp32 values.
constexpr int kStaticScratchEntries = ISPORE_TOPK_STATIC_ENTRIES;
constexpr size_t kStaticScratchBytes = static_cast<size_t>(kStaticScratchEntries) * (sizeof(int32_t) + sizeof(float));
static __device__ __align__(256) unsigned char g_topk_static_scratch[kStaticScratchBytes];

namespace ispore {
namespace {

constexpr int kMaxStaticDevices = 64;
std::mutex g_static_mutex;
unsigned char* g_static_scratch_addr[kMaxStaticDevices] = {};

// Device address of the scratch array on the CURRENT device.  In host code the array's name
// is only a handle for the runtime, not something a kernel may dereference; the address a
// kernel needs comes from cudaGetSymbolAddress, asked once per device with that device
// current, and is cached.
int static_scratch(unsigned char** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ISPORE_ELAUNCH, "topk_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxStaticDevices) return fail(ISPORE_ELIMIT, "topk_static: device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_topk_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            return fail(ISPORE_ELAUNCH, "topk_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        }
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return ISPORE_OK;
}

}  // namespace
}  // namespace ispore

#ifdef ISPORE_TUNING
extern "C" __attribute__((visibility("default"))) void ispore_topk_ts(long long* out) {
    cudaMemcpyFromSymbol(out, ispore::g_topk_ts, sizeof(long long) * 64);
}
extern "C" __attribute__((visibility("default"))) void ispore_topk_debug(int v) {
    cudaMemcpyToSymbol(ispore::g_topk_debug, &v, sizeof(int));
}
#endif

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
    const int64_t row_stride = static_cast<int64_t>(lists) * K;
    return ispore::merge_dispatch<float>(cand_ids, cand_vals, rows, lists, K, K, row_stride, K, row_stride, final_ids,
                                         final_vals, uniform, temperature, sampled_ids,
                                         static_cast<cudaStream_t>(stream));
}
int ispore_topk_merge_strided_f32(const int32_t* cand_ids, const float* cand_vals, int64_t rows, int32_t lists,
                                  int32_t K, int64_t id_list_stride, int64_t id_row_stride, int64_t val_list_stride,
                                  int64_t val_row_stride, int32_t* final_ids, float* final_vals, const float* uniform,
                                  float temperature, int32_t* sampled_ids, ispore_stream_t stream) {
    return ispore::merge_dispatch<float>(cand_ids, cand_vals, rows, lists, K, id_list_stride, id_row_stride,
                                         val_list_stride, val_row_stride, final_ids, final_vals, uniform, temperature,
                                         sampled_ids, static_cast<cudaStream_t>(stream));
}
int ispore_topk_merge_strided_f16(const int32_t* cand_ids, const void* cand_vals, int64_t rows, int32_t lists,
                                  int32_t K, int64_t id_list_stride, int64_t id_row_stride, int64_t val_list_stride,
                                  int64_t val_row_stride, int32_t* final_ids, void* final_vals, const float* uniform,
                                  float temperature, int32_t* sampled_ids, ispore_stream_t stream) {
    return ispore::merge_dispatch<__half>(cand_ids, static_cast<const __half*>(cand_vals), rows, lists, K,
                                          id_list_stride, id_row_stride, val_list_stride, val_row_stride, final_ids,
                                          static_cast<__half*>(final_vals), uniform, temperature, sampled_ids,
                                          static_cast<cudaStream_t>(stream));
}
int ispore_topk_merge_f16(const int32_t* cand_ids, const void* cand_vals, int64_t rows, int32_t lists,
                          int32_t K, int32_t* final_ids, void* final_vals, const float* uniform,
                          float temperature, int32_t* sampled_ids, ispore_stream_t stream) {
    const int64_t row_stride = static_cast<int64_t>(lists) * K;
    return ispore::merge_dispatch<__half>(cand_ids, static_cast<const __half*>(cand_vals), rows, lists, K, K,
                                          row_stride, K, row_stride, final_ids, static_cast<__half*>(final_vals),
                                          uniform, temperature, sampled_ids, static_cast<cudaStream_t>(stream));
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

int ispore_topk_static_f32(const float* probs, int64_t rows, int64_t vocab, int32_t K, int32_t* final_ids,
                           float* final_vals, int32_t index_offset, const float* uniform, float temperature,
                           int32_t* sampled_ids, ispore_stream_t stream) {
    if (K < 1 || K > ISPORE_TOPK_MAX_K)
        return ispore::fail(ISPORE_ELIMIT, "topk_static: K=%d outside [1,%d]", K, ISPORE_TOPK_MAX_K);
    if (rows < 0) return ispore::fail(ISPORE_ESHAPE, "topk_static: rows=%lld", (long long)rows);
    // The lists of one slice per row must fit; more slices are used when they fit too.
    const int64_t per_slice = rows * K;
    if (per_slice > kStaticScratchEntries)
        return ispore::fail(ISPORE_ELIMIT,
                            "topk_static: rows*K = %lld exceeds the built-in scratch of %d entries; use ispore_topk_f32 "
                            "with caller-provided scratch",
                            (long long)per_slice, kStaticScratchEntries);
    int32_t slices = per_slice > 0 ? static_cast<int32_t>(kStaticScratchEntries / per_slice) : ISPORE_TOPK_REF_SLICES;
    if (slices > ISPORE_TOPK_REF_SLICES) slices = ISPORE_TOPK_REF_SLICES;
    unsigned char* base = nullptr;
    if (int rc = ispore::static_scratch(&base)) return rc;
    int32_t* scratch_ids = reinterpret_cast<int32_t*>(base);
    float* scratch_vals = reinterpret_cast<float*>(base + static_cast<size_t>(kStaticScratchEntries) * sizeof(int32_t));
    // Round 1 writes every slot round 2 reads (empty slots included), so whatever an earlier
    // call left in the array is never seen and nothing has to be cleared.
    return ispore::topk_dispatch<float>(probs, rows, vocab, K, scratch_ids, scratch_vals, slices, final_ids,
                                        final_vals, index_offset, uniform, temperature, sampled_ids,
                                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
