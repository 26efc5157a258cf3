// Input-embedding gather for sm_100a.
//
// Semantics: src/kernels/input_embedding.cu:5-23 of the reference —
// output[t, :] = table[input_ids[t], :], a bit-exact row copy.  The reference
// moves one element per thread-iteration with a div/mod per element.  Default
// path here: TMA bulk copies, one lane per row (table row -> shared memory ->
// output row), nothing in registers.  Fallback for rows that are not a multiple
// of 16 bytes or larger than 32 KB: one warp per row moving 128-bit vectors,
// four independent loads in flight per lane; then a scalar kernel.
#include "common.cuh"
#include "tma.cuh"

namespace ispore {
namespace {

template <int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
embedding_gather_vec_kernel(const int32_t* __restrict__ ids, uint4* __restrict__ out,
                            const uint4* __restrict__ table, int64_t num_tokens, int row_vecs,
                            int64_t vocab, unsigned* __restrict__ status) {
    chain_begin();
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t warp_stride = static_cast<int64_t>(gridDim.x) * kWarps;
    for (int64_t t = warp_global; t < num_tokens; t += warp_stride) {
        const int64_t id = __ldg(ids + t);
        uint4* dst = out + t * row_vecs;
        if (vocab > 0 && (id < 0 || id >= vocab)) {
            if (lane == 0) atomicOr(status, ISPORE_DEV_BAD_TOKEN_ID);
            for (int v = lane; v < row_vecs; v += 32) st_stream(dst + v, make_uint4(0, 0, 0, 0));
            continue;
        }
        const uint4* src = table + id * row_vecs;
        for (int v0 = lane; v0 < row_vecs; v0 += 32 * UNROLL) {
            uint4 buf[UNROLL];
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const int v = v0 + 32 * k;
                if (v < row_vecs) buf[k] = ld_stream(src + v);
            }
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const int v = v0 + 32 * k;
                if (v < row_vecs) st_stream(dst + v, buf[k]);
            }
        }
    }
}

// TMA variant: a row never touches registers.  Lane l of a one-warp CTA owns row
// (blockIdx.x * ROWS + l): it asks the copy engine to bring the table row into its slot of
// shared memory (cp.async.bulk, completion on the lane's own mbarrier), waits, and hands the
// slot back to the engine for the store to the output row.  ROWS rows per CTA are in flight
// together and many small CTAs per SM keep several hundred KB on the wire without a single
// data register.  Needs row_bytes % 16 == 0 and 16-byte aligned bases.
template <int ROWS>
__global__ void __launch_bounds__(32)
embedding_gather_tma_kernel(const int32_t* __restrict__ ids, unsigned char* __restrict__ out,
                            const unsigned char* __restrict__ table, int64_t num_tokens, uint32_t row_bytes,
                            int64_t vocab, unsigned* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char slots[];  // [ROWS][row_bytes]
    __shared__ __align__(8) uint64_t full[ROWS];
    chain_begin();
    const int lane = threadIdx.x;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * ROWS + lane;
    const bool mine = lane < ROWS && t < num_tokens;
    if (lane < ROWS) tma::mbar_init(&full[lane], 1);
    tma::fence_mbar_init();
    __syncwarp();
    if (!mine) return;  // no block-level barrier below

    const int64_t id = __ldg(ids + t);
    unsigned char* dst = out + t * row_bytes;
    if (vocab > 0 && (id < 0 || id >= vocab)) {
        atomicOr(status, ISPORE_DEV_BAD_TOKEN_ID);
        for (uint32_t o = 0; o < row_bytes; o += 16) *reinterpret_cast<uint4*>(dst + o) = make_uint4(0, 0, 0, 0);
        return;
    }
    unsigned char* slot = slots + static_cast<size_t>(lane) * row_bytes;
    tma::mbar_arrive_expect_tx(&full[lane], row_bytes);
    tma::load(slot, table + id * row_bytes, row_bytes, &full[lane]);
    if (!tma::mbar_wait(&full[lane], 0)) {
        atomicOr(status, ISPORE_DEV_TIMEOUT);
        tma::mbar_wait(&full[lane], 0);  // one more bounded wait for the copy in flight, then give up
        return;
    }
    tma::store(dst, slot, row_bytes);
    tma::commit_group();
    tma::wait_group_read<0>();  // the slot must stay allocated until the engine has read it
}

template <typename T>
__global__ void embedding_gather_scalar_kernel(const int32_t* __restrict__ ids, T* __restrict__ out,
                                               const T* __restrict__ table, int64_t num_tokens,
                                               int64_t hidden, int64_t vocab,
                                               unsigned* __restrict__ status) {
    for (int64_t t = blockIdx.x; t < num_tokens; t += gridDim.x) {
        const int64_t id = ids[t];
        const bool bad = vocab > 0 && (id < 0 || id >= vocab);
        if (bad && threadIdx.x == 0) atomicOr(status, ISPORE_DEV_BAD_TOKEN_ID);
        for (int64_t j = threadIdx.x; j < hidden; j += blockDim.x)
            out[t * hidden + j] = bad ? from_float<T>(0.f) : table[id * hidden + j];
    }
}

template <typename T>
int embedding_dispatch(const int32_t* ids, T* out, const T* table, int64_t tokens, int64_t hidden,
                       int64_t vocab, cudaStream_t st) {
    if (tokens < 0 || hidden <= 0 || vocab < 0)
        return fail(ISPORE_ESHAPE, "input_embedding: bad shape tokens=%lld hidden=%lld vocab=%lld",
                    (long long)tokens, (long long)hidden, (long long)vocab);
    if (tokens == 0) return ISPORE_OK;
    if (ids == nullptr || out == nullptr || table == nullptr)
        return fail(ISPORE_ENULL, "input_embedding: NULL buffer");
    unsigned* status = device_status_ptr();
    if (status == nullptr) return fail(ISPORE_ELAUNCH, "input_embedding: no device status word");
    constexpr int E = VecTraits<T>::kElems;
    const int64_t row_bytes = hidden * static_cast<int64_t>(sizeof(T));
    if (tune(kTuneEmbedding, 1004) >= 1000 && row_bytes % 16 == 0 && row_bytes <= 32 * 1024 && aligned16(out) && aligned16(table)) {
        // rows per CTA so that one CTA's slots take about 32 KB of shared memory
        const int variant = tune(kTuneEmbedding, 1004) - 1000;
        const unsigned char* tb = reinterpret_cast<const unsigned char*>(table);
        unsigned char* ob = reinterpret_cast<unsigned char*>(out);
#define ISPORE_EMB_TMA(ROWS)                                                                                     \
    do {                                                                                                         \
        const size_t smem = static_cast<size_t>(ROWS) * row_bytes;                                               \
        if (!allow_dynamic_smem(embedding_gather_tma_kernel<ROWS>, smem)) break;                                \
        launch_chained(embedding_gather_tma_kernel<ROWS>, static_cast<unsigned>(ceil_div(tokens, ROWS)), 32,     \
                       smem, st, ids, ob, tb, tokens, static_cast<uint32_t>(row_bytes), vocab, status);          \
        return check_launch("embedding_gather_tma_kernel");                                                      \
    } while (0)
        if (variant == 1) ISPORE_EMB_TMA(1);
        if (variant == 2) ISPORE_EMB_TMA(2);
        if (variant == 8) ISPORE_EMB_TMA(8);
        ISPORE_EMB_TMA(4);
#undef ISPORE_EMB_TMA
    }
    if (hidden % E == 0 && hidden / E <= INT32_MAX && aligned16(out) && aligned16(table)) {
        constexpr int THREADS = 256, UNROLL = 4;
        const int64_t blocks = ceil_div(tokens, THREADS / 32);
        auto kernel = embedding_gather_vec_kernel<THREADS, UNROLL>;
        launch_chained(kernel, persistent_grid(kernel, THREADS, 0, blocks, 16), THREADS, 0, st, ids,
                       reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(table), tokens,
                       static_cast<int>(hidden / E), vocab, status);
        return check_launch("embedding_gather_vec_kernel");
    }
    embedding_gather_scalar_kernel<T><<<persistent_grid(embedding_gather_scalar_kernel<T>, 256, 0, tokens), 256, 0, st>>>(
        ids, out, table, tokens, hidden, vocab, status);
    return check_launch("embedding_gather_scalar_kernel");
}

}  // namespace
}  // namespace ispore

extern "C" {
int ispore_input_embedding_f32(const int32_t* input_ids, float* output, const float* table,
                               int64_t num_tokens, int64_t hidden, int64_t vocab_size,
                               ispore_stream_t stream) {
    return ispore::embedding_dispatch<float>(input_ids, output, table, num_tokens, hidden, vocab_size,
                                             static_cast<cudaStream_t>(stream));
}
int ispore_input_embedding_f16(const int32_t* input_ids, void* output, const void* table,
                               int64_t num_tokens, int64_t hidden, int64_t vocab_size,
                               ispore_stream_t stream) {
    return ispore::embedding_dispatch<__half>(input_ids, static_cast<__half*>(output),
                                              static_cast<const __half*>(table), num_tokens, hidden,
                                              vocab_size, static_cast<cudaStream_t>(stream));
}
}
