/*
 * ispore_kernels.h — C ABI of the B200 (sm_100a) fused layer-kernel library.
 *
 * One entry point per (operation, storage type).  Every pointer is a raw
 * DEVICE pointer owned by the caller unless a comment says "host"; sizes are
 * plain integers; `stream` is a cudaStream_t passed as void* (NULL = the
 * legacy default stream, which is what the reference launches on).  The
 * library allocates nothing, never synchronises the device and never frees
 * caller memory.  All launches are asynchronous.
 *
 * Return value: ISPORE_OK (0) or a negative ISPORE_E* code; the text of the
 * most recent failure on the calling thread is ispore_last_error_string().
 * Nothing here throws or exits.  The C++ templates under
 * inferspore_b200/compat/src/kernels/ (same file names, function names and
 * argument lists as the reference's src/kernels/ headers) unpack TensorWrapper /
 * BaseWeight arguments and forward to these symbols, turning a non-zero status
 * into std::runtime_error the way the reference's LLM_CHECK does
 * (src/utils/macro.h:90-110).
 *
 * Each declaration names the reference interface it replaces as
 * "ref: <file>:<lines>" (paths inside the m0dulo/InferSpore tree).
 */
#ifndef ISPORE_KERNELS_H_
#define ISPORE_KERNELS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define ISPORE_API
#else
#define ISPORE_API __attribute__((visibility("default")))
#endif

typedef void* ispore_stream_t; /* cudaStream_t */

enum {
    ISPORE_OK = 0,
    ISPORE_ENULL = -1,     /* a required pointer is NULL                       */
    ISPORE_ESHAPE = -2,    /* a size is negative, inconsistent or unsupported  */
    ISPORE_EALIGN = -3,    /* reserved: every op has an unaligned fallback     */
    ISPORE_ELAUNCH = -4,   /* the CUDA runtime refused the launch              */
    ISPORE_ESCRATCH = -5,  /* caller-provided scratch is too small             */
    ISPORE_ELIMIT = -6     /* size beyond a documented fixed limit             */
};

/* Bits of the device status word (see ispore_device_status). */
enum {
    ISPORE_DEV_BAD_TOKEN_ID = 1u << 0, /* embedding id outside [0, vocab)          */
    ISPORE_DEV_KV_OVERRUN = 1u << 1,   /* history+t >= max_seq_len: row skipped    */
    ISPORE_DEV_BAD_PADDING = 1u << 2,  /* un-padded token lands outside [0,bs*seq) */
    ISPORE_DEV_TIMEOUT = 1u << 3       /* a bounded wait on an async copy ran out     */
};

/* ---- library-level ------------------------------------------------------ */

ISPORE_API int ispore_version(void); /* major*10000 + minor*100 + patch */
ISPORE_API const char* ispore_last_error_string(void);

/* Thread-local stream used by the C++ launch templates, which (like the
 * reference launchers) take no stream argument.  Default: NULL. */
ISPORE_API void ispore_set_stream(ispore_stream_t stream);
ISPORE_API ispore_stream_t ispore_get_stream(void);

/* Programmatic dependent launch, per calling thread (default: off).
 * ref: none — the reference launches every kernel with plain stream order.
 * When on, the library's main kernels are launched with
 * cudaLaunchAttributeProgrammaticStreamSerialization: a kernel's launch may be
 * processed before its predecessor on the same stream has retired, and the kernel
 * waits on the device (griddepcontrol.wait) until that predecessor has completed
 * and its memory is visible before it touches global memory.  Results are
 * identical; what changes is that part of the launch latency of one kernel
 * overlaps the tail of the one before, which matters for chains of short kernels
 * launched one by one (decode steps, small token shards: 5 % on an eight-kernel
 * chain of 20-90 us kernels); inside a CUDA graph it is neutral.  Works for plain
 * launches and inside stream capture.  Only back-to-back kernels of this library overlap; anything else on
 * the stream (copies, events, other libraries' kernels) orders as usual. */
ISPORE_API void ispore_set_programmatic_launch(int enable);
ISPORE_API int ispore_get_programmatic_launch(void);

/* Copies the current device's status word to *flags_out (host) and optionally
 * clears it.  Synchronises the calling thread with the device; not for use
 * inside the hot loop.  Kernels never trap on bad data: they skip the access
 * and set a bit here instead. */
ISPORE_API int ispore_device_status(unsigned* flags_out, int clear);

/* ---- residual add (+bias) + RMSNorm ------------------------------------- *
 * ref: src/kernels/fused_addresidual_norm.h:9-15 (launchFusedAddBiasResidualRMSNorm),
 *      src/kernels/fused_addresidual_norm.cu:33-98 (fp32 kernel = the semantics),
 *      :143-170 (launcher).
 * Per row t of decoder_out[num_tokens, hidden], in place:
 *   s = decoder_out[t,:] + residual[t,:]      (skipped when residual == NULL)
 *   residual[t,:] = s                          (before the bias)
 *   s += bias                                  (skipped when bias == NULL)
 *   decoder_out[t,:] = (gamma * s) * rsqrt(mean(s^2) + eps)
 * f16: additions round to half exactly where the stored type forces it
 * (s and s+bias), the sum of squares, the mean and rsqrt are fp32, and the
 * product is rounded to half once.  residual == NULL && bias == NULL is the
 * plain RMSNorm the reference reaches through the same launcher (.cu:56,68). */
ISPORE_API int ispore_add_residual_rmsnorm_f32(float* decoder_out, float* residual,
                                               const float* bias, const float* gamma, float eps,
                                               int64_t num_tokens, int64_t hidden,
                                               ispore_stream_t stream);
ISPORE_API int ispore_add_residual_rmsnorm_f16(void* decoder_out, void* residual, const void* bias,
                                               const void* gamma, float eps, int64_t num_tokens,
                                               int64_t hidden, ispore_stream_t stream);

/* ---- plain RMSNorm ------------------------------------------------------- *
 * ref: no dedicated kernel file exists in the reference; the behaviour is
 *      src/kernels/fused_addresidual_norm.cu:33-98 with residual and bias
 *      absent, applied to attn_norm / ffn_norm / out_rmsnorm weights
 *      (src/weights/llama/layer_weights.h:32-33, llama_weights.h:19).
 * decoder_out[t,:] = (gamma * x) * rsqrt(mean(x^2) + eps), in place.  When
 * residual_copy != NULL it receives the un-normed input row (the value the
 * next residual add needs), so the activation is read from HBM once. */
ISPORE_API int ispore_rmsnorm_f32(float* decoder_out, float* residual_copy, const float* gamma,
                                  float eps, int64_t num_tokens, int64_t hidden,
                                  ispore_stream_t stream);
ISPORE_API int ispore_rmsnorm_f16(void* decoder_out, void* residual_copy, const void* gamma,
                                  float eps, int64_t num_tokens, int64_t hidden,
                                  ispore_stream_t stream);

/* ---- input embedding gather ---------------------------------------------- *
 * ref: src/kernels/input_embedding.h:6-9 (launchInputEmbedding),
 *      src/kernels/input_embedding.cu:5-23 (kernel), :25-45 (launcher).
 * output[t, :] = table[input_ids[t], :]  — a bit-exact row copy.
 * vocab_size > 0 enables the range check the reference lacks: a row whose id
 * is outside [0, vocab_size) is zero-filled and ISPORE_DEV_BAD_TOKEN_ID is
 * set.  vocab_size == 0 means "unknown" (the reference's tests leave the
 * table's shape empty) and ids are trusted. */
ISPORE_API int ispore_input_embedding_f32(const int32_t* input_ids, float* output,
                                          const float* table, int64_t num_tokens, int64_t hidden,
                                          int64_t vocab_size, ispore_stream_t stream);
ISPORE_API int ispore_input_embedding_f16(const int32_t* input_ids, void* output, const void* table,
                                          int64_t num_tokens, int64_t hidden, int64_t vocab_size,
                                          ispore_stream_t stream);

/* ---- QKV bias + RoPE + un-pad + head transpose (prefill) ------------------ *
 * ref: src/kernels/qkv_bias_and_RoPE.h:10-20 (launchAddFusedQKVBiasTransposeAndRoPE),
 *      src/kernels/qkv_bias_and_RoPE.cu:110-192 (fp32 kernel), :38-53 (frequency
 *      and rotation helpers), :236-252 (the bias indexing the fp32 kernel never
 *      applies), :286-330 (launcher).
 * QKV[token_num, head_num + 2*kv_head_num, head_size] packed without padding,
 * per token [q heads | k heads | v heads].  For packed token i:
 *   dst = i + padding_offset[i];  b = dst / seq_len;  s = dst % seq_len
 *   q[b, h, s, :], k[b, h, s, :], v[b, h, s, :] receive the token's heads.
 * bias (nullable, [(head_num + 2*kv_head_num) * head_size]) is added first.
 * q and k are rotated at position m = history_length[b] + s:
 *   theta_j = m / powf(base, 2j / rotary_dim),  j in [0, rotary_dim/2)
 *   out[j]            = cos*x[j] - sin*x[j + head_size/2]
 *   out[j+head_size/2] = cos*x[j + head_size/2] + sin*x[j]
 * Elements with j >= rotary_dim/2 pass through unrotated.  Padded (b, s)
 * positions are not written.  powf is evaluated on the host, once per call,
 * in fp32 (rotary_dim/2 <= 256 values travel as a kernel argument), so the
 * frequencies are the ones a CPU evaluation of the same formula produces;
 * the division and sincosf run on the device in fp32.  input_length,
 * max_position_embeddings and use_dynamic_ntk are accepted and unused, as in
 * the reference (.cu:161, :126-127). */
ISPORE_API int ispore_qkv_bias_rope_transpose_f32(
    float* q_buf, float* k_buf, float* v_buf, const float* QKV, const float* bias,
    const int32_t* padding_offset, const int32_t* history_length, const int32_t* input_length,
    int64_t batch_size, int64_t seq_len, int64_t token_num, int64_t head_num, int64_t kv_head_num,
    int64_t head_size, int32_t rotary_embedding_dim, float rotary_embedding_base,
    int32_t max_position_embeddings, int32_t use_dynamic_ntk, ispore_stream_t stream);
ISPORE_API int ispore_qkv_bias_rope_transpose_f16(
    void* q_buf, void* k_buf, void* v_buf, const void* QKV, const void* bias,
    const int32_t* padding_offset, const int32_t* history_length, const int32_t* input_length,
    int64_t batch_size, int64_t seq_len, int64_t token_num, int64_t head_num, int64_t kv_head_num,
    int64_t head_size, int32_t rotary_embedding_dim, float rotary_embedding_base,
    int32_t max_position_embeddings, int32_t use_dynamic_ntk, ispore_stream_t stream);

/* ---- decode-step RoPE, in place ------------------------------------------ *
 * ref: src/kernels/qkv_bias_and_RoPE.h:22-25 (launchRoPE),
 *      src/kernels/qkv_bias_and_RoPE.cu:352-390 (kernel), :404-438 (launcher).
 * qkv_buf[batch, head_num + 2*kv_head_num, head_size]: q and k heads are
 * rotated in place at position step-1 (the reference reads `step` from a CPU
 * tensor, so it is a by-value argument here).  The reference only accepts
 * batch 1 / 96 heads / head size 128 and leaves fp16 empty; both limits are
 * lifted. */
ISPORE_API int ispore_rope_decode_f32(float* qkv_buf, int64_t batch_size, int64_t head_num,
                                      int64_t kv_head_num, int64_t head_size, int32_t step,
                                      int32_t rotary_embedding_dim, float rotary_embedding_base,
                                      ispore_stream_t stream);
ISPORE_API int ispore_rope_decode_f16(void* qkv_buf, int64_t batch_size, int64_t head_num,
                                      int64_t kv_head_num, int64_t head_size, int32_t step,
                                      int32_t rotary_embedding_dim, float rotary_embedding_base,
                                      ispore_stream_t stream);

/* ---- SiLU(gate) * up ------------------------------------------------------ *
 * ref: src/kernels/act_kernel.h:8-9 (launchAct),
 *      src/kernels/act_kernel.cu:6-15 (silu), :18-55 (kernels), :57-71 (launcher).
 * input[rows, 2, inter] (gate row then up row per token) ->
 * out[r, i] = (g / (1 + exp(-g))) * u  evaluated in fp32, rounded once. */
ISPORE_API int ispore_silu_mul_f32(float* out, const float* input, int64_t rows, int64_t inter,
                                   ispore_stream_t stream);
ISPORE_API int ispore_silu_mul_f16(void* out, const void* input, int64_t rows, int64_t inter,
                                   ispore_stream_t stream);

/* ---- KV-cache concat ------------------------------------------------------- *
 * ref: src/kernels/concat_past_kv.h:7-14 (launchConcatKVCache),
 *      src/kernels/concat_past_kv.cu:8-73 (kernels), :75-113 (launcher).
 * k_src, v_src [batch, kv_heads, max_q_len, head_size];
 * k_dst, v_dst [num_layers, batch, kv_heads, max_seq_len, head_size];
 * for t < cur_query_length[b]:
 *   dst[layer, b, h, history_length[b] + t, :] = src[b, h, t, :]
 * K and V are written by one launch; all offsets are 64-bit (the reference's
 * int layer offset overflows from 2^31 elements, .cu:90-91).  `layer` is by
 * value (the reference reads it from a CPU tensor).  num_layers > 0 lets the
 * call reject layer >= num_layers; 0 = unknown.  A row that would land at or
 * beyond max_seq_len is skipped and ISPORE_DEV_KV_OVERRUN is set. */
ISPORE_API int ispore_concat_kv_f32(float* k_dst, float* v_dst, const float* k_src,
                                    const float* v_src, const int32_t* cur_query_length,
                                    const int32_t* history_length, int64_t layer,
                                    int64_t num_layers, int64_t batch_size, int64_t kv_head_num,
                                    int64_t max_q_len, int64_t max_seq_len, int64_t head_size,
                                    ispore_stream_t stream);
ISPORE_API int ispore_concat_kv_f16(void* k_dst, void* v_dst, const void* k_src, const void* v_src,
                                    const int32_t* cur_query_length, const int32_t* history_length,
                                    int64_t layer, int64_t num_layers, int64_t batch_size,
                                    int64_t kv_head_num, int64_t max_q_len, int64_t max_seq_len,
                                    int64_t head_size, ispore_stream_t stream);

/* ---- scale + mask + softmax ------------------------------------------------ *
 * ref: src/kernels/attn_softmax_kernel.h:7-11 (launchScaleMaskAndSoftmax),
 *      src/kernels/attn_softmax_kernel.cu:50-125 (fp32 kernel = the semantics),
 *      :265-297 (launcher).
 * qk, attn_score [batch, heads, q_len, k_len]; mask [batch, q_len, k_len] in
 * the same storage type, 1 = keep, 0 = masked, shared by all heads.
 *   z = scale*qk + (1 - mask)*(-10000);  m = max(FLT_MIN, max_k z)
 *   e = exp(z - m);  attn_score = e * (1 / (sum_k e + 1e-6))
 * All arithmetic is fp32 for both storage types; any k_len (odd included).
 * attn_score may alias qk. */
ISPORE_API int ispore_scale_mask_softmax_f32(float* attn_score, const float* qk, const float* mask,
                                             int64_t batch_size, int64_t head_num, int64_t q_len,
                                             int64_t k_len, float scale, ispore_stream_t stream);
ISPORE_API int ispore_scale_mask_softmax_f16(void* attn_score, const void* qk, const void* mask,
                                             int64_t batch_size, int64_t head_num, int64_t q_len,
                                             int64_t k_len, float scale, ispore_stream_t stream);

/* The same softmax with the mask derived inside the kernel from the two length arrays the
 * mask would have been built from; the [batch, q_len, k_len] mask tensor is never formed.
 * ref: the predicate of src/kernels/build_casual_mask.cu:36 applied inside the kernel of
 *      src/kernels/attn_softmax_kernel.cu:50-125; replaces the pair of calls
 *      launchBuildCausalMasks + launchScaleMaskAndSoftmax of the reference's context attention.
 * q_lens, k_lens [batch] int32.  Element for element the same arithmetic as ispore_build_causal_mask_*
 * followed by ispore_scale_mask_softmax_* on the same inputs; the two routes may run different kernels
 * for a shape, so row sums can be taken in another order (3e-6 relative in fp32, one half-ulp in fp16). */
ISPORE_API int ispore_scale_causal_softmax_f32(float* attn_score, const float* qk, const int32_t* q_lens,
                                               const int32_t* k_lens, int64_t batch_size, int64_t head_num,
                                               int64_t q_len, int64_t k_len, float scale, ispore_stream_t stream);
ISPORE_API int ispore_scale_causal_softmax_f16(void* attn_score, const void* qk, const int32_t* q_lens,
                                               const int32_t* k_lens, int64_t batch_size, int64_t head_num,
                                               int64_t q_len, int64_t k_len, float scale, ispore_stream_t stream);

/* ---- top-K (+ sampling) ----------------------------------------------------- *
 * ref: src/kernels/topK.h:41-46 (launchTopKforBeamSearch), src/kernels/topK.cu:17-74
 *      (two rounds), :76-110 (launcher; K fixed at 5, 8 blocks per row).
 * probs [rows, vocab] -> final_ids/final_vals [rows, K], sorted by
 * (value descending, index ascending): equal values tie on the LOWER index,
 * -0.0 == +0.0, NaNs order by their bit pattern above +inf / below -inf.
 * K is a run-time argument (1..ISPORE_TOPK_MAX_K).  Slots beyond the number
 * of available elements get id -1 and value -inf.
 * Round 1 splits each row in `slices` (chosen by the library, <= scratch_slices)
 * and writes per-slice top-K lists to the caller's scratch
 * scratch_ids/scratch_vals [rows, scratch_slices, K] — the same scratch
 * tensors the reference launcher takes; round 2 merges them.  The scratch only
 * bounds the number of slices: with scratch_slices <= 1 (or NULL scratch) one
 * CTA walks each row and writes the final lists directly, which is correct for
 * any vocab and is what the library chooses anyway for rows of up to 65536
 * elements (one launch; longer rows are cut into slices of 32768).  index_offset is
 * added to every emitted id (vocab-sharded callers pass the shard's first
 * column).  When uniform != NULL the merge also draws one id per row exactly
 * as ispore_sampling_* does and writes it to sampled_ids [rows]. */
#define ISPORE_TOPK_MAX_K 256
#define ISPORE_TOPK_REF_SLICES 8
ISPORE_API int ispore_topk_f32(const float* probs, int64_t rows, int64_t vocab, int32_t K,
                               int32_t* scratch_ids, float* scratch_vals, int32_t scratch_slices,
                               int32_t* final_ids, float* final_vals, int32_t index_offset,
                               const float* uniform, float temperature, int32_t* sampled_ids,
                               ispore_stream_t stream);
ISPORE_API int ispore_topk_f16(const void* probs, int64_t rows, int64_t vocab, int32_t K,
                               int32_t* scratch_ids, void* scratch_vals, int32_t scratch_slices,
                               int32_t* final_ids, void* final_vals, int32_t index_offset,
                               const float* uniform, float temperature, int32_t* sampled_ids,
                               ispore_stream_t stream);

/* ---- top-K without caller scratch and without any allocation --------------------------- *
 * ref: none — the reference has no counterpart; its launcher always takes
 *      caller-allocated scratch tensors (src/kernels/topK.h:41-46).
 * For callers that are not allowed to allocate device memory at the point where
 * they sample: code running inside a serving loop whose HBM is fully carved up
 * in advance (weights + KV cache own the device, so a cudaMalloc there can fail
 * or stall), plugin-style "enqueue" callbacks that must not allocate, and
 * latency-critical threads that cannot afford cudaMalloc's device-wide
 * synchronisation.  Same results as ispore_topk_f32; the per-slice candidate
 * lists live in a fixed array inside the library image instead of
 * caller-provided scratch.  Neither this call nor anything it reaches calls
 * cudaMalloc/cudaFree or any allocating library routine.  What the CUDA runtime
 * does on its own the first time a process touches this library on a device is
 * outside that promise: with lazy module loading (the default) the first call
 * loads the module, which places its image — this array included — in device
 * memory and synchronises.  So make ONE warm-up call per device while
 * allocation is still allowed (at start-up); from the second call on, the free
 * device memory does not move (tests/test_zz_no_alloc.py asserts it).
 *   - Limit: rows * K <= ISPORE_TOPK_STATIC_ENTRIES (131072 list entries,
 *     1 MiB of device memory that every GPU loading the library holds until the
 *     process exits).  Larger requests return ISPORE_ELIMIT with an explanatory
 *     message; use ispore_topk_f32 for those.
 *   - The first call on each device also looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current), raises the kernel's
 *     shared-memory limit and caches both; make that warm-up call before
 *     starting any stream capture on the device.
 *   - All calls on a device share the one array, which keeps whatever the last
 *     call left in it.  Nothing needs clearing (every slot that is read is
 *     written first), but two calls that overlap on the GPU — different streams,
 *     or different host threads — race on it: serialise them. */
#define ISPORE_TOPK_STATIC_ENTRIES 131072
ISPORE_API int ispore_topk_static_f32(const float* probs, int64_t rows, int64_t vocab, int32_t K,
                                      int32_t* final_ids, float* final_vals, int32_t index_offset,
                                      const float* uniform, float temperature, int32_t* sampled_ids,
                                      ispore_stream_t stream);

/* Merge of `lists` candidate lists per row (cand_ids/cand_vals [rows, lists, K],
 * id -1 = empty slot; lists sorted best-first, as ispore_topk_* emits them, merge
 * by binary search, any other order is detected and ranked pairwise) into the global top-K with the
 * same total order.  This is round 2 above, exported because vocab-sharded
 * sampling all-gathers per-shard lists and merges them on every rank.
 * ref: src/kernels/topK.cu:48-74 (round 2). */
ISPORE_API int ispore_topk_merge_f32(const int32_t* cand_ids, const float* cand_vals, int64_t rows,
                                     int32_t lists, int32_t K, int32_t* final_ids,
                                     float* final_vals, const float* uniform, float temperature,
                                     int32_t* sampled_ids, ispore_stream_t stream);
ISPORE_API int ispore_topk_merge_f16(const int32_t* cand_ids, const void* cand_vals, int64_t rows,
                                     int32_t lists, int32_t K, int32_t* final_ids, void* final_vals,
                                     const float* uniform, float temperature, int32_t* sampled_ids,
                                     ispore_stream_t stream);

/* The same merge for candidate lists that are not laid out [rows, lists, K]: entry k of list a of
 * row r is cand_ids[r * id_row_stride + a * id_list_stride + k] (values likewise; strides in
 * ELEMENTS of the respective type, the K entries of a list contiguous).  [rows, lists, K] is
 * (list stride K, row stride lists*K); a buffer that an all-gather filled with one block per rank,
 * each block = that rank's [rows, K] ids followed by its [rows, K] values, is merged in place with
 * list stride = block size and row stride K, cand_vals pointing rows*K ids into the first block —
 * no re-layout between the collective and the merge.
 * ref: src/kernels/topK.cu:48-74 (round 2); the strided form has no counterpart upstream. */
ISPORE_API int ispore_topk_merge_strided_f32(const int32_t* cand_ids, const float* cand_vals, int64_t rows,
                                             int32_t lists, int32_t K, int64_t id_list_stride, int64_t id_row_stride,
                                             int64_t val_list_stride, int64_t val_row_stride, int32_t* final_ids,
                                             float* final_vals, const float* uniform, float temperature,
                                             int32_t* sampled_ids, ispore_stream_t stream);
ISPORE_API int ispore_topk_merge_strided_f16(const int32_t* cand_ids, const void* cand_vals, int64_t rows,
                                             int32_t lists, int32_t K, int64_t id_list_stride, int64_t id_row_stride,
                                             int64_t val_list_stride, int64_t val_row_stride, int32_t* final_ids,
                                             void* final_vals, const float* uniform, float temperature,
                                             int32_t* sampled_ids, ispore_stream_t stream);

/* ---- sampling from a top-K list --------------------------------------------- *
 * ref: absent from the reference (the only trace is the top_k entry that
 *      tools/weights_convert.py:69 writes to config.ini).  Defined here in the
 *      reference's launcher style.
 * topk_vals [rows, K] descending, topk_ids [rows, K], uniform [rows] in [0,1)
 * drawn by the caller:  p_i = expf((v_i - v_0) / temperature),  S = sum_i p_i
 * accumulated in index order in fp32; the pick is the smallest i with
 * sum_{j<=i} p_j >= u*S (the last valid slot if none); output_ids[row] =
 * topk_ids[row, i].  Slots with id -1 are skipped. */
ISPORE_API int ispore_sampling_f32(const int32_t* topk_ids, const float* topk_vals,
                                   const float* uniform, int32_t* output_ids, int64_t rows,
                                   int32_t K, float temperature, ispore_stream_t stream);
ISPORE_API int ispore_sampling_f16(const int32_t* topk_ids, const void* topk_vals,
                                   const float* uniform, int32_t* output_ids, int64_t rows,
                                   int32_t K, float temperature, ispore_stream_t stream);

/* ---- layout kernels either side of attention ---------------------------------------------- *
 * Causal / padding mask.
 * ref: src/kernels/build_casual_mask.h:7-10 (launchBuildCausalMasks), .cu:5-42 (kernel; the
 *      predicate is line 36), :44-54 (launcher).
 * mask[b, q, k] = 1 if q < q_lens[b] && k < k_lens[b] && k <= q + (k_lens[b] - q_lens[b])
 *                      && k >= k_lens[b] - q_lens[b], else 0;   mask [batch, max_q_len, max_k_len]. */
ISPORE_API int ispore_build_causal_mask_f32(float* mask, const int32_t* q_lens, const int32_t* k_lens,
                                            int64_t batch_size, int64_t max_q_len, int64_t max_k_len,
                                            ispore_stream_t stream);
ISPORE_API int ispore_build_causal_mask_f16(void* mask, const int32_t* q_lens, const int32_t* k_lens,
                                            int64_t batch_size, int64_t max_q_len, int64_t max_k_len,
                                            ispore_stream_t stream);

/* Padding offsets of packed (un-padded) tokens.
 * ref: src/kernels/cal_paddingoffset.h:8-11 (launchCalPaddingoffset), .cu:18-45 (a one-thread
 *      serial loop), :49-59 (launcher).
 * cum_seqlens [batch+1]: tokens before each sequence (last = total); padding_offset: for token
 * i of sequence b, padding_offset[cum_seqlens[b] + i] = b*max_q_len - cum_seqlens[b]; entries
 * past the total are left untouched.  A block scan replaces the serial loop. */
ISPORE_API int ispore_cal_padding_offset(int32_t* padding_offset, int32_t* cum_seqlens,
                                         const int32_t* input_lengths, int64_t batch_size,
                                         int64_t max_q_len, ispore_stream_t stream);

/* Transpose + remove padding after attention.
 * ref: declared in src/kernels/fused_transpose_and_remv_pad.h:7-10 (launchTransposeOutRemovePadding)
 *      but never defined in the reference; semantics from tests/unittests/test_fused_trans_remv_pad.cu:3-4,28-38.
 * in [batch, heads, seq_len, head_size] -> out [num_tokens, heads, head_size]:
 * out[t, h, :] = in[b, h, s, :] with (b, s) = divmod(t + padding_offset[t], seq_len). */
ISPORE_API int ispore_transpose_remove_padding_f32(float* out, const float* in, const int32_t* padding_offset,
                                                   int64_t batch_size, int64_t head_num, int64_t seq_len,
                                                   int64_t head_size, int64_t num_tokens, ispore_stream_t stream);
ISPORE_API int ispore_transpose_remove_padding_f16(void* out, const void* in, const int32_t* padding_offset,
                                                   int64_t batch_size, int64_t head_num, int64_t seq_len,
                                                   int64_t head_size, int64_t num_tokens, ispore_stream_t stream);

/* Repeat-KV: broadcast cached K/V heads to the query heads (GQA / MQA).
 * ref: src/kernels/repeat_kv.h:7-13 (launchRepeatKVCache), .cu:11-50 (kernel), :52-100 (launcher).
 * src caches [num_layers, batch, kv_heads, max_seq_len, head_size] ->
 * dst [batch, heads, max_k_len, head_size]:
 * dst[b, h, s, :] = src[layer, b, h / (heads/kv_heads), s, :] for s < context_length[b];
 * other positions of dst are left untouched.  K and V in one launch; 64-bit offsets. */
ISPORE_API int ispore_repeat_kv_f32(float* k_dst, float* v_dst, const float* k_src, const float* v_src,
                                    const int32_t* context_length, int64_t layer, int64_t num_layers,
                                    int64_t batch_size, int64_t kv_head_num, int64_t head_num,
                                    int64_t max_seq_len, int64_t max_k_len, int64_t head_size,
                                    ispore_stream_t stream);
ISPORE_API int ispore_repeat_kv_f16(void* k_dst, void* v_dst, const void* k_src, const void* v_src,
                                    const int32_t* context_length, int64_t layer, int64_t num_layers,
                                    int64_t batch_size, int64_t kv_head_num, int64_t head_num,
                                    int64_t max_seq_len, int64_t max_k_len, int64_t head_size,
                                    ispore_stream_t stream);

/* ---- decode-time fused masked multi-head attention (one new token per sequence) ----------- *
 * ref: src/kernels/fused_decoder_self_attention.h:10-18 (launchDecoderMaskedMHA),
 *      src/kernels/fused_decoder_self_attention.cu:112-250 (fp32 kernel), :251-379 (fp16),
 *      :381-441 (launcher); CPU function tests/unittests/test_fused_decoder_attention.cu:12-143.
 * qkv_buf [batch, head_num + 2*kv_head_num, head_size] (q heads, k heads, v heads of the new
 * token); qkv_bias [(head_num + 2*kv_head_num) * head_size] or NULL; k_cache, v_cache
 * [num_layers, batch, kv_head_num, max_seq_len, head_size]; mha_output [batch, head_num, head_size].
 *   q, k, v (+ bias);  RoPE on q and k: pairs (2i, 2i+1), angle rope_timestep / base^(2i/rot_dim)
 *   for 2i < rot_dim (the reference launcher passes rope_timestep = step);
 *   cache[layer, b, g, step-1, :] = k, v;  logit_i = rsqrt(head_size) * <q, K_i> for i < step;
 *   p = exp(logit - max) / (sum + 1e-6);  out = sum_i p_i V_i.
 * Every one of the `step` logits takes part in the softmax and the maximum is the true one, as
 * in the reference's CPU function (its kernel covers only the first head_size/vec logits and
 * floors the maximum at 0); the batch stride of qkv_buf is the tensor's own.  fp16 computes in
 * fp32 with q, k, v rounded to half where the reference holds them in half registers.
 * head_size must be (4 for f32, 8 for f16) times a power of two up to 32 (128 in every config).
 * workspace: optional scratch that lets the kernel split long sequences over several CTAs
 * (needed to fill the GPU at small batch); ispore_decoder_masked_mha_workspace_bytes gives the
 * size the call will use.  Without it the call runs one CTA per (sequence, head group) and
 * returns ISPORE_ESCRATCH only when step exceeds what shared memory can hold (40960 logits per
 * head group). */
ISPORE_API int64_t ispore_decoder_masked_mha_workspace_bytes(int64_t batch_size, int64_t head_num,
                                                             int64_t kv_head_num, int64_t head_size, int64_t step);
ISPORE_API int ispore_decoder_masked_mha_f32(float* mha_output, const float* qkv_buf, const float* qkv_bias,
                                             float* k_cache, float* v_cache, int64_t layer, int64_t num_layers,
                                             int64_t batch_size, int64_t head_num, int64_t kv_head_num,
                                             int64_t max_seq_len, int64_t head_size, int64_t step,
                                             int32_t rotary_embedding_dim, float rotary_embedding_base,
                                             float rope_timestep, void* workspace, int64_t workspace_bytes,
                                             ispore_stream_t stream);
ISPORE_API int ispore_decoder_masked_mha_f16(void* mha_output, const void* qkv_buf, const void* qkv_bias,
                                             void* k_cache, void* v_cache, int64_t layer, int64_t num_layers,
                                             int64_t batch_size, int64_t head_num, int64_t kv_head_num,
                                             int64_t max_seq_len, int64_t head_size, int64_t step,
                                             int32_t rotary_embedding_dim, float rotary_embedding_base,
                                             float rope_timestep, void* workspace, int64_t workspace_bytes,
                                             ispore_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* ISPORE_KERNELS_H_ */
