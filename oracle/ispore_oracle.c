/*
 * ispore_oracle.c — CPU restatement of InferSpore's fused layer kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library:
 * tests/, the smoke check and the CPU-baseline legs of bench.py call it; the
 * product (inferspore_b200/) never does.
 *
 * Every function restates, in plain C and scalar fp32 arithmetic, what one
 * reference kernel computes; the comment above it names the reference lines it
 * follows (paths inside the m0dulo/InferSpore tree).  Where a reference kernel
 * is unfinished (fp16 norm, fp16 RoPE, bias add, K = 50, sampling) the function
 * follows the finished fp32 sibling and says so.
 *
 * Parity pins: the closed-form fixtures of the reference's own unit tests
 * (tests/unittests/test_*.cu) are replayed against these functions in
 * tests/test_oracle_golden.py, and the reference's CPU functions themselves
 * (CPUSwiGLU, cpuEmbedding, CPUfunc, CPUfusedresidandRMSNorm), compiled from
 * where they lie into oracle/_ref/, are compared with these functions on
 * random inputs in tests/test_oracle_vs_ref.py.
 *
 * fp16 tensors travel as uint16_t bit patterns.  The *_f16 functions compute
 * in fp32 and round once to half (round-to-nearest-even); several also return
 * the unrounded fp32 result so a test can budget the rounding separately.
 *
 * Rows are independent in every op; loops over rows carry an OpenMP pragma so
 * the same code serves as the multi-core CPU baseline (orc_set_threads).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---- threads ------------------------------------------------------------------ */

ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- half <-> float, bit exact with IEEE binary16 ------------------------------- */

ORC_API float orc_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: value = man * 2^-24 */
            const float f = (float)man * 5.9604644775390625e-8f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

ORC_API uint16_t orc_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (absx > 0x7F800000u ? (0x200u | ((absx >> 13) & 0x3FFu)) : 0u));
    if (absx >= 0x477FF000u) /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    if (absx < 0x33000001u) /* <= 2^-25 rounds to zero (ties-to-even at exactly 2^-25) */
        return sign;
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    int shift;                                   /* bits to drop from m */
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    const uint32_t kept = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half_ulp = 1u << (shift - 1);
    uint32_t out = base + kept;
    if (rem > half_ulp || (rem == half_ulp && (out & 1u))) out += 1u; /* carries into the exponent correctly */
    return (uint16_t)(sign | out);
}

static inline float h2f(uint16_t h) { return orc_half_to_float(h); }
static inline uint16_t f2h(float f) { return orc_float_to_half(f); }
static inline float round_half(float f) { return h2f(f2h(f)); }

/* ---- residual add (+bias) + RMSNorm ---------------------------------------------- *
 * Follows src/kernels/fused_addresidual_norm.cu:33-98 (fp32 kernel):
 *   :55-66  x += r; r = x            (only when residual != NULL, :56)
 *   :68-73  x += bias                (only when bias != NULL)
 *   :74-77  sum of squares
 *   :82-84  inv = rsqrt(sum / hidden + eps)
 *   :91-97  x = scale * x * inv      (product order (scale*x)*inv)
 * The sum of squares is accumulated in double and rounded to float once: the
 * kernel's tree order and a sequential fp32 loop are both approximations of
 * that value, and the tests' tolerance covers either.                            */
ORC_API void orc_add_residual_rmsnorm_f32(float* x, float* r, const float* bias, const float* gamma,
                                          float eps, int64_t tokens, int64_t hidden) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tokens; ++t) {
        float* xr = x + t * hidden;
        float* rr = r ? r + t * hidden : NULL;
        double acc = 0.0;
        for (int64_t i = 0; i < hidden; ++i) {
            float s = xr[i];
            if (rr) {
                s = s + rr[i];
                rr[i] = s;
            }
            if (bias) s = s + bias[i];
            xr[i] = s;
            acc += (double)s * (double)s;
        }
        const float mean = (float)(acc / (double)hidden);
        const float inv = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < hidden; ++i) xr[i] = (gamma[i] * xr[i]) * inv;
    }
}

/* fp16 storage.  The reference's fp16 kernel (:100-141) is unfinished (the sum
 * is never stored, a barrier is missing, 2048-thread launch); this follows the
 * fp32 kernel's algorithm with the roundings the half storage type forces:
 * x+r is rounded to half (it is stored as the new residual and the reference
 * adds with __hadd2, :121), +bias rounds again (:121), everything after is fp32
 * with a single final rounding.  x_unrounded (nullable, [tokens, hidden])
 * receives the fp32 value before that final rounding.                            */
ORC_API void orc_add_residual_rmsnorm_f16(uint16_t* x, uint16_t* r, const uint16_t* bias,
                                          const uint16_t* gamma, float eps, int64_t tokens,
                                          int64_t hidden, float* x_unrounded) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tokens; ++t) {
        uint16_t* xr = x + t * hidden;
        uint16_t* rr = r ? r + t * hidden : NULL;
        float* tmp = (float*)malloc((size_t)hidden * sizeof(float));
        double acc = 0.0;
        for (int64_t i = 0; i < hidden; ++i) {
            float s = h2f(xr[i]);
            if (rr) {
                s = round_half(s + h2f(rr[i]));
                rr[i] = f2h(s);
            }
            if (bias) s = round_half(s + h2f(bias[i]));
            tmp[i] = s;
            acc += (double)s * (double)s;
        }
        const float mean = (float)(acc / (double)hidden);
        const float inv = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < hidden; ++i) {
            const float y = (h2f(gamma[i]) * tmp[i]) * inv;
            if (x_unrounded) x_unrounded[t * hidden + i] = y;
            xr[i] = f2h(y);
        }
        free(tmp);
    }
}

/* Plain RMSNorm: the same kernel with residual and bias absent (:56, :68).
 * residual_copy (nullable) receives the un-normed input.                          */
ORC_API void orc_rmsnorm_f32(float* x, float* residual_copy, const float* gamma, float eps,
                             int64_t tokens, int64_t hidden) {
    if (residual_copy) memcpy(residual_copy, x, (size_t)(tokens * hidden) * sizeof(float));
    orc_add_residual_rmsnorm_f32(x, NULL, NULL, gamma, eps, tokens, hidden);
}

ORC_API void orc_rmsnorm_f16(uint16_t* x, uint16_t* residual_copy, const uint16_t* gamma, float eps,
                             int64_t tokens, int64_t hidden, float* x_unrounded) {
    if (residual_copy) memcpy(residual_copy, x, (size_t)(tokens * hidden) * sizeof(uint16_t));
    orc_add_residual_rmsnorm_f16(x, NULL, NULL, gamma, eps, tokens, hidden, x_unrounded);
}

/* ---- input embedding ---------------------------------------------------------------- *
 * Follows src/kernels/input_embedding.cu:5-23: out[t, j] = table[ids[t]*hidden + j].
 * elem_size is 4 (fp32) or 2 (fp16); the copy is bit exact.  vocab > 0 adds the
 * range check of the CUDA library (rows with a bad id become zeros).              */
ORC_API void orc_input_embedding(const int32_t* ids, void* out, const void* table, int64_t tokens,
                                 int64_t hidden, int64_t elem_size, int64_t vocab) {
    const size_t row_bytes = (size_t)(hidden * elem_size);
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tokens; ++t) {
        const int64_t id = ids[t];
        char* dst = (char*)out + (size_t)t * row_bytes;
        if (vocab > 0 && (id < 0 || id >= vocab))
            memset(dst, 0, row_bytes);
        else
            memcpy(dst, (const char*)table + (size_t)id * row_bytes, row_bytes);
    }
}

/* ---- QKV bias + RoPE + un-pad + head transpose ------------------------------------------ *
 * Follows src/kernels/qkv_bias_and_RoPE.cu:110-192 (fp32 kernel):
 *   :135-140  dst = i + padding_offset[i]; b = dst / seq_len; s = dst % seq_len
 *   :142-145  q/k/v element offsets inside the packed token
 *   :148-158  transposed destinations; v written for head < kv_head_num
 *   :160-163  timestep = history_length[b] + s
 *   :165-168  only j < rotary_dim/2 is rotated
 *   :170, :38-45   theta = timestep / powf(base, 2j / rotary_dim); cos, sin in float
 *   :182-190, :47-53  out[j] = c*x[j] - s*x[j+d/2];  out[j+d/2] = c*x[j+d/2] + s*x[j]
 * and the bias rule of the fp16 draft (:236-252): bias[head*d + j] on q,
 * bias[(head_num + head)*d + j] on k, bias[(head_num + kv_head_num + head)*d + j]
 * on v, added before the rotation, skipped when bias == NULL.
 * Elements with j in [rotary_dim/2, d/2) are copied through unrotated (the
 * reference leaves them unwritten).  Positions no token maps to keep whatever
 * the output buffers held.                                                          */
static void rope_coeffs(float* cs, float* sn, int rot_half, int rot_dim, float base, float position) {
    for (int j = 0; j < rot_half; ++j) {
        const float theta = position / powf(base, (float)(2 * j) / (float)rot_dim);
        cs[j] = cosf(theta);
        sn[j] = sinf(theta);
    }
}

ORC_API void orc_qkv_bias_rope_transpose_f32(float* q, float* k, float* v, const float* QKV,
                                             const float* bias, const int32_t* padding_offset,
                                             const int32_t* history_length, int64_t batch,
                                             int64_t seq_len, int64_t token_num, int64_t head_num,
                                             int64_t kv_head_num, int64_t head_size, int32_t rot_dim,
                                             float base) {
    const int64_t half = head_size / 2;
    const int rot_half = rot_dim / 2;
    const int64_t qkv_heads = head_num + 2 * kv_head_num;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < token_num; ++i) {
        const int64_t dst = i + padding_offset[i];
        if (dst < 0 || dst >= batch * seq_len) continue;
        const int64_t b = dst / seq_len, s = dst % seq_len;
        const float position = (float)(history_length[b] + (int32_t)s);
        float cs[256], sn[256];
        rope_coeffs(cs, sn, rot_half, rot_dim, base, position);
        const float* tok = QKV + i * qkv_heads * head_size;
        for (int64_t hh = 0; hh < head_num + kv_head_num; ++hh) {
            const int is_q = hh < head_num;
            const int64_t h = is_q ? hh : hh - head_num;
            float* out = is_q ? q + ((b * head_num + h) * seq_len + s) * head_size
                              : k + ((b * kv_head_num + h) * seq_len + s) * head_size;
            const float* in = tok + hh * head_size;
            const float* bb = bias ? bias + hh * head_size : NULL;
            for (int64_t j = 0; j < half; ++j) {
                float x0 = in[j], x1 = in[j + half];
                if (bb) {
                    x0 = x0 + bb[j];
                    x1 = x1 + bb[j + half];
                }
                if (j < rot_half) {
                    out[j] = cs[j] * x0 - sn[j] * x1;
                    out[j + half] = cs[j] * x1 + sn[j] * x0;
                } else {
                    out[j] = x0;
                    out[j + half] = x1;
                }
            }
        }
        for (int64_t h = 0; h < kv_head_num; ++h) {
            const float* in = tok + (head_num + kv_head_num + h) * head_size;
            const float* bb = bias ? bias + (head_num + kv_head_num + h) * head_size : NULL;
            float* out = v + ((b * kv_head_num + h) * seq_len + s) * head_size;
            for (int64_t j = 0; j < head_size; ++j) out[j] = bb ? in[j] + bb[j] : in[j];
        }
    }
}

/* fp16 storage: the reference's fp16 kernel body is commented out (:194-280);
 * this is the fp32 algorithm above on widened inputs with one rounding at the
 * end.  q_f32 / k_f32 (nullable, same shapes as q / k) receive the unrounded
 * values.                                                                            */
ORC_API void orc_qkv_bias_rope_transpose_f16(uint16_t* q, uint16_t* k, uint16_t* v, const uint16_t* QKV,
                                             const uint16_t* bias, const int32_t* padding_offset,
                                             const int32_t* history_length, int64_t batch,
                                             int64_t seq_len, int64_t token_num, int64_t head_num,
                                             int64_t kv_head_num, int64_t head_size, int32_t rot_dim,
                                             float base, float* q_f32, float* k_f32) {
    const int64_t half = head_size / 2;
    const int rot_half = rot_dim / 2;
    const int64_t qkv_heads = head_num + 2 * kv_head_num;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < token_num; ++i) {
        const int64_t dst = i + padding_offset[i];
        if (dst < 0 || dst >= batch * seq_len) continue;
        const int64_t b = dst / seq_len, s = dst % seq_len;
        const float position = (float)(history_length[b] + (int32_t)s);
        float cs[256], sn[256];
        rope_coeffs(cs, sn, rot_half, rot_dim, base, position);
        const uint16_t* tok = QKV + i * qkv_heads * head_size;
        for (int64_t hh = 0; hh < head_num + kv_head_num; ++hh) {
            const int is_q = hh < head_num;
            const int64_t h = is_q ? hh : hh - head_num;
            const int64_t at = is_q ? ((b * head_num + h) * seq_len + s) * head_size
                                    : ((b * kv_head_num + h) * seq_len + s) * head_size;
            uint16_t* out = (is_q ? q : k) + at;
            float* out32 = is_q ? (q_f32 ? q_f32 + at : NULL) : (k_f32 ? k_f32 + at : NULL);
            const uint16_t* in = tok + hh * head_size;
            const uint16_t* bb = bias ? bias + hh * head_size : NULL;
            for (int64_t j = 0; j < half; ++j) {
                float x0 = h2f(in[j]), x1 = h2f(in[j + half]);
                if (bb) {
                    x0 = x0 + h2f(bb[j]);
                    x1 = x1 + h2f(bb[j + half]);
                }
                float o0 = x0, o1 = x1;
                if (j < rot_half) {
                    o0 = cs[j] * x0 - sn[j] * x1;
                    o1 = cs[j] * x1 + sn[j] * x0;
                }
                out[j] = f2h(o0);
                out[j + half] = f2h(o1);
                if (out32) {
                    out32[j] = o0;
                    out32[j + half] = o1;
                }
            }
        }
        for (int64_t h = 0; h < kv_head_num; ++h) {
            const uint16_t* in = tok + (head_num + kv_head_num + h) * head_size;
            const uint16_t* bb = bias ? bias + (head_num + kv_head_num + h) * head_size : NULL;
            uint16_t* out = v + ((b * kv_head_num + h) * seq_len + s) * head_size;
            for (int64_t j = 0; j < head_size; ++j) out[j] = bb ? f2h(h2f(in[j]) + h2f(bb[j])) : in[j];
        }
    }
}

/* ---- decode-step RoPE, in place ------------------------------------------------------------ *
 * Follows src/kernels/qkv_bias_and_RoPE.cu:352-390: q and k heads of
 * qkv[batch, head_num + 2*kv_head_num, head_size] rotated at position step-1
 * (:380); k starts after the q heads (:418-419).  Every k head is rotated once
 * (the reference maps q heads onto k heads and would rotate a shared k head
 * several times under GQA, :366; it only runs with kv_head_num == head_num).        */
ORC_API void orc_rope_decode_f32(float* qkv, int64_t batch, int64_t head_num, int64_t kv_head_num,
                                 int64_t head_size, int32_t step, int32_t rot_dim, float base) {
    const int64_t half = head_size / 2;
    const int rot_half = rot_dim / 2;
    float cs[256], sn[256];
    rope_coeffs(cs, sn, rot_half, rot_dim, base, (float)(step - 1));
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t hh = 0; hh < head_num + kv_head_num; ++hh) {
            float* p = qkv + (b * (head_num + 2 * kv_head_num) + hh) * head_size;
            for (int j = 0; j < rot_half; ++j) {
                const float x0 = p[j], x1 = p[j + half];
                p[j] = cs[j] * x0 - sn[j] * x1;
                p[j + half] = cs[j] * x1 + sn[j] * x0;
            }
        }
}

ORC_API void orc_rope_decode_f16(uint16_t* qkv, int64_t batch, int64_t head_num, int64_t kv_head_num,
                                 int64_t head_size, int32_t step, int32_t rot_dim, float base,
                                 float* unrounded /* nullable, same shape */) {
    const int64_t half = head_size / 2;
    const int rot_half = rot_dim / 2;
    float cs[256], sn[256];
    rope_coeffs(cs, sn, rot_half, rot_dim, base, (float)(step - 1));
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t hh = 0; hh < head_num + kv_head_num; ++hh) {
            const int64_t at = (b * (head_num + 2 * kv_head_num) + hh) * head_size;
            uint16_t* p = qkv + at;
            for (int j = 0; j < rot_half; ++j) {
                const float x0 = h2f(p[j]), x1 = h2f(p[j + half]);
                const float o0 = cs[j] * x0 - sn[j] * x1, o1 = cs[j] * x1 + sn[j] * x0;
                p[j] = f2h(o0);
                p[j + half] = f2h(o1);
                if (unrounded) {
                    unrounded[at + j] = o0;
                    unrounded[at + j + half] = o1;
                }
            }
        }
}

/* ---- SiLU(gate) * up ---------------------------------------------------------------------------- *
 * Follows src/kernels/act_kernel.cu:6-15 (silu = x / (1 + expf(-x)) in float)
 * and :18-34 (out[r,i] = silu(in[r,0,i]) * in[r,1,i]); identical to the
 * reference's CPU function tests/unittests/test_act.cu:13-25.                            */
ORC_API void orc_silu_mul_f32(float* out, const float* in, int64_t rows, int64_t inter) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* g = in + r * 2 * inter;
        const float* u = g + inter;
        for (int64_t i = 0; i < inter; ++i) out[r * inter + i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
    }
}

/* fp16 storage: fp32 math, one rounding — what tests/unittests/test_act.cu:13-25
 * does for T = half.  (The reference's fp16 GPU kernel rounds silu to half and
 * multiplies in half, :14, :53 — two roundings.)                                         */
ORC_API void orc_silu_mul_f16(uint16_t* out, const uint16_t* in, int64_t rows, int64_t inter,
                              float* out_unrounded) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* g = in + r * 2 * inter;
        const uint16_t* u = g + inter;
        for (int64_t i = 0; i < inter; ++i) {
            const float gf = h2f(g[i]);
            const float y = (gf / (1.0f + expf(-gf))) * h2f(u[i]);
            if (out_unrounded) out_unrounded[r * inter + i] = y;
            out[r * inter + i] = f2h(y);
        }
    }
}

/* ---- KV-cache concat ---------------------------------------------------------------------------------- *
 * Follows src/kernels/concat_past_kv.cu:8-39 (K) and :41-73 (V):
 *   :28-38  for t < cur_query_length[b]:
 *           dst[layer_offset + ((b*H + h)*max_seq_len + history_length[b] + t)*d + j]
 *             = src[((b*H + h)*max_q_len + t)*d + j]
 *   :90-91  layer_offset = layer * bs * H * max_seq_len * d  (64-bit here)
 * One call handles one of K / V; bit exact for any elem_size.  Rows that would
 * land at or beyond max_seq_len are skipped, like the CUDA library does.           */
ORC_API void orc_concat_kv(void* dst, const void* src, const int32_t* cur_query_length,
                           const int32_t* history_length, int64_t layer, int64_t batch,
                           int64_t kv_heads, int64_t max_q_len, int64_t max_seq_len,
                           int64_t head_size, int64_t elem_size) {
    const int64_t row_bytes = head_size * elem_size;
    const int64_t layer_offset = layer * batch * kv_heads * max_seq_len * row_bytes;
#pragma omp parallel for schedule(static)
    for (int64_t bh = 0; bh < batch * kv_heads; ++bh) {
        const int64_t b = bh / kv_heads;
        int64_t cur = cur_query_length[b];
        const int64_t hist = history_length[b];
        if (cur > max_q_len) cur = max_q_len;
        if (hist < 0) continue;
        for (int64_t t = 0; t < cur; ++t) {
            if (hist + t >= max_seq_len) break;
            memcpy((char*)dst + layer_offset + (bh * max_seq_len + hist + t) * row_bytes,
                   (const char*)src + (bh * max_q_len + t) * row_bytes, (size_t)row_bytes);
        }
    }
}

/* ---- scale + mask + softmax ------------------------------------------------------------------------------ *
 * Follows src/kernels/attn_softmax_kernel.cu:50-125 (fp32 kernel):
 *   :82-86  mask[b, q, k] shared by all heads
 *   :88     z = scale*qk + (1 - mask)*(-10000)
 *   :77,:46 the running max starts at FLT_MIN and idle warps feed 0 into the
 *           block max, so m = max(FLT_MIN, max_k z)
 *   :106    e = expf(z - m)
 *   :113    inv = 1 / (sum + 1e-6)
 *   :121    out = e * inv
 * The sum is accumulated in double and rounded to float once.                      */
ORC_API void orc_scale_mask_softmax_f32(float* score, const float* qk, const float* mask, int64_t batch,
                                        int64_t heads, int64_t q_len, int64_t k_len, float scale) {
    const int64_t rows = batch * heads * q_len;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t b = row / (heads * q_len), qi = row % q_len;
        const float* qr = qk + row * k_len;
        const float* mr = mask + (b * q_len + qi) * k_len;
        float* out = score + row * k_len;
        float m = FLT_MIN;
        for (int64_t j = 0; j < k_len; ++j) {
            const float z = scale * qr[j] + (1.0f - mr[j]) * (-10000.0f);
            out[j] = z;
            if (z > m) m = z;
        }
        double sum = 0.0;
        for (int64_t j = 0; j < k_len; ++j) {
            out[j] = expf(out[j] - m);
            sum += (double)out[j];
        }
        const float inv = 1.0f / ((float)sum + 1e-6f);
        for (int64_t j = 0; j < k_len; ++j) out[j] = out[j] * inv;
    }
}

/* fp16 storage, fp32 arithmetic, one rounding.  (The reference's fp16 kernel,
 * :127-212, does the affine map and exp in half precision; its results lie
 * within half-precision error of these.)  score_f32 (nullable) receives the
 * unrounded values.                                                                  */
ORC_API void orc_scale_mask_softmax_f16(uint16_t* score, const uint16_t* qk, const uint16_t* mask,
                                        int64_t batch, int64_t heads, int64_t q_len, int64_t k_len,
                                        float scale, float* score_f32) {
    const int64_t rows = batch * heads * q_len;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t b = row / (heads * q_len), qi = row % q_len;
        const uint16_t* qr = qk + row * k_len;
        const uint16_t* mr = mask + (b * q_len + qi) * k_len;
        float* tmp = (float*)malloc((size_t)k_len * sizeof(float));
        float m = FLT_MIN;
        for (int64_t j = 0; j < k_len; ++j) {
            const float z = scale * h2f(qr[j]) + (1.0f - h2f(mr[j])) * (-10000.0f);
            tmp[j] = z;
            if (z > m) m = z;
        }
        double sum = 0.0;
        for (int64_t j = 0; j < k_len; ++j) {
            tmp[j] = expf(tmp[j] - m);
            sum += (double)tmp[j];
        }
        const float inv = 1.0f / ((float)sum + 1e-6f);
        for (int64_t j = 0; j < k_len; ++j) {
            const float y = tmp[j] * inv;
            if (score_f32) score_f32[row * k_len + j] = y;
            score[row * k_len + j] = f2h(y);
        }
        free(tmp);
    }
}

/* ---- top-K ------------------------------------------------------------------------------------------------------ *
 * Output contract of src/kernels/topK.cu:68-72 (final ids / values [rows, K],
 * best first; topK.h:21-37 keeps the list sorted by value descending) with K a
 * run-time value and a total order: value descending, then index ascending;
 * -0.0 ties with +0.0.  Comparison runs on the order-preserving 32-bit key of
 * the float bit pattern, so NaNs are ordered by their bits (positive NaNs above
 * +inf, negative NaNs below -inf) instead of poisoning the comparison.  Slots
 * beyond the number of elements get id -1 and value -inf.                            */
static inline uint32_t order_key(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    if (b == 0x80000000u) b = 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
static inline uint64_t composite(uint32_t key, uint32_t idx) { return ((uint64_t)key << 32) | (uint32_t)(~idx); }

static void heap_sift_down(uint64_t* h, int n, int i) { /* min-heap */
    for (;;) {
        int l = 2 * i + 1, r = l + 1, s = i;
        if (l < n && h[l] < h[s]) s = l;
        if (r < n && h[r] < h[s]) s = r;
        if (s == i) return;
        const uint64_t t = h[i];
        h[i] = h[s];
        h[s] = t;
        i = s;
    }
}
static int cmp_desc_u64(const void* a, const void* b) {
    const uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
    return x < y ? 1 : (x > y ? -1 : 0);
}

/* Selects the K largest composites of n candidates into best[K] (descending);
 * returns how many are valid.  key_of(i) / id_of(i) come from the caller's arrays. */
static int select_topk(const uint64_t* comp, int64_t n, int K, uint64_t* best) {
    int filled = 0;
    for (int64_t i = 0; i < n; ++i) {
        const uint64_t c = comp[i];
        if (c == 0) continue; /* empty slot */
        if (filled < K) {
            best[filled++] = c;
            if (filled == K)
                for (int j = K / 2 - 1; j >= 0; --j) heap_sift_down(best, K, j);
        } else if (c > best[0]) {
            best[0] = c;
            heap_sift_down(best, K, 0);
        }
    }
    qsort(best, (size_t)filled, sizeof(uint64_t), cmp_desc_u64);
    return filled;
}

/* elem_size 4: probs / vals are float; 2: half bit patterns.  index_offset is
 * added to every id (vocab-sharded callers).                                        */
ORC_API void orc_topk(const void* probs, int64_t rows, int64_t vocab, int32_t K, int32_t* ids, void* vals,
                      int32_t index_offset, int64_t elem_size) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t r = 0; r < rows; ++r) {
        uint64_t* comp = (uint64_t*)malloc((size_t)vocab * sizeof(uint64_t));
        uint64_t* best = (uint64_t*)malloc((size_t)K * sizeof(uint64_t));
        for (int64_t i = 0; i < vocab; ++i) {
            const float f = elem_size == 4 ? ((const float*)probs)[r * vocab + i]
                                           : h2f(((const uint16_t*)probs)[r * vocab + i]);
            comp[i] = composite(order_key(f), (uint32_t)i);
        }
        const int filled = select_topk(comp, vocab, K, best);
        for (int s = 0; s < K; ++s) {
            if (s < filled) {
                const uint32_t idx = ~(uint32_t)best[s];
                ids[r * K + s] = (int32_t)idx + index_offset;
                if (elem_size == 4)
                    ((float*)vals)[r * K + s] = ((const float*)probs)[r * vocab + idx];
                else
                    ((uint16_t*)vals)[r * K + s] = ((const uint16_t*)probs)[r * vocab + idx];
            } else {
                ids[r * K + s] = -1;
                if (elem_size == 4)
                    ((float*)vals)[r * K + s] = -INFINITY;
                else
                    ((uint16_t*)vals)[r * K + s] = 0xFC00u;
            }
        }
        free(comp);
        free(best);
    }
}

/* Merge of `lists` candidate lists of K (id, value) pairs per row (id -1 =
 * empty) into the top-K under the same order; round 2 of the reference
 * (src/kernels/topK.cu:48-74) with the row offset it forgets (:64).                  */
ORC_API void orc_topk_merge(const int32_t* cand_ids, const void* cand_vals, int64_t rows, int32_t lists,
                            int32_t K, int32_t* ids, void* vals, int64_t elem_size) {
    const int64_t n = (int64_t)lists * K;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        uint64_t* comp = (uint64_t*)malloc((size_t)n * sizeof(uint64_t));
        uint64_t* best = (uint64_t*)malloc((size_t)K * sizeof(uint64_t));
        for (int64_t i = 0; i < n; ++i) {
            const int32_t id = cand_ids[r * n + i];
            const float f = elem_size == 4 ? ((const float*)cand_vals)[r * n + i]
                                           : h2f(((const uint16_t*)cand_vals)[r * n + i]);
            comp[i] = id < 0 ? 0 : composite(order_key(f), (uint32_t)id);
        }
        const int filled = select_topk(comp, n, K, best);
        for (int s = 0; s < K; ++s) {
            int64_t src = -1;
            if (s < filled) /* find the candidate that produced this composite (ids are unique) */
                for (int64_t i = 0; i < n; ++i)
                    if (comp[i] == best[s]) {
                        src = i;
                        break;
                    }
            if (src >= 0) {
                ids[r * K + s] = cand_ids[r * n + src];
                if (elem_size == 4)
                    ((float*)vals)[r * K + s] = ((const float*)cand_vals)[r * n + src];
                else
                    ((uint16_t*)vals)[r * K + s] = ((const uint16_t*)cand_vals)[r * n + src];
            } else {
                ids[r * K + s] = -1;
                if (elem_size == 4)
                    ((float*)vals)[r * K + s] = -INFINITY;
                else
                    ((uint16_t*)vals)[r * K + s] = 0xFC00u;
            }
        }
        free(comp);
        free(best);
    }
}

/* ---- sampling from a top-K list ------------------------------------------------------------------------------------ *
 * No counterpart in the reference.  p_i = expf((v_i - v_0)/temperature);
 * S = sum_i p_i in index order in fp32; pick = smallest i with
 * sum_{j<=i} p_j >= u*S, the last valid slot if none; slots with id -1 are
 * skipped.  margin (nullable, [rows]) receives min_i |cum_i - u*S| / S, the
 * distance of the draw from the nearest CDF boundary, so a test can tell a real
 * disagreement from a draw that sits on a boundary.                                    */
ORC_API void orc_sampling(const int32_t* topk_ids, const void* topk_vals, const float* uniform,
                          int32_t* output_ids, int64_t rows, int32_t K, float temperature,
                          int64_t elem_size, float* margin) {
    for (int64_t r = 0; r < rows; ++r) {
        const int32_t* ids = topk_ids + r * K;
        float p[1024];
        float v0 = 0.f;
        float total = 0.f;
        int last = -1;
        for (int i = 0; i < K; ++i) {
            const float v = elem_size == 4 ? ((const float*)topk_vals)[r * K + i]
                                           : h2f(((const uint16_t*)topk_vals)[r * K + i]);
            if (i == 0) v0 = v;
            p[i] = ids[i] < 0 ? 0.f : expf((v - v0) / temperature);
            if (ids[i] >= 0) {
                total += p[i];
                last = i;
            }
        }
        const float target = uniform[r] * total;
        float cum = 0.f, best_margin = INFINITY;
        int pick = -1;
        for (int i = 0; i < K; ++i) {
            if (ids[i] < 0) continue;
            cum += p[i];
            const float d = fabsf(cum - target);
            if (d < best_margin) best_margin = d;
            if (pick < 0 && cum >= target) pick = i;
        }
        if (pick < 0) pick = last;
        output_ids[r] = pick >= 0 ? ids[pick] : -1;
        if (margin) margin[r] = total > 0.f ? best_margin / total : 0.f;
    }
}

/* ---- layout kernels either side of attention ------------------------------------------------------------- */

/* Causal / padding mask.  Follows src/kernels/build_casual_mask.cu:5-42; the predicate is line 36:
 *   q < qlen && k < klen && k <= q + (klen - qlen) && k >= klen - qlen.
 * (The reference's CPU function, tests/unittests/test_casual_mask.cu:12-32, lacks the last
 * clause; the two agree whenever klen == qlen, which is what its fixture uses.)
 * elem_size 4 writes floats, 2 writes half bit patterns.                                            */
ORC_API void orc_build_causal_mask(void* mask, const int32_t* q_lens, const int32_t* k_lens, int64_t batch,
                                   int64_t max_q_len, int64_t max_k_len, int64_t elem_size) {
    for (int64_t b = 0; b < batch; ++b) {
        const int qlen = q_lens[b], klen = k_lens[b];
        for (int64_t q = 0; q < max_q_len; ++q)
            for (int64_t k = 0; k < max_k_len; ++k) {
                const int one = q < qlen && k < klen && k <= q + (klen - qlen) && k >= klen - qlen;
                const int64_t at = (b * max_q_len + q) * max_k_len + k;
                if (elem_size == 4)
                    ((float*)mask)[at] = one ? 1.0f : 0.0f;
                else
                    ((uint16_t*)mask)[at] = one ? 0x3C00u : 0u;
            }
    }
}

/* Padding offsets.  Follows src/kernels/cal_paddingoffset.cu:18-45 line by line (lengths are
 * clamped to [0, max_q_len], which the reference leaves to the caller).                            */
ORC_API void orc_cal_padding_offset(int32_t* padding_offset, int32_t* cum_seqlens, const int32_t* input_lengths,
                                    int64_t batch, int64_t max_q_len) {
    int64_t ind = 0, cum_offset = 0, total = 0;
    for (int64_t b = 0; b < batch; ++b) {
        int64_t len = input_lengths[b];
        if (len < 0) len = 0;
        if (len > max_q_len) len = max_q_len;
        cum_seqlens[b] = (int32_t)total;
        for (int64_t i = 0; i < len; ++i) padding_offset[ind++] = (int32_t)cum_offset;
        cum_offset += max_q_len - len;
        total += len;
    }
    cum_seqlens[batch] = (int32_t)total;
}

/* Transpose + remove padding: [b, h, s, d] -> [num_tokens, h, d]
 * (tests/unittests/test_fused_trans_remv_pad.cu:3-4; the launcher is declared in
 * src/kernels/fused_transpose_and_remv_pad.h:7-10 and never defined upstream).                      */
ORC_API void orc_transpose_remove_padding(void* out, const void* in, const int32_t* padding_offset, int64_t batch,
                                          int64_t heads, int64_t seq_len, int64_t head_size, int64_t num_tokens,
                                          int64_t elem_size) {
    const int64_t row = head_size * elem_size;
    for (int64_t t = 0; t < num_tokens; ++t) {
        const int64_t dst = t + padding_offset[t];
        if (dst < 0 || dst >= batch * seq_len) continue;
        const int64_t b = dst / seq_len, s = dst % seq_len;
        for (int64_t h = 0; h < heads; ++h)
            memcpy((char*)out + (t * heads + h) * row, (const char*)in + (((b * heads + h) * seq_len) + s) * row,
                   (size_t)row);
    }
}

/* Repeat-KV.  Follows src/kernels/repeat_kv.cu:11-50 (index arithmetic :34-47) and the layer
 * offset of the launcher (:71), in 64 bits.  One call handles one of K / V.                          */
ORC_API void orc_repeat_kv(void* dst, const void* src, const int32_t* context_length, int64_t layer, int64_t batch,
                           int64_t kv_heads, int64_t heads, int64_t max_seq_len, int64_t max_k_len,
                           int64_t head_size, int64_t elem_size) {
    const int64_t row = head_size * elem_size;
    const int64_t q_per_kv = heads / kv_heads;
    const char* base = (const char*)src + layer * batch * kv_heads * max_seq_len * row;
    for (int64_t b = 0; b < batch; ++b) {
        int64_t len = context_length[b];
        if (len > max_k_len) len = max_k_len;
        if (len > max_seq_len) len = max_seq_len;
        for (int64_t h = 0; h < heads; ++h)
            for (int64_t s = 0; s < len; ++s)
                memcpy((char*)dst + ((b * heads + h) * max_k_len + s) * row,
                       base + ((b * kv_heads + h / q_per_kv) * max_seq_len + s) * row, (size_t)row);
    }
}

/* ---- decode-time fused masked multi-head attention ----------------------------------------------------- *
 * Follows the reference's CPU function CPUMaskedAttn
 * (tests/unittests/test_fused_decoder_attention.cu:12-143) for the attention itself — every one
 * of the `step` logits in the softmax, true maximum — and the reference kernel
 * (src/kernels/fused_decoder_self_attention.cu:112-250, fp16 :251-379) for what the CPU function
 * leaves out or only approximates:
 *   :163-188  bias added to q, k, v (in the storage type: half adds round to half)
 *   :57-110   RoPE on adjacent pairs (2i, 2i+1), angle t / powf(base, 2i / rot_dim), 2i < rot_dim,
 *             result kept in the storage type
 *   :206-209, :240-243  the new k, v written to cache[layer, b, g, step-1, :]
 *   :230-233  denominator = sum + 1e-6
 * The cache is [layers, bs, kv_heads, max_seq_len, d] (launcher :381-441), qkv is
 * [bs, heads + 2*kv_heads, d].  Sums are accumulated in double.  out_unrounded (nullable) receives
 * the fp32 output before the final rounding of the f16 variant.                                        */
static float ld_elem(const void* p, int64_t i, int64_t elem_size) {
    return elem_size == 4 ? ((const float*)p)[i] : h2f(((const uint16_t*)p)[i]);
}
static void st_elem(void* p, int64_t i, int64_t elem_size, float v) {
    if (elem_size == 4)
        ((float*)p)[i] = v;
    else
        ((uint16_t*)p)[i] = f2h(v);
}
static float round_elem(float v, int64_t elem_size) { return elem_size == 4 ? v : round_half(v); }

ORC_API void orc_decoder_masked_mha(void* out, const void* qkv, const void* bias, void* k_cache, void* v_cache,
                                    int64_t layer, int64_t batch, int64_t heads, int64_t kv_heads,
                                    int64_t max_seq_len, int64_t d, int64_t step, int32_t rot_dim, float base,
                                    float rope_t, int64_t elem_size, float* out_unrounded) {
    const int64_t qkv_heads = heads + 2 * kv_heads, q_per_kv = heads / kv_heads;
    const float scale = 1.0f / sqrtf((float)d);
    const int64_t layer_off = layer * batch * kv_heads * max_seq_len * d;
    float* rows = (float*)malloc((size_t)(batch * qkv_heads * d) * sizeof(float)); /* q, k, v after bias + RoPE */
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t r = 0; r < qkv_heads; ++r) {
            float* dst = rows + (b * qkv_heads + r) * d;
            for (int64_t i = 0; i < d; ++i) {
                float x = ld_elem(qkv, (b * qkv_heads + r) * d + i, elem_size);
                if (bias) x = round_elem(x + ld_elem(bias, r * d + i, elem_size), elem_size);
                dst[i] = x;
            }
            if (r < heads + kv_heads) /* q and k heads are rotated, v is not */
                for (int64_t i = 0; 2 * i + 1 < d && 2 * i < rot_dim; ++i) {
                    const float theta = rope_t / powf(base, (float)(2 * i) / (float)rot_dim);
                    const float c = cosf(theta), s = sinf(theta);
                    const float x0 = dst[2 * i], x1 = dst[2 * i + 1];
                    dst[2 * i] = round_elem(c * x0 - s * x1, elem_size);
                    dst[2 * i + 1] = round_elem(c * x1 + s * x0, elem_size);
                }
        }
    /* cache append */
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t g = 0; g < kv_heads; ++g) {
            const int64_t at = layer_off + ((b * kv_heads + g) * max_seq_len + (step - 1)) * d;
            for (int64_t i = 0; i < d; ++i) {
                st_elem(k_cache, at + i, elem_size, rows[(b * qkv_heads + heads + g) * d + i]);
                st_elem(v_cache, at + i, elem_size, rows[(b * qkv_heads + heads + kv_heads + g) * d + i]);
            }
        }
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t h = 0; h < heads; ++h) {
            const int64_t g = h / q_per_kv;
            const float* q = rows + (b * qkv_heads + h) * d;
            const int64_t c0 = layer_off + (b * kv_heads + g) * max_seq_len * d;
            double* logit = (double*)malloc((size_t)step * sizeof(double));
            double mx = -DBL_MAX;
            for (int64_t s = 0; s < step; ++s) {
                double acc = 0.0;
                for (int64_t i = 0; i < d; ++i) acc += (double)q[i] * (double)ld_elem(k_cache, c0 + s * d + i, elem_size);
                logit[s] = (double)(float)(acc * (double)scale);
                if (logit[s] > mx) mx = logit[s];
            }
            double sum = 0.0;
            for (int64_t s = 0; s < step; ++s) {
                logit[s] = (double)expf((float)(logit[s] - mx));
                sum += logit[s];
            }
            const double inv = 1.0 / (sum + 1e-6);
            for (int64_t i = 0; i < d; ++i) {
                double o = 0.0;
                for (int64_t s = 0; s < step; ++s) o += logit[s] * (double)ld_elem(v_cache, c0 + s * d + i, elem_size);
                const float y = (float)(o * inv);
                if (out_unrounded) out_unrounded[(b * heads + h) * d + i] = y;
                st_elem(out, (b * heads + h) * d + i, elem_size, y);
            }
            free(logit);
        }
    free(rows);
}
