"""numpy front end of oracle/libispore_oracle.so and of the reference-built
libraries in oracle/_ref/.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
CPU-baseline legs of bench.py.  fp16 arrays are numpy float16 (same bits as the
uint16 patterns the C side takes).  Functions return new arrays; inputs are not
modified unless the docstring says so.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "libispore_oracle.so"
REF_DIR = HERE / "_ref"

_p, _i64, _i32, _f = C.c_void_p, C.c_int64, C.c_int32, C.c_float
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not ORACLE_SO.exists():
            raise RuntimeError(f"{ORACLE_SO} missing: run `python oracle/build.py`")
        _lib = C.CDLL(str(ORACLE_SO))
        _lib.orc_half_to_float.restype = C.c_float
        _lib.orc_half_to_float.argtypes = [C.c_uint16]
        _lib.orc_float_to_half.restype = C.c_uint16
        _lib.orc_float_to_half.argtypes = [C.c_float]
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def _ptr(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return C.c_void_p(a.ctypes.data)


def _is16(a: np.ndarray) -> bool:
    if a.dtype == np.float16:
        return True
    if a.dtype == np.float32:
        return False
    raise TypeError(f"float32 or float16 expected, got {a.dtype}")


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(n))


def max_threads() -> int:
    return lib().orc_max_threads()


def add_residual_rmsnorm(x, residual, bias, gamma, eps):
    """Returns (normed, new_residual_or_None, unrounded_fp32_or_None)."""
    x = np.array(x, copy=True)
    r = None if residual is None else np.array(residual, copy=True)
    tokens, hidden = x.shape
    if _is16(x):
        unr = np.empty(x.shape, np.float32)
        lib().orc_add_residual_rmsnorm_f16(_ptr(x), _ptr(r), _ptr(bias), _ptr(gamma), _f(eps), _i64(tokens),
                                           _i64(hidden), _ptr(unr))
        return x, r, unr
    lib().orc_add_residual_rmsnorm_f32(_ptr(x), _ptr(r), _ptr(bias), _ptr(gamma), _f(eps), _i64(tokens), _i64(hidden))
    return x, r, None


def rmsnorm(x, gamma, eps, want_copy=False):
    """Returns (normed, residual_copy_or_None, unrounded_fp32_or_None)."""
    x = np.array(x, copy=True)
    cp = np.empty_like(x) if want_copy else None
    tokens, hidden = x.shape
    if _is16(x):
        unr = np.empty(x.shape, np.float32)
        lib().orc_rmsnorm_f16(_ptr(x), _ptr(cp), _ptr(gamma), _f(eps), _i64(tokens), _i64(hidden), _ptr(unr))
        return x, cp, unr
    lib().orc_rmsnorm_f32(_ptr(x), _ptr(cp), _ptr(gamma), _f(eps), _i64(tokens), _i64(hidden))
    return x, cp, None


def input_embedding(ids, table, vocab_check=True):
    ids = np.ascontiguousarray(ids, np.int32)
    tokens, hidden = ids.size, table.shape[1]
    out = np.empty((tokens, hidden), table.dtype)
    lib().orc_input_embedding(_ptr(ids), _ptr(out), _ptr(table), _i64(tokens), _i64(hidden),
                              _i64(table.dtype.itemsize), _i64(table.shape[0] if vocab_check else 0))
    return out


def qkv_bias_rope_transpose(QKV, bias, padding_offset, history_length, batch, seq_len, head_num, kv_head_num,
                            rot_dim, base, fill=0.0):
    """Returns (q, k, v, q_fp32_or_None, k_fp32_or_None); unwritten (padded) positions hold `fill`."""
    token_num, qkv_heads, head_size = QKV.shape
    assert qkv_heads == head_num + 2 * kv_head_num
    dt = QKV.dtype
    q = np.full((batch, head_num, seq_len, head_size), fill, dt)
    k = np.full((batch, kv_head_num, seq_len, head_size), fill, dt)
    v = np.full((batch, kv_head_num, seq_len, head_size), fill, dt)
    po = np.ascontiguousarray(padding_offset, np.int32)
    hl = np.ascontiguousarray(history_length, np.int32)
    args = [_ptr(q), _ptr(k), _ptr(v), _ptr(QKV), _ptr(bias), _ptr(po), _ptr(hl), _i64(batch), _i64(seq_len),
            _i64(token_num), _i64(head_num), _i64(kv_head_num), _i64(head_size), _i32(rot_dim), _f(base)]
    if _is16(QKV):
        q32 = np.full(q.shape, fill, np.float32)
        k32 = np.full(k.shape, fill, np.float32)
        lib().orc_qkv_bias_rope_transpose_f16(*args, _ptr(q32), _ptr(k32))
        return q, k, v, q32, k32
    lib().orc_qkv_bias_rope_transpose_f32(*args)
    return q, k, v, None, None


def rope_decode(qkv, head_num, kv_head_num, step, rot_dim, base):
    """Returns (rotated, unrounded_fp32_or_None)."""
    qkv = np.array(qkv, copy=True)
    batch, _, head_size = qkv.shape
    args = [_ptr(qkv), _i64(batch), _i64(head_num), _i64(kv_head_num), _i64(head_size), _i32(step), _i32(rot_dim),
            _f(base)]
    if _is16(qkv):
        unr = qkv.astype(np.float32)
        lib().orc_rope_decode_f16(*args, _ptr(unr))
        return qkv, unr
    lib().orc_rope_decode_f32(*args)
    return qkv, None


def silu_mul(inp):
    """inp [rows, 2, inter] -> (out [rows, inter], unrounded_fp32_or_None)."""
    rows, two, inter = inp.shape
    assert two == 2
    out = np.empty((rows, inter), inp.dtype)
    if _is16(inp):
        unr = np.empty((rows, inter), np.float32)
        lib().orc_silu_mul_f16(_ptr(out), _ptr(inp), _i64(rows), _i64(inter), _ptr(unr))
        return out, unr
    lib().orc_silu_mul_f32(_ptr(out), _ptr(inp), _i64(rows), _i64(inter))
    return out, None


def concat_kv(dst, src, cur_query_length, history_length, layer):
    """Writes into a copy of dst ([layers, bs, heads, max_seq, d] or 4-D single layer) and returns it."""
    dst = np.array(dst, copy=True)
    batch, kv_heads, max_q_len, head_size = src.shape
    max_seq_len = dst.shape[3] if dst.ndim == 5 else dst.shape[2]
    cl = np.ascontiguousarray(cur_query_length, np.int32)
    hl = np.ascontiguousarray(history_length, np.int32)
    lib().orc_concat_kv(_ptr(dst), _ptr(src), _ptr(cl), _ptr(hl), _i64(layer), _i64(batch), _i64(kv_heads),
                        _i64(max_q_len), _i64(max_seq_len), _i64(head_size), _i64(src.dtype.itemsize))
    return dst


def scale_mask_softmax(qk, mask, scale):
    """Returns (score, unrounded_fp32_or_None)."""
    batch, heads, q_len, k_len = qk.shape
    score = np.empty_like(qk)
    args = [_ptr(score), _ptr(qk), _ptr(mask), _i64(batch), _i64(heads), _i64(q_len), _i64(k_len), _f(scale)]
    if _is16(qk):
        unr = np.empty(qk.shape, np.float32)
        lib().orc_scale_mask_softmax_f16(*args, _ptr(unr))
        return score, unr
    lib().orc_scale_mask_softmax_f32(*args)
    return score, None


def topk(probs, K, index_offset=0):
    rows, vocab = probs.shape
    _is16(probs)
    ids = np.empty((rows, K), np.int32)
    vals = np.empty((rows, K), probs.dtype)
    lib().orc_topk(_ptr(probs), _i64(rows), _i64(vocab), _i32(K), _ptr(ids), _ptr(vals), _i32(index_offset),
                   _i64(probs.dtype.itemsize))
    return ids, vals


def topk_merge(cand_ids, cand_vals, K):
    rows, lists, k_in = cand_ids.shape
    assert k_in == K
    cand_ids = np.ascontiguousarray(cand_ids, np.int32)
    ids = np.empty((rows, K), np.int32)
    vals = np.empty((rows, K), cand_vals.dtype)
    lib().orc_topk_merge(_ptr(cand_ids), _ptr(cand_vals), _i64(rows), _i32(lists), _i32(K), _ptr(ids), _ptr(vals),
                         _i64(cand_vals.dtype.itemsize))
    return ids, vals


def sampling(topk_ids, topk_vals, uniform, temperature):
    """Returns (picked ids [rows], margin [rows] = distance of the draw to the nearest CDF boundary / S)."""
    rows, K = topk_ids.shape
    topk_ids = np.ascontiguousarray(topk_ids, np.int32)
    uniform = np.ascontiguousarray(uniform, np.float32)
    out = np.empty(rows, np.int32)
    margin = np.empty(rows, np.float32)
    lib().orc_sampling(_ptr(topk_ids), _ptr(topk_vals), _ptr(uniform), _ptr(out), _i64(rows), _i32(K),
                       _f(temperature), _i64(topk_vals.dtype.itemsize), _ptr(margin))
    return out, margin


# ---- the reference's own code, built into oracle/_ref/ by oracle/build.py ------------------

_ref_libs: dict[str, C.CDLL] = {}


def ref_available(name: str) -> bool:
    return (REF_DIR / name).exists()


def ref_lib(name: str) -> C.CDLL:
    """Loads oracle/_ref/<name> (e.g. 'libref_act.so')."""
    if name not in _ref_libs:
        path = REF_DIR / name
        if not path.exists():
            raise RuntimeError(f"{path} missing: build it where the reference tree is mounted (oracle/build.py)")
        _ref_libs[name] = C.CDLL(str(path))
    return _ref_libs[name]


def ref_cpu_swiglu(inp):
    """The reference's CPUSwiGLU (tests/unittests/test_act.cu:13-25), unmodified."""
    rows, _, inter = inp.shape
    out = np.empty((rows, inter), inp.dtype)
    fn = ref_lib("libref_act.so").ref_cpu_swiglu_f16 if _is16(inp) else ref_lib("libref_act.so").ref_cpu_swiglu_f32
    fn(_ptr(np.ascontiguousarray(inp)), _ptr(out), C.c_int(rows), C.c_int(inter))
    return out


def ref_cpu_embedding(ids, table):
    """The reference's cpuEmbedding (tests/unittests/test_input_embedding.cu:35-41), fp32 only."""
    ids = np.ascontiguousarray(ids, np.int32)
    table = np.ascontiguousarray(table, np.float32)
    out = np.empty((ids.size, table.shape[1]), np.float32)
    ref_lib("libref_embedding.so").ref_cpu_embedding_f32(_ptr(ids), _ptr(out), _ptr(table), C.c_int(ids.size),
                                                         C.c_int(table.shape[1]), C.c_int(table.shape[0]))
    return out


def ref_cpu_fused_resid_rmsnorm(residual, decoder_out, bias, scale, eps):
    """The reference's CPUfusedresidandRMSNorm (tests/unittests/test_fused_addresidual_norm.cu:33-55):
    returns the overwritten decoder_out.  Only meaningful when every row is constant."""
    out = np.array(decoder_out, np.float32, copy=True)
    tokens, hidden = out.shape
    ref_lib("libref_norm.so").ref_cpu_fused_resid_rmsnorm_f32(
        _ptr(np.ascontiguousarray(residual, np.float32)), _ptr(out), _ptr(np.ascontiguousarray(bias, np.float32)),
        _ptr(np.ascontiguousarray(scale, np.float32)), _f(eps), C.c_int(hidden), C.c_int(tokens))
    return out


def ref_cpu_qkv_rope(QKV, bias, history_length, batch, seq_len, head_num, kv_head_num, head_size, rot_dim, base):
    """The reference's CPUfunc (tests/unittests/test_bias_and_RoPE.cu:12-76) in its own layout:
    returns q [b, s, head, d] and k [b, s, kv_head, d] (not transposed)."""
    QKV = np.ascontiguousarray(QKV, np.float32)
    q = np.zeros((batch, seq_len, head_num, head_size), np.float32)
    k = np.zeros((batch, seq_len, kv_head_num, head_size), np.float32)
    v = np.zeros((batch, seq_len, kv_head_num, head_size), np.float32)
    po = np.zeros(batch * seq_len, np.int32)
    hl = np.ascontiguousarray(history_length, np.int32)
    il = np.full(batch, seq_len, np.int32)
    ref_lib("libref_rope.so").ref_cpu_qkv_rope_f32(
        _ptr(q), _ptr(k), _ptr(v), _ptr(QKV), _ptr(np.ascontiguousarray(bias, np.float32)), _ptr(po), _ptr(hl),
        _ptr(il), C.c_int(batch), C.c_int(seq_len), C.c_int(batch * seq_len), C.c_int(head_num),
        C.c_int(kv_head_num), C.c_int(head_size), C.c_int(rot_dim), _f(base))
    return q, k


# ---- layout kernels either side of attention ---------------------------------------------------------

def build_causal_mask(q_lens, k_lens, max_q_len, max_k_len, dtype=np.float32):
    ql = np.ascontiguousarray(q_lens, np.int32)
    kl = np.ascontiguousarray(k_lens, np.int32)
    mask = np.empty((ql.size, max_q_len, max_k_len), dtype)
    lib().orc_build_causal_mask(_ptr(mask), _ptr(ql), _ptr(kl), _i64(ql.size), _i64(max_q_len), _i64(max_k_len),
                                _i64(mask.dtype.itemsize))
    return mask


def cal_padding_offset(input_lengths, max_q_len, fill=-1):
    """Returns (padding_offset [bs, max_q_len] with untouched entries = fill, cum_seqlens [bs+1])."""
    il = np.ascontiguousarray(input_lengths, np.int32)
    po = np.full((il.size, max_q_len), fill, np.int32)
    cum = np.empty(il.size + 1, np.int32)
    lib().orc_cal_padding_offset(_ptr(po), _ptr(cum), _ptr(il), _i64(il.size), _i64(max_q_len))
    return po, cum


def transpose_remove_padding(inp, padding_offset, num_tokens, fill=0):
    batch, heads, seq_len, head_size = inp.shape
    po = np.ascontiguousarray(padding_offset, np.int32)
    out = np.full((num_tokens, heads, head_size), fill, inp.dtype)
    lib().orc_transpose_remove_padding(_ptr(out), _ptr(np.ascontiguousarray(inp)), _ptr(po), _i64(batch), _i64(heads),
                                       _i64(seq_len), _i64(head_size), _i64(num_tokens), _i64(inp.dtype.itemsize))
    return out


def repeat_kv(dst, src, context_length, layer, heads):
    """Writes into a copy of dst [bs, heads, max_k_len, d] from src [layers, bs, kv_heads, max_seq, d]."""
    dst = np.array(dst, copy=True)
    _, batch, kv_heads, max_seq_len, head_size = src.shape
    cl = np.ascontiguousarray(context_length, np.int32)
    lib().orc_repeat_kv(_ptr(dst), _ptr(np.ascontiguousarray(src)), _ptr(cl), _i64(layer), _i64(batch), _i64(kv_heads),
                        _i64(heads), _i64(max_seq_len), _i64(dst.shape[2]), _i64(head_size), _i64(src.dtype.itemsize))
    return dst


def ref_cpu_causal_mask(q_lens, k_lens, max_q_len, max_k_len):
    """The reference's CPUbuildCasualMask (tests/unittests/test_casual_mask.cu:12-32)."""
    ql = np.ascontiguousarray(q_lens, np.int32)
    kl = np.ascontiguousarray(k_lens, np.int32)
    mask = np.empty((ql.size, max_q_len, max_k_len), np.float32)
    ref_lib("libref_layout.so").ref_cpu_causal_mask_f32(_ptr(mask), _ptr(ql), _ptr(kl), C.c_int(max_q_len),
                                                       C.c_int(max_k_len), C.c_int(ql.size))
    return mask


def decoder_masked_mha(qkv, bias, k_cache, v_cache, layer, step, rot_dim, base, rope_t=None):
    """qkv [bs, heads + 2*kv, d]; caches [layers, bs, kv, max_seq, d].  Returns
    (out [bs, heads, d], new_k_cache, new_v_cache, unrounded_fp32_out)."""
    batch, qkv_heads, d = qkv.shape
    _, _, kv_heads, max_seq_len, _ = k_cache.shape
    heads = qkv_heads - 2 * kv_heads
    kc, vc = np.array(k_cache, copy=True), np.array(v_cache, copy=True)
    out = np.empty((batch, heads, d), qkv.dtype)
    unr = np.empty((batch, heads, d), np.float32)
    _is16(qkv)
    lib().orc_decoder_masked_mha(_ptr(out), _ptr(np.ascontiguousarray(qkv)), _ptr(bias), _ptr(kc), _ptr(vc), _i64(layer),
                                 _i64(batch), _i64(heads), _i64(kv_heads), _i64(max_seq_len), _i64(d), _i64(step),
                                 _i32(rot_dim), _f(base), _f(float(step) if rope_t is None else rope_t),
                                 _i64(qkv.dtype.itemsize), _ptr(unr))
    return out, kc, vc, unr


def ref_cpu_masked_attn(q, k, v, k_cache, v_cache, step):
    """The reference's CPUMaskedAttn without RoPE (tests/unittests/test_fused_decoder_attention.cu:12-143).
    q [bs, heads, d], k, v [bs, kv, d], caches [bs, kv, step, d] fp32.  Returns (out, k_cache, v_cache)."""
    batch, heads, d = q.shape
    kv_heads = k.shape[1]
    kc, vc = np.array(k_cache, np.float32, copy=True), np.array(v_cache, np.float32, copy=True)
    assert kc.shape == (batch, kv_heads, step, d)
    out = np.empty((batch, heads, d), np.float32)
    f = lambda a: _ptr(np.ascontiguousarray(a, np.float32))
    qq, kk, vv = np.ascontiguousarray(q, np.float32), np.ascontiguousarray(k, np.float32), np.ascontiguousarray(v, np.float32)
    ref_lib("libref_mha.so").ref_cpu_masked_attn_f32(_ptr(qq), _ptr(kk), _ptr(vv), _ptr(kc), _ptr(vc), _ptr(out),
                                                    C.c_int(batch), C.c_int(heads), C.c_int(kv_heads), C.c_int(d),
                                                    C.c_int(step))
    return out, kc, vc
