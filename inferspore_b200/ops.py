"""torch-tensor front end of the C ABI, named after the reference's launchers.

PyTorch is plumbing here: it owns device memory and the current stream.  Each
function validates its arguments, picks the f32 or f16 entry point from the
tensor dtype and calls libispore_kernels.so on torch's current stream.
Nothing is computed in Python and there is no fallback path.

Validation comes first and never touches the device: every length / offset /
id tensor must be int32 (torch's default int64 would be read as pairs of
int32), all floating tensors of one call must share one dtype (float32 or
float16), and every output, scratch and cache tensor must have exactly the
shape the sizes passed to the C ABI are derived from — a mismatch would
otherwise become an out-of-bounds device write.  Shape and dtype errors raise
ValueError / TypeError before anything is launched; only then are device and
contiguity checked.

Argument order follows the reference launchers (src/kernels/*.h of
m0dulo/InferSpore); TensorWrapper shapes become tensor shapes.
"""
from __future__ import annotations

import threading
from typing import Optional, Sequence

import torch

from . import capi

_SUFFIX = {torch.float32: "f32", torch.float16: "f16"}


# ---- validation helpers (host only) ---------------------------------------------------------------

def _suffix(t: torch.Tensor) -> str:
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise TypeError(f"layer kernels take float32 or float16 tensors, got {t.dtype}") from None


def _floats(**tensors: Optional[torch.Tensor]) -> str:
    """All given (non-None) tensors share one storage type, float32 or float16; returns its suffix."""
    dtype, first = None, None
    for name, t in tensors.items():
        if t is None:
            continue
        if dtype is None:
            dtype, first = t.dtype, name
            _suffix(t)
        elif t.dtype != dtype:
            raise TypeError(f"{name} is {t.dtype} but {first} is {dtype}: one call takes one floating type")
    if dtype is None:
        raise ValueError("no floating tensor given")
    return _SUFFIX[dtype]


def _ints(**tensors: Optional[torch.Tensor]) -> None:
    for name, t in tensors.items():
        if t is not None and t.dtype != torch.int32:
            raise TypeError(f"{name} must be int32, got {t.dtype}")


def _shape(name: str, t: Optional[torch.Tensor], expected: Sequence[int]) -> None:
    if t is not None and tuple(t.shape) != tuple(expected):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(expected)}")


def _dims(name: str, t: torch.Tensor, n: int) -> None:
    if t.dim() != n:
        raise ValueError(f"{name} must have {n} dimensions, got shape {tuple(t.shape)}")


def _numel(name: str, t: Optional[torch.Tensor], n: int, at_least: bool = False) -> None:
    if t is None:
        return
    if (t.numel() < n) if at_least else (t.numel() != n):
        raise ValueError(f"{name} holds {t.numel()} elements, expected {'at least ' if at_least else ''}{n}")


def _dev(*tensors: Optional[torch.Tensor]) -> None:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("layer kernels take CUDA tensors (no CPU path exists)")
        if not t.is_contiguous():
            raise ValueError("layer kernels take contiguous tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors of one call must live on the same GPU")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_recording = threading.local()


def _call(name: str, ref: torch.Tensor, *args) -> None:
    lib = capi.load()
    record = getattr(_recording, "calls", None)
    if record is not None:  # inside prepare(): validated, not launched
        record.append(PreparedLaunch(getattr(lib, name), args, ref.device))
        return
    with torch.cuda.device(ref.device):
        capi.check(getattr(lib, name)(*args, _stream(ref)))


class PreparedLaunch:
    """One validated call of the C ABI bound to its buffers: calling it launches on torch's current
    stream of the tensors' device and does nothing else (no re-validation, no device switch — the
    tensors' device must be the current one).  The tensors it was prepared with must stay alive and
    in place, as for a captured CUDA graph."""

    __slots__ = ("fn", "args", "device")

    def __init__(self, fn, args, device):
        self.fn, self.args, self.device = fn, args, device

    def __call__(self) -> None:
        rc = self.fn(*self.args, torch.cuda.current_stream(self.device).cuda_stream)
        if rc != capi.ISPORE_OK:
            capi.check(rc)


def prepare(launcher, *args, **kwargs) -> PreparedLaunch:
    """Validates launcher(*args, **kwargs) once, without launching, and returns the bound call:
    for loops over fixed buffers, where per-call argument checks would cost more host time than a
    short kernel takes on the device."""
    _recording.calls = []
    try:
        launcher(*args, **kwargs)
        calls = _recording.calls
    finally:
        _recording.calls = None
    if len(calls) != 1:
        raise RuntimeError("prepare() takes a launcher that makes exactly one C ABI call")
    return calls[0]


def set_programmatic_launch(enable: bool) -> None:
    """Switches programmatic dependent launch on or off for the calling thread
    (ispore_set_programmatic_launch): back-to-back kernels of the library overlap one kernel's
    ramp-up with the tail of the one before; results are unchanged."""
    capi.load().ispore_set_programmatic_launch(1 if enable else 0)


# ---- launchers ------------------------------------------------------------------------------------

def launchFusedAddBiasResidualRMSNorm(residual: Optional[torch.Tensor], decoder_out: torch.Tensor,
                                      bias: Optional[torch.Tensor], scale: torch.Tensor, eps: float) -> None:
    """residual, decoder_out [tokens, hidden] updated in place (fused_addresidual_norm.h:9-15)."""
    _dims("decoder_out", decoder_out, 2)
    tokens, hidden = decoder_out.shape
    sfx = _floats(decoder_out=decoder_out, residual=residual, bias=bias, scale=scale)
    _shape("residual", residual, (tokens, hidden))
    _numel("bias", bias, hidden)
    _numel("scale", scale, hidden)
    _dev(residual, decoder_out, bias, scale)
    _call(f"ispore_add_residual_rmsnorm_{sfx}", decoder_out, _ptr(decoder_out), _ptr(residual),
          _ptr(bias), _ptr(scale), eps, tokens, hidden)


def launchRMSNorm(decoder_out: torch.Tensor, decoder_residual: Optional[torch.Tensor], gamma: torch.Tensor,
                  eps: float) -> None:
    """Plain RMSNorm in place; decoder_residual (optional) receives the un-normed input."""
    _dims("decoder_out", decoder_out, 2)
    tokens, hidden = decoder_out.shape
    sfx = _floats(decoder_out=decoder_out, decoder_residual=decoder_residual, gamma=gamma)
    _shape("decoder_residual", decoder_residual, (tokens, hidden))
    _numel("gamma", gamma, hidden)
    _dev(decoder_out, decoder_residual, gamma)
    _call(f"ispore_rmsnorm_{sfx}", decoder_out, _ptr(decoder_out), _ptr(decoder_residual),
          _ptr(gamma), eps, tokens, hidden)


def launchInputEmbedding(input_ids: torch.Tensor, output: torch.Tensor, embed_table: torch.Tensor) -> None:
    """output[t] = embed_table[input_ids[t]] (input_embedding.h:6-9).  input_ids is int32; an id
    outside the table zero-fills its row and sets a device status bit instead of reading out of
    bounds."""
    _ints(input_ids=input_ids)
    _dims("output", output, 2)
    _dims("embed_table", embed_table, 2)
    tokens, hidden = output.shape
    sfx = _floats(output=output, embed_table=embed_table)
    if input_ids.numel() != tokens:
        raise ValueError("input ids 1st shape should equal to 1st shape of output")
    if embed_table.shape[1] != hidden:
        raise ValueError(f"embed_table rows are {embed_table.shape[1]} long, output rows {hidden}")
    if embed_table.shape[0] < 1:
        raise ValueError("embed_table is empty")
    _dev(input_ids, output, embed_table)
    _call(f"ispore_input_embedding_{sfx}", output, _ptr(input_ids), _ptr(output), _ptr(embed_table),
          tokens, hidden, embed_table.shape[0])


def launchAddFusedQKVBiasTransposeAndRoPE(q_buf: torch.Tensor, k_buf: torch.Tensor, v_buf: torch.Tensor,
                                          QKV: torch.Tensor, qkv_bias: Optional[torch.Tensor],
                                          padding_offset: torch.Tensor, history_length: torch.Tensor,
                                          input_length: torch.Tensor, rotary_embedding_dim: int,
                                          rotary_embedding_base: float, max_position_embeddings: int = 4096,
                                          use_dynamic_ntk: bool = False) -> None:
    """QKV [tokens, heads+2*kv_heads, d] -> q [bs, heads, seq, d], k/v [bs, kv_heads, seq, d]
    (qkv_bias_and_RoPE.h:10-20)."""
    _dims("QKV", QKV, 3)
    _dims("q_buf", q_buf, 4)
    token_num, qkv_heads, head_size = QKV.shape
    batch, head_num, seq_len, _ = q_buf.shape
    sfx = _floats(QKV=QKV, q_buf=q_buf, k_buf=k_buf, v_buf=v_buf, qkv_bias=qkv_bias)
    _ints(padding_offset=padding_offset, history_length=history_length, input_length=input_length)
    if (qkv_heads - head_num) < 2 or (qkv_heads - head_num) % 2:
        raise ValueError(f"QKV holds {qkv_heads} heads per token, q_buf {head_num}: no whole number of k and v heads is left")
    kv_head_num = (qkv_heads - head_num) // 2
    _shape("q_buf", q_buf, (batch, head_num, seq_len, head_size))
    _shape("k_buf", k_buf, (batch, kv_head_num, seq_len, head_size))
    _shape("v_buf", v_buf, (batch, kv_head_num, seq_len, head_size))
    _numel("qkv_bias", qkv_bias, qkv_heads * head_size)
    _numel("padding_offset", padding_offset, token_num, at_least=True)
    _numel("history_length", history_length, batch)
    _numel("input_length", input_length, batch)
    if rotary_embedding_dim < 0 or rotary_embedding_dim > head_size or rotary_embedding_dim % 2:
        raise ValueError(f"rotary_embedding_dim {rotary_embedding_dim} must be even and at most the head size {head_size}")
    _dev(q_buf, k_buf, v_buf, QKV, qkv_bias, padding_offset, history_length, input_length)
    _call(f"ispore_qkv_bias_rope_transpose_{sfx}", QKV, _ptr(q_buf), _ptr(k_buf), _ptr(v_buf), _ptr(QKV),
          _ptr(qkv_bias), _ptr(padding_offset), _ptr(history_length), _ptr(input_length), batch, seq_len,
          token_num, head_num, kv_head_num, head_size, rotary_embedding_dim, rotary_embedding_base,
          max_position_embeddings, int(use_dynamic_ntk))


def launchRoPE(qkv_buf: torch.Tensor, step: int, head_num: int, kv_head_num: int, rotary_embedding_dim: int,
               rotary_embedding_base: float) -> None:
    """Decode-step RoPE in place on qkv_buf [batch, heads+2*kv_heads, d] at position step-1
    (qkv_bias_and_RoPE.h:22-25)."""
    _dims("qkv_buf", qkv_buf, 3)
    batch, qkv_heads, head_size = qkv_buf.shape
    sfx = _floats(qkv_buf=qkv_buf)
    if head_num < 1 or kv_head_num < 1 or head_num + 2 * kv_head_num != qkv_heads:
        raise ValueError(f"qkv_buf holds {qkv_heads} heads per sequence, not {head_num} + 2 * {kv_head_num}")
    if rotary_embedding_dim < 0 or rotary_embedding_dim > head_size or rotary_embedding_dim % 2:
        raise ValueError(f"rotary_embedding_dim {rotary_embedding_dim} must be even and at most the head size {head_size}")
    _dev(qkv_buf)
    _call(f"ispore_rope_decode_{sfx}", qkv_buf, _ptr(qkv_buf), batch, head_num, kv_head_num,
          head_size, step, rotary_embedding_dim, rotary_embedding_base)


def launchAct(input: torch.Tensor, out: torch.Tensor) -> None:
    """input [rows, 2, inter] -> out [rows, inter] = silu(gate) * up (act_kernel.h:8-9)."""
    _dims("input", input, 3)
    rows, two, inter = input.shape
    if two != 2:
        raise ValueError("input must be [rows, 2, inter]")
    sfx = _floats(input=input, out=out)
    _shape("out", out, (rows, inter))
    _dev(input, out)
    _call(f"ispore_silu_mul_{sfx}", input, _ptr(out), _ptr(input), rows, inter)


def launchConcatKVCache(k_src: torch.Tensor, v_src: torch.Tensor, layer_id: int, cur_query_length: torch.Tensor,
                        history_length: torch.Tensor, k_dst: torch.Tensor, v_dst: torch.Tensor) -> None:
    """k_src/v_src [bs, kv_heads, max_q_len, d] -> caches [layers, bs, kv_heads, max_seq, d]
    (or the 4-D single-layer cache) at history_length[b] (concat_past_kv.h:7-14)."""
    _dims("k_src", k_src, 4)
    batch, kv_heads, max_q_len, head_size = k_src.shape
    sfx = _floats(k_src=k_src, v_src=v_src, k_dst=k_dst, v_dst=v_dst)
    _ints(cur_query_length=cur_query_length, history_length=history_length)
    _shape("v_src", v_src, k_src.shape)
    if k_dst.dim() == 5:
        num_layers, max_seq_len = k_dst.shape[0], k_dst.shape[3]
        _shape("k_dst", k_dst, (num_layers, batch, kv_heads, max_seq_len, head_size))
    elif k_dst.dim() == 4:
        num_layers, max_seq_len = 1, k_dst.shape[2]
        _shape("k_dst", k_dst, (batch, kv_heads, max_seq_len, head_size))
    else:
        raise ValueError(f"k_dst must be [layers, bs, kv_heads, max_seq, d] or [bs, kv_heads, max_seq, d], got {tuple(k_dst.shape)}")
    _shape("v_dst", v_dst, k_dst.shape)
    if not 0 <= layer_id < num_layers:
        raise ValueError(f"layer_id {layer_id} outside the cache's {num_layers} layer(s)")
    _numel("cur_query_length", cur_query_length, batch)
    _numel("history_length", history_length, batch)
    _dev(k_src, v_src, cur_query_length, history_length, k_dst, v_dst)
    _call(f"ispore_concat_kv_{sfx}", k_src, _ptr(k_dst), _ptr(v_dst), _ptr(k_src), _ptr(v_src),
          _ptr(cur_query_length), _ptr(history_length), layer_id, num_layers, batch, kv_heads, max_q_len,
          max_seq_len, head_size)


def launchScaleMaskAndSoftmax(qk: torch.Tensor, mask: torch.Tensor, attn_score: torch.Tensor, scale: float) -> None:
    """qk, attn_score [bs, heads, q, k]; mask [bs, q, k] (attn_softmax_kernel.h:7-11)."""
    _dims("qk", qk, 4)
    batch, heads, q_len, k_len = qk.shape
    sfx = _floats(qk=qk, mask=mask, attn_score=attn_score)
    _shape("attn_score", attn_score, qk.shape)
    _shape("mask", mask, (batch, q_len, k_len))
    _dev(qk, mask, attn_score)
    _call(f"ispore_scale_mask_softmax_{sfx}", qk, _ptr(attn_score), _ptr(qk), _ptr(mask), batch, heads,
          q_len, k_len, scale)


def launchScaleCausalSoftmax(qk: torch.Tensor, q_lens: torch.Tensor, k_lens: torch.Tensor, attn_score: torch.Tensor,
                             scale: float) -> None:
    """launchBuildCausalMasks + launchScaleMaskAndSoftmax in one kernel: the mask comes from the
    int32 length arrays q_lens, k_lens [bs] and is never materialised."""
    _dims("qk", qk, 4)
    batch, heads, q_len, k_len = qk.shape
    sfx = _floats(qk=qk, attn_score=attn_score)
    _ints(q_lens=q_lens, k_lens=k_lens)
    _shape("attn_score", attn_score, qk.shape)
    _numel("q_lens", q_lens, batch)
    _numel("k_lens", k_lens, batch)
    _dev(qk, q_lens, k_lens, attn_score)
    _call(f"ispore_scale_causal_softmax_{sfx}", qk, _ptr(attn_score), _ptr(qk), _ptr(q_lens), _ptr(k_lens),
          batch, heads, q_len, k_len, scale)


def _check_sampling(rows: int, uniform: Optional[torch.Tensor], sampled_ids: Optional[torch.Tensor]) -> None:
    if uniform is None:
        return
    if uniform.dtype != torch.float32:
        raise TypeError(f"uniform must be float32, got {uniform.dtype}")
    if sampled_ids is None:
        raise ValueError("uniform given without sampled_ids")
    _ints(sampled_ids=sampled_ids)
    _numel("uniform", uniform, rows)
    _numel("sampled_ids", sampled_ids, rows)


def launchTopKforBeamSearch(probs: torch.Tensor, topk_ids: Optional[torch.Tensor], topk_vals: Optional[torch.Tensor],
                            final_topk_ids: torch.Tensor, final_topk_vals: torch.Tensor, index_offset: int = 0,
                            uniform: Optional[torch.Tensor] = None, temperature: float = 1.0,
                            sampled_ids: Optional[torch.Tensor] = None) -> None:
    """probs [rows, vocab] -> final_topk_ids/vals [rows, K]; topk_ids/vals are the
    [rows, slices, K] scratch of the reference launcher (topK.h:41-46; both None: one CTA per row).
    With `uniform` the merge also samples one id per row into sampled_ids."""
    _dims("probs", probs, 2)
    _dims("final_topk_ids", final_topk_ids, 2)
    rows, vocab = probs.shape
    K = final_topk_ids.shape[1]
    sfx = _floats(probs=probs, topk_vals=topk_vals, final_topk_vals=final_topk_vals)
    _ints(topk_ids=topk_ids, final_topk_ids=final_topk_ids)
    _shape("final_topk_ids", final_topk_ids, (rows, K))
    _shape("final_topk_vals", final_topk_vals, (rows, K))
    if (topk_ids is None) != (topk_vals is None):
        raise ValueError("topk_ids and topk_vals (the scratch) come together or not at all")
    slices = 0
    if topk_ids is not None:
        per_slice = max(1, rows * K)
        if topk_ids.numel() != topk_vals.numel() or topk_ids.numel() % per_slice or topk_ids.numel() < per_slice:
            raise ValueError(f"scratch must be [rows, slices, K] ids and values of equal size, got {tuple(topk_ids.shape)} "
                             f"and {tuple(topk_vals.shape)} for rows={rows}, K={K}")
        slices = topk_ids.numel() // per_slice
    _check_sampling(rows, uniform, sampled_ids)
    _dev(probs, topk_ids, topk_vals, final_topk_ids, final_topk_vals, uniform, sampled_ids)
    _call(f"ispore_topk_{sfx}", probs, _ptr(probs), rows, vocab, K, _ptr(topk_ids), _ptr(topk_vals),
          slices, _ptr(final_topk_ids), _ptr(final_topk_vals), index_offset, _ptr(uniform), temperature,
          _ptr(sampled_ids))


def launchTopKMerge(cand_ids: torch.Tensor, cand_vals: torch.Tensor, final_topk_ids: torch.Tensor,
                    final_topk_vals: torch.Tensor, uniform: Optional[torch.Tensor] = None,
                    temperature: float = 1.0, sampled_ids: Optional[torch.Tensor] = None) -> None:
    """cand_ids/vals [rows, lists, K] -> final [rows, K] (round 2 of the top-K)."""
    _dims("cand_ids", cand_ids, 3)
    rows, lists, K = cand_ids.shape
    sfx = _floats(cand_vals=cand_vals, final_topk_vals=final_topk_vals)
    _ints(cand_ids=cand_ids, final_topk_ids=final_topk_ids)
    _shape("cand_vals", cand_vals, cand_ids.shape)
    _shape("final_topk_ids", final_topk_ids, (rows, K))
    _shape("final_topk_vals", final_topk_vals, (rows, K))
    _check_sampling(rows, uniform, sampled_ids)
    _dev(cand_ids, cand_vals, final_topk_ids, final_topk_vals, uniform, sampled_ids)
    _call(f"ispore_topk_merge_{sfx}", cand_vals, _ptr(cand_ids), _ptr(cand_vals), rows, lists, K,
          _ptr(final_topk_ids), _ptr(final_topk_vals), _ptr(uniform), temperature, _ptr(sampled_ids))


def launchTopKMergeGathered(gathered: torch.Tensor, lists: int, rows: int, K: int, final_topk_ids: torch.Tensor,
                            final_topk_vals: torch.Tensor, uniform: Optional[torch.Tensor] = None,
                            temperature: float = 1.0, sampled_ids: Optional[torch.Tensor] = None) -> None:
    """Round 2 of the top-K straight from an all-gather's output: `gathered` is a uint8 tensor
    [lists, record] in which rank l's record holds its [rows, K] int32 ids followed by its
    [rows, K] values (the storage type of final_topk_vals), padded to a multiple of 16 bytes —
    the layout packed_record_bytes() describes.  No re-layout copy is needed between the
    collective and the merge."""
    sfx = _floats(final_topk_vals=final_topk_vals)
    _ints(final_topk_ids=final_topk_ids)
    if gathered.dtype != torch.uint8:
        raise TypeError(f"gathered must be uint8, got {gathered.dtype}")
    record = packed_record_bytes(rows, K, final_topk_vals.dtype)
    _shape("gathered", gathered, (lists, record))
    _shape("final_topk_ids", final_topk_ids, (rows, K))
    _shape("final_topk_vals", final_topk_vals, (rows, K))
    _check_sampling(rows, uniform, sampled_ids)
    _dev(gathered, final_topk_ids, final_topk_vals, uniform, sampled_ids)
    esize = final_topk_vals.element_size()
    ids_bytes = rows * K * 4
    _call(f"ispore_topk_merge_strided_{sfx}", final_topk_vals, gathered.data_ptr(), gathered.data_ptr() + ids_bytes,
          rows, lists, K, record // 4, K, record // esize, K, _ptr(final_topk_ids), _ptr(final_topk_vals),
          _ptr(uniform), temperature, _ptr(sampled_ids))


def packed_record_bytes(rows: int, K: int, dtype: torch.dtype) -> int:
    """Bytes of one rank's packed candidate record: [rows, K] int32 ids, then [rows, K] values,
    rounded up to a multiple of 16 bytes."""
    esize = torch.empty((), dtype=dtype).element_size()
    return -(-(rows * K * (4 + esize)) // 16) * 16


def launchSampling(topk_id: torch.Tensor, topk_val: torch.Tensor, uniform: torch.Tensor, output_id: torch.Tensor,
                   temperature: float) -> None:
    """Inverse-CDF draw from softmax(topk_val / temperature) with caller-drawn uniforms."""
    _dims("topk_id", topk_id, 2)
    rows, K = topk_id.shape
    sfx = _floats(topk_val=topk_val)
    _ints(topk_id=topk_id)
    _shape("topk_val", topk_val, (rows, K))
    _check_sampling(rows, uniform, output_id)
    _dev(topk_id, topk_val, uniform, output_id)
    _call(f"ispore_sampling_{sfx}", topk_val, _ptr(topk_id), _ptr(topk_val), _ptr(uniform),
          _ptr(output_id), rows, K, temperature)


def launchBuildCausalMasks(mask: torch.Tensor, q_lens: torch.Tensor, k_lens: torch.Tensor) -> None:
    """mask [bs, max_q_len, max_k_len] of 0/1 from per-sequence lengths (build_casual_mask.h:7-10)."""
    _dims("mask", mask, 3)
    batch, max_q, max_k = mask.shape
    sfx = _floats(mask=mask)
    _ints(q_lens=q_lens, k_lens=k_lens)
    _numel("q_lens", q_lens, batch)
    _numel("k_lens", k_lens, batch)
    _dev(mask, q_lens, k_lens)
    _call(f"ispore_build_causal_mask_{sfx}", mask, _ptr(mask), _ptr(q_lens), _ptr(k_lens), batch, max_q, max_k)


def launchCalPaddingoffset(padding_offset: torch.Tensor, cum_seqlens: torch.Tensor, input_lengths: torch.Tensor) -> None:
    """padding_offset [bs, max_q_len], cum_seqlens [bs+1] from input_lengths [bs] (cal_paddingoffset.h:8-11)."""
    _dims("padding_offset", padding_offset, 2)
    _ints(padding_offset=padding_offset, cum_seqlens=cum_seqlens, input_lengths=input_lengths)
    batch, max_q = padding_offset.shape
    if input_lengths.numel() != batch or cum_seqlens.numel() != batch + 1:
        raise ValueError("input lengths must be [bs] and cum_seqlens [bs + 1]")
    _dev(padding_offset, cum_seqlens, input_lengths)
    _call("ispore_cal_padding_offset", padding_offset, _ptr(padding_offset), _ptr(cum_seqlens), _ptr(input_lengths),
          batch, max_q)


def launchTransposeOutRemovePadding(qkv_buf_w_pad: torch.Tensor, padding_offset: torch.Tensor,
                                    qkv_buf_wo_pad: torch.Tensor) -> None:
    """[bs, heads, seq, d] -> [num_tokens, heads, d] (fused_transpose_and_remv_pad.h:7-10)."""
    _dims("qkv_buf_w_pad", qkv_buf_w_pad, 4)
    _dims("qkv_buf_wo_pad", qkv_buf_wo_pad, 3)
    batch, heads, seq_len, head_size = qkv_buf_w_pad.shape
    num_tokens = qkv_buf_wo_pad.shape[0]
    sfx = _floats(qkv_buf_w_pad=qkv_buf_w_pad, qkv_buf_wo_pad=qkv_buf_wo_pad)
    _ints(padding_offset=padding_offset)
    _shape("qkv_buf_wo_pad", qkv_buf_wo_pad, (num_tokens, heads, head_size))
    if num_tokens > batch * seq_len:
        raise ValueError(f"{num_tokens} packed tokens cannot come from {batch} x {seq_len} padded positions")
    _numel("padding_offset", padding_offset, num_tokens, at_least=True)
    _dev(qkv_buf_w_pad, padding_offset, qkv_buf_wo_pad)
    _call(f"ispore_transpose_remove_padding_{sfx}", qkv_buf_w_pad, _ptr(qkv_buf_wo_pad),
          _ptr(qkv_buf_w_pad), _ptr(padding_offset), batch, heads, seq_len, head_size, num_tokens)


def launchRepeatKVCache(k_cache_src: torch.Tensor, v_cache_src: torch.Tensor, context_length: torch.Tensor,
                        layer_id: int, k_cache_dst: torch.Tensor, v_cache_dst: torch.Tensor) -> None:
    """caches [layers, bs, kv_heads, max_seq, d] -> [bs, heads, max_k_len, d] (repeat_kv.h:7-13)."""
    _dims("k_cache_src", k_cache_src, 5)
    _dims("k_cache_dst", k_cache_dst, 4)
    num_layers, batch, kv_heads, max_seq_len, head_size = k_cache_src.shape
    heads, max_k_len = k_cache_dst.shape[1], k_cache_dst.shape[2]
    sfx = _floats(k_cache_src=k_cache_src, v_cache_src=v_cache_src, k_cache_dst=k_cache_dst, v_cache_dst=v_cache_dst)
    _ints(context_length=context_length)
    _shape("v_cache_src", v_cache_src, k_cache_src.shape)
    _shape("k_cache_dst", k_cache_dst, (batch, heads, max_k_len, head_size))
    _shape("v_cache_dst", v_cache_dst, k_cache_dst.shape)
    if kv_heads < 1 or heads % kv_heads:
        raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
    if not 0 <= layer_id < num_layers:
        raise ValueError(f"layer_id {layer_id} outside the cache's {num_layers} layer(s)")
    _numel("context_length", context_length, batch)
    _dev(k_cache_src, v_cache_src, context_length, k_cache_dst, v_cache_dst)
    _call(f"ispore_repeat_kv_{sfx}", k_cache_src, _ptr(k_cache_dst), _ptr(v_cache_dst),
          _ptr(k_cache_src), _ptr(v_cache_src), _ptr(context_length), layer_id, num_layers, batch, kv_heads, heads,
          max_seq_len, max_k_len, head_size)


def decoderMaskedMHAWorkspaceBytes(batch: int, head_num: int, kv_head_num: int, head_size: int, step: int) -> int:
    """Bytes of scratch launchDecoderMaskedMHA can use to split long sequences over several CTAs."""
    return int(capi.load().ispore_decoder_masked_mha_workspace_bytes(batch, head_num, kv_head_num, head_size, step))


def launchDecoderMaskedMHA(qkv_buf: torch.Tensor, qkv_bias: Optional[torch.Tensor], layer_id: int,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, finished: Optional[torch.Tensor], step: int,
                           mha_output: torch.Tensor, rotary_embedding_dim: int, rotary_embedding_base: float,
                           workspace: Optional[torch.Tensor] = None, rope_timestep: Optional[float] = None) -> None:
    """qkv_buf [bs, heads+2*kv_heads, d], caches [layers, bs, kv_heads, max_seq, d] (updated at
    step-1), mha_output [bs, heads, d] (fused_decoder_self_attention.h:10-18).  `finished` is
    accepted and unused, as in the reference; rope_timestep defaults to `step`, the reference's
    choice; workspace is any CUDA tensor used as scratch (see decoderMaskedMHAWorkspaceBytes)."""
    _dims("qkv_buf", qkv_buf, 3)
    _dims("k_cache", k_cache, 5)
    batch, qkv_heads, head_size = qkv_buf.shape
    num_layers, _, kv_heads, max_seq_len, _ = k_cache.shape
    sfx = _floats(qkv_buf=qkv_buf, qkv_bias=qkv_bias, k_cache=k_cache, v_cache=v_cache, mha_output=mha_output)
    heads = qkv_heads - 2 * kv_heads
    if kv_heads < 1 or heads < 1 or heads % kv_heads:
        raise ValueError(f"qkv_buf holds {qkv_heads} heads per sequence and the cache {kv_heads} kv heads: "
                         f"{heads} query heads are not a positive multiple of them")
    _shape("k_cache", k_cache, (num_layers, batch, kv_heads, max_seq_len, head_size))
    _shape("v_cache", v_cache, k_cache.shape)
    _shape("mha_output", mha_output, (batch, heads, head_size))
    _numel("qkv_bias", qkv_bias, qkv_heads * head_size)
    if not 0 <= layer_id < num_layers:
        raise ValueError(f"layer_id {layer_id} outside the cache's {num_layers} layer(s)")
    if not 1 <= step <= max_seq_len:
        raise ValueError(f"step {step} outside [1, max_seq_len = {max_seq_len}]")
    _dev(qkv_buf, qkv_bias, k_cache, v_cache, mha_output, workspace)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _call(f"ispore_decoder_masked_mha_{sfx}", qkv_buf, _ptr(mha_output), _ptr(qkv_buf), _ptr(qkv_bias),
          _ptr(k_cache), _ptr(v_cache), layer_id, num_layers, batch, heads, kv_heads, max_seq_len,
          head_size, step, rotary_embedding_dim, rotary_embedding_base,
          float(step) if rope_timestep is None else rope_timestep, _ptr(workspace), ws_bytes)
