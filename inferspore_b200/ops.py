"""torch-tensor front end of the C ABI, named after the reference's launchers.

PyTorch is plumbing here: it owns device memory and the current stream.  Each
function checks device / dtype / contiguity, picks the f32 or f16 entry point
from the tensor dtype and calls libispore_kernels.so on torch's current stream.
Nothing is computed in Python and there is no fallback path.

Argument order follows the reference launchers (src/kernels/*.h of
m0dulo/InferSpore); TensorWrapper shapes become tensor shapes.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import capi

_SUFFIX = {torch.float32: "f32", torch.float16: "f16"}


def _suffix(t: torch.Tensor) -> str:
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise TypeError(f"layer kernels take float32 or float16 tensors, got {t.dtype}") from None


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


def _call(name: str, ref: torch.Tensor, *args) -> None:
    lib = capi.load()
    with torch.cuda.device(ref.device):
        capi.check(getattr(lib, name)(*args, _stream(ref)))


def launchFusedAddBiasResidualRMSNorm(residual: Optional[torch.Tensor], decoder_out: torch.Tensor,
                                      bias: Optional[torch.Tensor], scale: torch.Tensor, eps: float) -> None:
    """residual, decoder_out [tokens, hidden] updated in place (fused_addresidual_norm.h:9-15)."""
    _dev(residual, decoder_out, bias, scale)
    tokens, hidden = decoder_out.shape
    _call(f"ispore_add_residual_rmsnorm_{_suffix(decoder_out)}", decoder_out, _ptr(decoder_out), _ptr(residual),
          _ptr(bias), _ptr(scale), eps, tokens, hidden)


def launchRMSNorm(decoder_out: torch.Tensor, decoder_residual: Optional[torch.Tensor], gamma: torch.Tensor,
                  eps: float) -> None:
    """Plain RMSNorm in place; decoder_residual (optional) receives the un-normed input."""
    _dev(decoder_out, decoder_residual, gamma)
    tokens, hidden = decoder_out.shape
    _call(f"ispore_rmsnorm_{_suffix(decoder_out)}", decoder_out, _ptr(decoder_out), _ptr(decoder_residual),
          _ptr(gamma), eps, tokens, hidden)


def launchInputEmbedding(input_ids: torch.Tensor, output: torch.Tensor, embed_table: torch.Tensor,
                         check_ids: bool = True) -> None:
    """output[t] = embed_table[input_ids[t]] (input_embedding.h:6-9).  input_ids is int32."""
    _dev(input_ids, output, embed_table)
    if input_ids.dtype != torch.int32:
        raise TypeError("input_ids must be int32")
    tokens, hidden = output.shape
    if input_ids.numel() != tokens:
        raise ValueError("input ids 1st shape should equal to 1st shape of output")
    vocab = embed_table.shape[0] if check_ids else 0
    _call(f"ispore_input_embedding_{_suffix(output)}", output, _ptr(input_ids), _ptr(output), _ptr(embed_table),
          tokens, hidden, vocab)


def launchAddFusedQKVBiasTransposeAndRoPE(q_buf: torch.Tensor, k_buf: torch.Tensor, v_buf: torch.Tensor,
                                          QKV: torch.Tensor, qkv_bias: Optional[torch.Tensor],
                                          padding_offset: torch.Tensor, history_length: torch.Tensor,
                                          input_length: torch.Tensor, rotary_embedding_dim: int,
                                          rotary_embedding_base: float, max_position_embeddings: int = 4096,
                                          use_dynamic_ntk: bool = False) -> None:
    """QKV [tokens, heads+2*kv_heads, d] -> q [bs, heads, seq, d], k/v [bs, kv_heads, seq, d]
    (qkv_bias_and_RoPE.h:10-20)."""
    _dev(q_buf, k_buf, v_buf, QKV, qkv_bias, padding_offset, history_length, input_length)
    token_num, qkv_heads, head_size = QKV.shape
    batch, head_num, seq_len, _ = q_buf.shape
    kv_head_num = (qkv_heads - head_num) // 2
    _call(f"ispore_qkv_bias_rope_transpose_{_suffix(QKV)}", QKV, _ptr(q_buf), _ptr(k_buf), _ptr(v_buf), _ptr(QKV),
          _ptr(qkv_bias), _ptr(padding_offset), _ptr(history_length), _ptr(input_length), batch, seq_len,
          token_num, head_num, kv_head_num, head_size, rotary_embedding_dim, rotary_embedding_base,
          max_position_embeddings, int(use_dynamic_ntk))


def launchRoPE(qkv_buf: torch.Tensor, step: int, head_num: int, kv_head_num: int, rotary_embedding_dim: int,
               rotary_embedding_base: float) -> None:
    """Decode-step RoPE in place on qkv_buf [batch, heads+2*kv_heads, d] at position step-1
    (qkv_bias_and_RoPE.h:22-25)."""
    _dev(qkv_buf)
    batch, _, head_size = qkv_buf.shape
    _call(f"ispore_rope_decode_{_suffix(qkv_buf)}", qkv_buf, _ptr(qkv_buf), batch, head_num, kv_head_num,
          head_size, step, rotary_embedding_dim, rotary_embedding_base)


def launchAct(input: torch.Tensor, out: torch.Tensor) -> None:
    """input [rows, 2, inter] -> out [rows, inter] = silu(gate) * up (act_kernel.h:8-9)."""
    _dev(input, out)
    rows, two, inter = input.shape
    if two != 2:
        raise ValueError("input must be [rows, 2, inter]")
    _call(f"ispore_silu_mul_{_suffix(input)}", input, _ptr(out), _ptr(input), rows, inter)


def launchConcatKVCache(k_src: torch.Tensor, v_src: torch.Tensor, layer_id: int, cur_query_length: torch.Tensor,
                        history_length: torch.Tensor, k_dst: torch.Tensor, v_dst: torch.Tensor) -> None:
    """k_src/v_src [bs, kv_heads, max_q_len, d] -> caches [layers, bs, kv_heads, max_seq, d]
    at history_length[b] (concat_past_kv.h:7-14)."""
    _dev(k_src, v_src, cur_query_length, history_length, k_dst, v_dst)
    batch, kv_heads, max_q_len, head_size = k_src.shape
    if k_dst.dim() == 5:
        num_layers, max_seq_len = k_dst.shape[0], k_dst.shape[3]
    else:
        num_layers, max_seq_len = 1, k_dst.shape[2]
    _call(f"ispore_concat_kv_{_suffix(k_src)}", k_src, _ptr(k_dst), _ptr(v_dst), _ptr(k_src), _ptr(v_src),
          _ptr(cur_query_length), _ptr(history_length), layer_id, num_layers, batch, kv_heads, max_q_len,
          max_seq_len, head_size)


def launchScaleMaskAndSoftmax(qk: torch.Tensor, mask: torch.Tensor, attn_score: torch.Tensor, scale: float) -> None:
    """qk, attn_score [bs, heads, q, k]; mask [bs, q, k] (attn_softmax_kernel.h:7-11)."""
    _dev(qk, mask, attn_score)
    batch, heads, q_len, k_len = qk.shape
    _call(f"ispore_scale_mask_softmax_{_suffix(qk)}", qk, _ptr(attn_score), _ptr(qk), _ptr(mask), batch, heads,
          q_len, k_len, scale)


def launchScaleCausalSoftmax(qk: torch.Tensor, q_lens: torch.Tensor, k_lens: torch.Tensor, attn_score: torch.Tensor,
                             scale: float) -> None:
    """launchBuildCausalMasks + launchScaleMaskAndSoftmax in one kernel: the mask comes from the
    int32 length arrays q_lens, k_lens [bs] and is never materialised."""
    _dev(qk, q_lens, k_lens, attn_score)
    batch, heads, q_len, k_len = qk.shape
    _call(f"ispore_scale_causal_softmax_{_suffix(qk)}", qk, _ptr(attn_score), _ptr(qk), _ptr(q_lens), _ptr(k_lens),
          batch, heads, q_len, k_len, scale)


def launchTopKforBeamSearch(probs: torch.Tensor, topk_ids: torch.Tensor, topk_vals: torch.Tensor,
                            final_topk_ids: torch.Tensor, final_topk_vals: torch.Tensor, index_offset: int = 0,
                            uniform: Optional[torch.Tensor] = None, temperature: float = 1.0,
                            sampled_ids: Optional[torch.Tensor] = None) -> None:
    """probs [rows, vocab] -> final_topk_ids/vals [rows, K]; topk_ids/vals are the
    [rows, slices, K] scratch of the reference launcher (topK.h:41-46).  With
    `uniform` the merge also samples one id per row into sampled_ids."""
    _dev(probs, topk_ids, topk_vals, final_topk_ids, final_topk_vals, uniform, sampled_ids)
    rows, vocab = probs.shape
    K = final_topk_ids.shape[1]
    slices = topk_ids.numel() // max(1, rows * K)
    _call(f"ispore_topk_{_suffix(probs)}", probs, _ptr(probs), rows, vocab, K, _ptr(topk_ids), _ptr(topk_vals),
          slices, _ptr(final_topk_ids), _ptr(final_topk_vals), index_offset, _ptr(uniform), temperature,
          _ptr(sampled_ids))


def launchTopKMerge(cand_ids: torch.Tensor, cand_vals: torch.Tensor, final_topk_ids: torch.Tensor,
                    final_topk_vals: torch.Tensor, uniform: Optional[torch.Tensor] = None,
                    temperature: float = 1.0, sampled_ids: Optional[torch.Tensor] = None) -> None:
    """cand_ids/vals [rows, lists, K] -> final [rows, K] (round 2 of the top-K)."""
    _dev(cand_ids, cand_vals, final_topk_ids, final_topk_vals, uniform, sampled_ids)
    rows, lists, K = cand_ids.shape
    _call(f"ispore_topk_merge_{_suffix(cand_vals)}", cand_vals, _ptr(cand_ids), _ptr(cand_vals), rows, lists, K,
          _ptr(final_topk_ids), _ptr(final_topk_vals), _ptr(uniform), temperature, _ptr(sampled_ids))


def launchSampling(topk_id: torch.Tensor, topk_val: torch.Tensor, uniform: torch.Tensor, output_id: torch.Tensor,
                   temperature: float) -> None:
    """Inverse-CDF draw from softmax(topk_val / temperature) with caller-drawn uniforms."""
    _dev(topk_id, topk_val, uniform, output_id)
    rows, K = topk_id.shape
    _call(f"ispore_sampling_{_suffix(topk_val)}", topk_val, _ptr(topk_id), _ptr(topk_val), _ptr(uniform),
          _ptr(output_id), rows, K, temperature)


def launchBuildCausalMasks(mask: torch.Tensor, q_lens: torch.Tensor, k_lens: torch.Tensor) -> None:
    """mask [bs, max_q_len, max_k_len] of 0/1 from per-sequence lengths (build_casual_mask.h:7-10)."""
    _dev(mask, q_lens, k_lens)
    batch, max_q, max_k = mask.shape
    _call(f"ispore_build_causal_mask_{_suffix(mask)}", mask, _ptr(mask), _ptr(q_lens), _ptr(k_lens), batch, max_q, max_k)


def launchCalPaddingoffset(padding_offset: torch.Tensor, cum_seqlens: torch.Tensor, input_lengths: torch.Tensor) -> None:
    """padding_offset [bs, max_q_len], cum_seqlens [bs+1] from input_lengths [bs] (cal_paddingoffset.h:8-11)."""
    _dev(padding_offset, cum_seqlens, input_lengths)
    batch, max_q = padding_offset.shape
    if input_lengths.shape[0] != batch or cum_seqlens.shape[0] != batch + 1:
        raise ValueError("input lengths must be [bs] and cum_seqlens [bs + 1]")
    _call("ispore_cal_padding_offset", padding_offset, _ptr(padding_offset), _ptr(cum_seqlens), _ptr(input_lengths),
          batch, max_q)


def launchTransposeOutRemovePadding(qkv_buf_w_pad: torch.Tensor, padding_offset: torch.Tensor,
                                    qkv_buf_wo_pad: torch.Tensor) -> None:
    """[bs, heads, seq, d] -> [num_tokens, heads, d] (fused_transpose_and_remv_pad.h:7-10)."""
    _dev(qkv_buf_w_pad, padding_offset, qkv_buf_wo_pad)
    batch, heads, seq_len, head_size = qkv_buf_w_pad.shape
    num_tokens = qkv_buf_wo_pad.shape[0]
    _call(f"ispore_transpose_remove_padding_{_suffix(qkv_buf_w_pad)}", qkv_buf_w_pad, _ptr(qkv_buf_wo_pad),
          _ptr(qkv_buf_w_pad), _ptr(padding_offset), batch, heads, seq_len, head_size, num_tokens)


def launchRepeatKVCache(k_cache_src: torch.Tensor, v_cache_src: torch.Tensor, context_length: torch.Tensor,
                        layer_id: int, k_cache_dst: torch.Tensor, v_cache_dst: torch.Tensor) -> None:
    """caches [layers, bs, kv_heads, max_seq, d] -> [bs, heads, max_k_len, d] (repeat_kv.h:7-13)."""
    _dev(k_cache_src, v_cache_src, context_length, k_cache_dst, v_cache_dst)
    num_layers, batch, kv_heads, max_seq_len, head_size = k_cache_src.shape
    heads, max_k_len = k_cache_dst.shape[1], k_cache_dst.shape[2]
    _call(f"ispore_repeat_kv_{_suffix(k_cache_src)}", k_cache_src, _ptr(k_cache_dst), _ptr(v_cache_dst),
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
    _dev(qkv_buf, qkv_bias, k_cache, v_cache, mha_output, workspace)
    batch, qkv_heads, head_size = qkv_buf.shape
    num_layers, _, kv_heads, max_seq_len, _ = k_cache.shape
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _call(f"ispore_decoder_masked_mha_{_suffix(qkv_buf)}", qkv_buf, _ptr(mha_output), _ptr(qkv_buf), _ptr(qkv_bias),
          _ptr(k_cache), _ptr(v_cache), layer_id, num_layers, batch, qkv_heads - 2 * kv_heads, kv_heads, max_seq_len,
          head_size, step, rotary_embedding_dim, rotary_embedding_base,
          float(step) if rope_timestep is None else rope_timestep, _ptr(workspace), ws_bytes)
