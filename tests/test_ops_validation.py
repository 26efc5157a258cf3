"""Host-side argument validation of the torch front end (inferspore_b200/ops.py), on CPU.

Every launcher checks dtypes and shapes before it looks at the device: a length tensor in torch's
default int64, tensors of different floating types in one call, or an output / scratch / cache
tensor whose shape does not match the sizes handed to the C ABI would otherwise become a wrong
result or an out-of-bounds device write.  The checks run before the device check, so CPU tensors
exercise them here; a well-formed call on CPU tensors must still be refused (there is no CPU path).
"""
import pytest
import torch

from inferspore_b200 import ops

f32, f16, i32, i64 = torch.float32, torch.float16, torch.int32, torch.int64


def z(*shape, dtype=f32):
    return torch.zeros(shape, dtype=dtype)


def good_calls():
    """One well-formed call per launcher (CPU tensors)."""
    B, H, KV, S, D, T = 2, 4, 2, 8, 16, 13
    return {
        "add_residual_rmsnorm": lambda: ops.launchFusedAddBiasResidualRMSNorm(z(T, 64), z(T, 64), z(64), z(64), 1e-6),
        "rmsnorm": lambda: ops.launchRMSNorm(z(T, 64), z(T, 64), z(64), 1e-6),
        "embedding": lambda: ops.launchInputEmbedding(z(T, dtype=i32), z(T, 64), z(100, 64)),
        "qkv_rope": lambda: ops.launchAddFusedQKVBiasTransposeAndRoPE(
            z(B, H, S, D), z(B, KV, S, D), z(B, KV, S, D), z(T, H + 2 * KV, D), z((H + 2 * KV) * D), z(T, dtype=i32),
            z(B, dtype=i32), z(B, dtype=i32), D, 10000.0),
        "rope_decode": lambda: ops.launchRoPE(z(B, H + 2 * KV, D), 5, H, KV, D, 10000.0),
        "act": lambda: ops.launchAct(z(T, 2, 32), z(T, 32)),
        "concat_kv": lambda: ops.launchConcatKVCache(z(B, KV, S, D), z(B, KV, S, D), 1, z(B, dtype=i32), z(B, dtype=i32),
                                                     z(3, B, KV, 32, D), z(3, B, KV, 32, D)),
        "softmax": lambda: ops.launchScaleMaskAndSoftmax(z(B, H, S, S), z(B, S, S), z(B, H, S, S), 0.5),
        "causal_softmax": lambda: ops.launchScaleCausalSoftmax(z(B, H, S, S), z(B, dtype=i32), z(B, dtype=i32),
                                                               z(B, H, S, S), 0.5),
        "topk": lambda: ops.launchTopKforBeamSearch(z(T, 100), z(T, 8, 5, dtype=i32), z(T, 8, 5), z(T, 5, dtype=i32),
                                                    z(T, 5), 0, z(T), 1.0, z(T, dtype=i32)),
        "topk_merge": lambda: ops.launchTopKMerge(z(T, 3, 5, dtype=i32), z(T, 3, 5), z(T, 5, dtype=i32), z(T, 5)),
        "topk_merge_gathered": lambda: ops.launchTopKMergeGathered(
            z(3, ops.packed_record_bytes(T, 5, f32), dtype=torch.uint8), 3, T, 5, z(T, 5, dtype=i32), z(T, 5)),
        "sampling": lambda: ops.launchSampling(z(T, 5, dtype=i32), z(T, 5), z(T), z(T, dtype=i32), 1.0),
        "causal_mask": lambda: ops.launchBuildCausalMasks(z(B, S, S), z(B, dtype=i32), z(B, dtype=i32)),
        "padding_offset": lambda: ops.launchCalPaddingoffset(z(B, S, dtype=i32), z(B + 1, dtype=i32), z(B, dtype=i32)),
        "transpose_remove_padding": lambda: ops.launchTransposeOutRemovePadding(z(B, H, S, D), z(T, dtype=i32), z(T, H, D)),
        "repeat_kv": lambda: ops.launchRepeatKVCache(z(3, B, KV, 32, D), z(3, B, KV, 32, D), z(B, dtype=i32), 1,
                                                     z(B, H, 20, D), z(B, H, 20, D)),
        "decoder_mha": lambda: ops.launchDecoderMaskedMHA(z(B, H + 2 * KV, D), None, 0, z(1, B, KV, 32, D), z(1, B, KV, 32, D),
                                                          None, 7, z(B, H, D), D, 10000.0),
    }


@pytest.mark.parametrize("name", sorted(good_calls()))
def test_well_formed_cpu_call_passes_validation_and_is_refused_for_its_device(name):
    with pytest.raises(ValueError, match="CUDA tensors"):
        good_calls()[name]()


def bad_calls():
    B, H, KV, S, D, T = 2, 4, 2, 8, 16, 13
    i = lambda *s: z(*s, dtype=i32)
    l = lambda *s: z(*s, dtype=i64)
    h = lambda *s: z(*s, dtype=f16)
    return [
        # int64 length / offset / id tensors
        ("embedding ids int64", TypeError, lambda: ops.launchInputEmbedding(l(T), z(T, 64), z(100, 64))),
        ("qkv padding_offset int64", TypeError, lambda: ops.launchAddFusedQKVBiasTransposeAndRoPE(
            z(B, H, S, D), z(B, KV, S, D), z(B, KV, S, D), z(T, H + 2 * KV, D), None, l(T), i(B), i(B), D, 1e4)),
        ("qkv history_length int64", TypeError, lambda: ops.launchAddFusedQKVBiasTransposeAndRoPE(
            z(B, H, S, D), z(B, KV, S, D), z(B, KV, S, D), z(T, H + 2 * KV, D), None, i(T), l(B), i(B), D, 1e4)),
        ("concat cur_query_length int64", TypeError, lambda: ops.launchConcatKVCache(
            z(B, KV, S, D), z(B, KV, S, D), 0, l(B), i(B), z(1, B, KV, 32, D), z(1, B, KV, 32, D))),
        ("causal softmax q_lens int64", TypeError, lambda: ops.launchScaleCausalSoftmax(z(B, H, S, S), l(B), i(B), z(B, H, S, S), 1.0)),
        ("causal mask k_lens int64", TypeError, lambda: ops.launchBuildCausalMasks(z(B, S, S), i(B), l(B))),
        ("padding offsets int64", TypeError, lambda: ops.launchCalPaddingoffset(l(B, S), i(B + 1), i(B))),
        ("transpose padding_offset int64", TypeError, lambda: ops.launchTransposeOutRemovePadding(z(B, H, S, D), l(T), z(T, H, D))),
        ("repeat_kv context_length int64", TypeError, lambda: ops.launchRepeatKVCache(
            z(1, B, KV, 32, D), z(1, B, KV, 32, D), l(B), 0, z(B, H, 20, D), z(B, H, 20, D))),
        ("topk final ids int64", TypeError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T, 8, 5), z(T, 8, 5), l(T, 5), z(T, 5))),
        ("sampling ids int64", TypeError, lambda: ops.launchSampling(l(T, 5), z(T, 5), z(T), i(T), 1.0)),
        # mixed floating types in one call
        ("softmax fp16 score for fp32 qk", TypeError, lambda: ops.launchScaleMaskAndSoftmax(z(B, H, S, S), z(B, S, S), h(B, H, S, S), 1.0)),
        ("softmax fp16 mask for fp32 qk", TypeError, lambda: ops.launchScaleMaskAndSoftmax(z(B, H, S, S), h(B, S, S), z(B, H, S, S), 1.0)),
        ("rmsnorm fp16 gamma", TypeError, lambda: ops.launchRMSNorm(z(T, 64), None, h(64), 1e-6)),
        ("act fp16 out", TypeError, lambda: ops.launchAct(z(T, 2, 32), h(T, 32))),
        ("topk fp16 values for fp32 logits", TypeError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T, 8, 5), z(T, 8, 5), i(T, 5), h(T, 5))),
        ("mha fp16 cache for fp32 qkv", TypeError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), None, 0, h(1, B, KV, 32, D), h(1, B, KV, 32, D), None, 7, z(B, H, D), D, 1e4)),
        ("float64 input", TypeError, lambda: ops.launchAct(z(T, 2, 32, dtype=torch.float64), z(T, 32, dtype=torch.float64))),
        ("uniform fp16", TypeError, lambda: ops.launchSampling(i(T, 5), z(T, 5), h(T), i(T), 1.0)),
        # shapes of outputs, scratch and caches
        ("residual shape", ValueError, lambda: ops.launchFusedAddBiasResidualRMSNorm(z(T, 32), z(T, 64), None, z(64), 1e-6)),
        ("gamma length", ValueError, lambda: ops.launchRMSNorm(z(T, 64), None, z(32), 1e-6)),
        ("embedding table width", ValueError, lambda: ops.launchInputEmbedding(i(T), z(T, 64), z(100, 32))),
        ("embedding id count", ValueError, lambda: ops.launchInputEmbedding(i(T + 1), z(T, 64), z(100, 64))),
        ("k_buf shape", ValueError, lambda: ops.launchAddFusedQKVBiasTransposeAndRoPE(
            z(B, H, S, D), z(B, H, S, D), z(B, KV, S, D), z(T, H + 2 * KV, D), None, i(T), i(B), i(B), D, 1e4)),
        ("v_buf seq", ValueError, lambda: ops.launchAddFusedQKVBiasTransposeAndRoPE(
            z(B, H, S, D), z(B, KV, S, D), z(B, KV, S + 1, D), z(T, H + 2 * KV, D), None, i(T), i(B), i(B), D, 1e4)),
        ("padding_offset too short", ValueError, lambda: ops.launchAddFusedQKVBiasTransposeAndRoPE(
            z(B, H, S, D), z(B, KV, S, D), z(B, KV, S, D), z(T, H + 2 * KV, D), None, i(T - 1), i(B), i(B), D, 1e4)),
        ("odd rotary dim", ValueError, lambda: ops.launchRoPE(z(B, H + 2 * KV, D), 5, H, KV, 7, 1e4)),
        ("decode rope head counts", ValueError, lambda: ops.launchRoPE(z(B, H + 2 * KV, D), 5, H, KV + 1, D, 1e4)),
        ("act out shape", ValueError, lambda: ops.launchAct(z(T, 2, 32), z(T, 33))),
        ("concat v_src shape", ValueError, lambda: ops.launchConcatKVCache(
            z(B, KV, S, D), z(B, KV, S + 1, D), 0, i(B), i(B), z(1, B, KV, 32, D), z(1, B, KV, 32, D))),
        ("concat cache batch", ValueError, lambda: ops.launchConcatKVCache(
            z(B, KV, S, D), z(B, KV, S, D), 0, i(B), i(B), z(1, B + 1, KV, 32, D), z(1, B + 1, KV, 32, D))),
        ("concat cache head size", ValueError, lambda: ops.launchConcatKVCache(
            z(B, KV, S, D), z(B, KV, S, D), 0, i(B), i(B), z(1, B, KV, 32, 2 * D), z(1, B, KV, 32, 2 * D))),
        ("concat v_dst shape", ValueError, lambda: ops.launchConcatKVCache(
            z(B, KV, S, D), z(B, KV, S, D), 0, i(B), i(B), z(1, B, KV, 32, D), z(1, B, KV, 16, D))),
        ("concat layer", ValueError, lambda: ops.launchConcatKVCache(
            z(B, KV, S, D), z(B, KV, S, D), 3, i(B), i(B), z(3, B, KV, 32, D), z(3, B, KV, 32, D))),
        ("softmax score shape", ValueError, lambda: ops.launchScaleMaskAndSoftmax(z(B, H, S, S), z(B, S, S), z(B, H, S, S - 1), 1.0)),
        ("softmax mask shape", ValueError, lambda: ops.launchScaleMaskAndSoftmax(z(B, H, S, S), z(B, H, S, S), z(B, H, S, S), 1.0)),
        ("causal softmax lengths", ValueError, lambda: ops.launchScaleCausalSoftmax(z(B, H, S, S), i(B + 1), i(B), z(B, H, S, S), 1.0)),
        ("topk values shape", ValueError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T, 8, 5), z(T, 8, 5), i(T, 5), z(T, 6))),
        ("topk scratch size", ValueError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T, 8, 5), z(T, 4, 5), i(T, 5), z(T, 5))),
        ("topk scratch not whole slices", ValueError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T * 8 * 5 + 1), z(T * 8 * 5 + 1), i(T, 5), z(T, 5))),
        ("topk uniform without sampled ids", ValueError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T, 8, 5), z(T, 8, 5), i(T, 5), z(T, 5), 0, z(T))),
        ("topk sampled ids length", ValueError, lambda: ops.launchTopKforBeamSearch(z(T, 100), i(T, 8, 5), z(T, 8, 5), i(T, 5), z(T, 5), 0, z(T), 1.0, i(T - 1))),
        ("merge final shape", ValueError, lambda: ops.launchTopKMerge(i(T, 3, 5), z(T, 3, 5), i(T, 4), z(T, 4))),
        ("merge gathered record size", ValueError, lambda: ops.launchTopKMergeGathered(
            z(3, 17, dtype=torch.uint8), 3, T, 5, i(T, 5), z(T, 5))),
        ("sampling output length", ValueError, lambda: ops.launchSampling(i(T, 5), z(T, 5), z(T), i(T + 1), 1.0)),
        ("mask lengths", ValueError, lambda: ops.launchBuildCausalMasks(z(B, S, S), i(B), i(B - 1))),
        ("padding offset cum length", ValueError, lambda: ops.launchCalPaddingoffset(i(B, S), i(B), i(B))),
        ("transpose out shape", ValueError, lambda: ops.launchTransposeOutRemovePadding(z(B, H, S, D), i(T), z(T, H, D + 1))),
        ("transpose too many tokens", ValueError, lambda: ops.launchTransposeOutRemovePadding(z(B, H, S, D), i(B * S + 1), z(B * S + 1, H, D))),
        ("repeat_kv dst batch", ValueError, lambda: ops.launchRepeatKVCache(
            z(1, B, KV, 32, D), z(1, B, KV, 32, D), i(B), 0, z(B + 1, H, 20, D), z(B + 1, H, 20, D))),
        ("repeat_kv heads", ValueError, lambda: ops.launchRepeatKVCache(
            z(1, B, KV, 32, D), z(1, B, KV, 32, D), i(B), 0, z(B, 3, 20, D), z(B, 3, 20, D))),
        ("repeat_kv layer", ValueError, lambda: ops.launchRepeatKVCache(
            z(1, B, KV, 32, D), z(1, B, KV, 32, D), i(B), 1, z(B, H, 20, D), z(B, H, 20, D))),
        ("mha cache batch", ValueError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), None, 0, z(1, B + 1, KV, 32, D), z(1, B + 1, KV, 32, D), None, 7, z(B, H, D), D, 1e4)),
        ("mha cache head size", ValueError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), None, 0, z(1, B, KV, 32, 2 * D), z(1, B, KV, 32, 2 * D), None, 7, z(B, H, D), D, 1e4)),
        ("mha output shape", ValueError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), None, 0, z(1, B, KV, 32, D), z(1, B, KV, 32, D), None, 7, z(B, H + 1, D), D, 1e4)),
        ("mha step beyond the cache", ValueError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), None, 0, z(1, B, KV, 32, D), z(1, B, KV, 32, D), None, 33, z(B, H, D), D, 1e4)),
        ("mha layer", ValueError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), None, 1, z(1, B, KV, 32, D), z(1, B, KV, 32, D), None, 7, z(B, H, D), D, 1e4)),
        ("mha bias length", ValueError, lambda: ops.launchDecoderMaskedMHA(
            z(B, H + 2 * KV, D), z(5), 0, z(1, B, KV, 32, D), z(1, B, KV, 32, D), None, 7, z(B, H, D), D, 1e4)),
    ]


@pytest.mark.parametrize("what,exc,call", bad_calls(), ids=[c[0] for c in bad_calls()])
def test_malformed_call_raises_before_anything_is_launched(what, exc, call):
    with pytest.raises(exc) as info:
        call()
    assert "CUDA tensors" not in str(info.value)  # refused for what is wrong with it, not for being on the CPU
