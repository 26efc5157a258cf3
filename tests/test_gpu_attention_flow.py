"""The kernels either side of attention, composed the way the reference's context attention uses
them: padding offsets -> QKV bias + RoPE + un-pad + transpose -> KV-cache concat -> repeat-KV ->
[QK^T] -> causal mask + softmax -> [PV] -> transpose + remove padding.  The two GEMMs are
torch.matmul; everything else is this library.  The result is compared with a plain float64
attention written per sequence from the packed inputs, so the test fails if any two kernels
disagree about a layout, an offset or a position.  Marked gpu.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda):
    from inferspore_b200 import ops as _ops

    return _ops


def _rope_rotate_half(x, pos, base):
    """x [..., d] float64, rotate-half pairs (j, j + d/2), angle pos / base^(2j/d)."""
    d = x.shape[-1]
    j = np.arange(d // 2)
    theta = pos / base ** (2.0 * j / d)
    c, s = np.cos(theta), np.sin(theta)
    lo, hi = x[..., : d // 2], x[..., d // 2:]
    return np.concatenate([c * lo - s * hi, c * hi + s * lo], -1)


@pytest.mark.parametrize("lens,heads,kv_heads,d", [([5, 9, 1, 7], 4, 4, 16), ([12, 3], 8, 2, 32), ([6], 2, 1, 8)])
def test_context_attention_flow(ops, rng, lens, heads, kv_heads, d):
    dev = "cuda:0"
    batch, seq = len(lens), max(lens)
    tokens, base = sum(lens), 10000.0
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    d_lens = i32(lens)
    # 1. padding offsets
    pad = torch.zeros((batch, seq), dtype=torch.int32, device=dev)
    cum = torch.zeros(batch + 1, dtype=torch.int32, device=dev)
    ops.launchCalPaddingoffset(pad, cum, d_lens)
    assert cum.cpu().tolist() == np.concatenate([[0], np.cumsum(lens)]).tolist()
    pad_flat = pad.view(-1)[:tokens].contiguous()
    # 2. packed QKV -> q, k, v [b, h, s, d] with bias and RoPE (positions 0.., no history)
    qkv = rng.standard_normal((tokens, heads + 2 * kv_heads, d), dtype=np.float32)
    bias = (rng.standard_normal((heads + 2 * kv_heads) * d) * 0.1).astype(np.float32)
    q = torch.zeros((batch, heads, seq, d), device=dev)
    k = torch.zeros((batch, kv_heads, seq, d), device=dev)
    v = torch.zeros_like(k)
    hist = torch.zeros(batch, dtype=torch.int32, device=dev)
    ops.launchAddFusedQKVBiasTransposeAndRoPE(q, k, v, torch.from_numpy(qkv).to(dev), torch.from_numpy(bias).to(dev),
                                              pad_flat, hist, d_lens, d, base)
    # 3. into the cache of layer 1 of 2, then broadcast to the q heads
    max_seq = seq + 3
    kc = torch.zeros((2, batch, kv_heads, max_seq, d), device=dev)
    vc = torch.zeros_like(kc)
    ops.launchConcatKVCache(k, v, 1, d_lens, hist, kc, vc)
    k_rep = torch.zeros((batch, heads, seq, d), device=dev)
    v_rep = torch.zeros_like(k_rep)
    ops.launchRepeatKVCache(kc, vc, d_lens, 1, k_rep, v_rep)
    # 4. scores, mask, softmax (both routes), context
    qk = torch.matmul(q, k_rep.transpose(-1, -2)).contiguous()
    mask = torch.empty((batch, seq, seq), device=dev)
    ops.launchBuildCausalMasks(mask, d_lens, d_lens)
    score = torch.empty_like(qk)
    scale = 1.0 / float(np.sqrt(d))
    ops.launchScaleMaskAndSoftmax(qk, mask, score, scale)
    fused = torch.empty_like(qk)
    ops.launchScaleCausalSoftmax(qk, d_lens, d_lens, fused, scale)
    assert torch.allclose(score, fused, rtol=3e-6, atol=0.0)
    ctx = torch.matmul(score, v_rep).contiguous()  # [b, h, s, d]
    # 5. back to packed tokens
    out = torch.full((tokens, heads, d), 7.0, device=dev)
    ops.launchTransposeOutRemovePadding(ctx, pad_flat, out)
    got = out.cpu().numpy().astype(np.float64)

    # the same attention, sequence by sequence, in float64 from the packed inputs
    x = qkv.astype(np.float64) + bias.reshape(heads + 2 * kv_heads, d).astype(np.float64)
    group = heads // kv_heads
    start = 0
    for n in lens:
        pos = np.arange(n)[:, None, None]
        tok = x[start:start + n]
        qq = _rope_rotate_half(tok[:, :heads], pos, base)                       # [n, heads, d]
        kk = _rope_rotate_half(tok[:, heads:heads + kv_heads], pos, base)       # [n, kv, d]
        vv = tok[:, heads + kv_heads:]
        for h in range(heads):
            logits = qq[:, h] @ kk[:, h // group].T * scale                     # [n, n]
            logits = np.where(np.tril(np.ones((n, n), bool)), logits, -np.inf)
            p = np.exp(logits - logits.max(-1, keepdims=True))
            p /= p.sum(-1, keepdims=True)
            want = p @ vv[:, h // group]
            assert np.allclose(got[start:start + n, h], want, rtol=2e-4, atol=2e-5), (n, h)
        start += n


def test_decode_steps_build_the_cache_they_read(ops, rng):
    """Six decode steps from an empty cache: step s appends at position s-1 and attends to
    positions < s, so every step's output depends on every earlier append being where the later
    steps look for it.  Adjacent-pair RoPE at position `step`, as the reference's decode kernel."""
    dev = "cuda:0"
    batch, heads, kv_heads, d, max_seq, base = 2, 4, 2, 16, 8, 10000.0
    group = heads // kv_heads
    kc = torch.zeros((1, batch, kv_heads, max_seq, d), device=dev)
    vc = torch.zeros_like(kc)
    out = torch.empty((batch, heads, d), device=dev)
    hist_k = np.zeros((batch, kv_heads, 0, d))
    hist_v = np.zeros((batch, kv_heads, 0, d))
    i = np.arange(d // 2)
    for step in range(1, 7):
        qkv = rng.standard_normal((batch, heads + 2 * kv_heads, d), dtype=np.float32)
        ops.launchDecoderMaskedMHA(torch.from_numpy(qkv).to(dev), None, 0, kc, vc, None, step, out, d, base)
        x = qkv.astype(np.float64)
        theta = step / base ** (2.0 * i / d)
        c, s = np.cos(theta), np.sin(theta)
        rot = x.copy()
        rot[:, :heads + kv_heads, 0::2] = c * x[:, :heads + kv_heads, 0::2] - s * x[:, :heads + kv_heads, 1::2]
        rot[:, :heads + kv_heads, 1::2] = c * x[:, :heads + kv_heads, 1::2] + s * x[:, :heads + kv_heads, 0::2]
        hist_k = np.concatenate([hist_k, rot[:, heads:heads + kv_heads, None]], 2)
        hist_v = np.concatenate([hist_v, rot[:, heads + kv_heads:, None]], 2)
        got = out.cpu().numpy().astype(np.float64)
        for b in range(batch):
            for h in range(heads):
                logits = hist_k[b, h // group] @ rot[b, h] / np.sqrt(d)
                p = np.exp(logits - logits.max())
                want = (p / (p.sum() + 1e-6)) @ hist_v[b, h // group]
                assert np.allclose(got[b, h], want, rtol=1e-4, atol=1e-5), (step, b, h)
    assert np.allclose(kc[0, :, :, :6].cpu().numpy(), hist_k, rtol=1e-5, atol=1e-6)
    assert not kc[0, :, :, 6:].any()
