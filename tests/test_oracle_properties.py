"""The oracle against independent numpy restatements on random shapes (CPU only).  The golden
fixtures and the reference's CPU functions pin the oracle on the cases the reference has; these
widen the pin to ragged shapes, ties and the ops the reference has no CPU code for."""
import numpy as np
import pytest


@pytest.mark.parametrize("seed", range(6))
def test_topk_equals_a_stable_sort(orc, seed):
    rng = np.random.default_rng(seed)
    rows, vocab, K = int(rng.integers(1, 9)), int(rng.integers(5, 3000)), int(rng.integers(1, 60))
    K = min(K, vocab)
    probs = rng.standard_normal((rows, vocab)).astype(np.float32)
    probs[:, rng.integers(0, vocab, vocab // 3)] = probs[:, :1]  # many ties
    ids, vals = orc.topk(probs, K)
    for r in range(rows):
        order = np.lexsort((np.arange(vocab), -probs[r].astype(np.float64)))[:K]  # value desc, index asc
        assert np.array_equal(ids[r], order.astype(np.int32))
        assert np.array_equal(vals[r], probs[r, order])


@pytest.mark.parametrize("seed", range(6))
def test_softmax_equals_numpy(orc, seed):
    rng = np.random.default_rng(100 + seed)
    b, h, q = (int(rng.integers(1, 4)) for _ in range(3))
    k = int(rng.integers(1, 300))
    qk = (rng.standard_normal((b, h, q, k)) * 4).astype(np.float32)
    mask = (rng.random((b, q, k)) < 0.8).astype(np.float32)
    got, _ = orc.scale_mask_softmax(qk, mask, np.float32(0.3))
    z = 0.3 * qk.astype(np.float64) + (1.0 - mask[:, None].astype(np.float64)) * -10000.0
    m = np.maximum(z.max(-1, keepdims=True), np.finfo(np.float32).tiny)
    e = np.exp(z - m)
    want = e / (e.sum(-1, keepdims=True) + 1e-6)
    assert np.allclose(got, want, rtol=2e-6, atol=1e-30)


@pytest.mark.parametrize("seed", range(6))
def test_layout_ops_equal_numpy_indexing(orc, seed):
    rng = np.random.default_rng(200 + seed)
    batch, seq, heads, kv, d = int(rng.integers(1, 6)), int(rng.integers(1, 12)), 6, 3, int(rng.integers(1, 5)) * 2
    lens = rng.integers(0, seq + 1, batch)
    # padding offsets
    po, cum = orc.cal_padding_offset(lens, seq)
    assert cum.tolist() == np.concatenate([[0], np.cumsum(lens)]).tolist()
    want_po = np.concatenate([np.full(n, b * seq - cum[b]) for b, n in enumerate(lens)]) if lens.sum() else np.zeros(0)
    assert po.reshape(-1)[:lens.sum()].tolist() == want_po.astype(int).tolist()
    # transpose + remove padding is fancy indexing with (b, s) = divmod(t + offset, seq)
    tokens = int(cum[-1])
    offs = po.reshape(-1)[:tokens]
    x = rng.standard_normal((batch, heads, seq, d)).astype(np.float32)
    dst = np.arange(tokens) + offs
    want = x[dst // seq, :, dst % seq] if tokens else np.zeros((0, heads, d), np.float32)
    assert np.array_equal(orc.transpose_remove_padding(x, offs, tokens), want)
    # causal mask predicate, element by element
    ql = rng.integers(0, seq + 1, batch)
    kl = np.minimum(ql + rng.integers(0, 5, batch), seq + 3)
    got = orc.build_causal_mask(ql, kl, seq, seq + 3)
    qq, kk = np.arange(seq)[None, :, None], np.arange(seq + 3)[None, None, :]
    qlen, klen = ql[:, None, None], kl[:, None, None]
    want = ((qq < qlen) & (kk < klen) & (kk <= qq + klen - qlen) & (kk >= klen - qlen)).astype(np.float32)
    assert np.array_equal(got, want)
    # repeat-KV is np.repeat along the head axis, cut at the context length
    src = rng.standard_normal((2, batch, kv, seq + 2, d)).astype(np.float32)
    ctx = rng.integers(0, seq + 1, batch)
    out = orc.repeat_kv(np.zeros((batch, heads, seq, d), np.float32), src, ctx, 1, heads)
    rep = np.repeat(src[1], heads // kv, axis=1)[:, :, :seq]
    for b in range(batch):
        assert np.array_equal(out[b, :, :ctx[b]], rep[b, :, :ctx[b]])
        assert not out[b, :, ctx[b]:].any()


@pytest.mark.parametrize("seed", range(4))
def test_decoder_attention_equals_numpy(orc, seed):
    rng = np.random.default_rng(300 + seed)
    batch, kv, group, d, max_seq = int(rng.integers(1, 4)), 2, int(rng.integers(1, 4)), 8, 20
    heads, step, rot = kv * group, int(rng.integers(1, max_seq + 1)), 8
    qkv = rng.standard_normal((batch, heads + 2 * kv, d)).astype(np.float32)
    bias = (rng.standard_normal((heads + 2 * kv) * d) * 0.1).astype(np.float32)
    kc = rng.standard_normal((1, batch, kv, max_seq, d)).astype(np.float32)
    vc = rng.standard_normal((1, batch, kv, max_seq, d)).astype(np.float32)
    out, nk, nv, _ = orc.decoder_masked_mha(qkv, bias, kc, vc, 0, step, rot, 10000.0)
    x = (qkv + bias.reshape(heads + 2 * kv, d)).astype(np.float64)
    theta = step / 10000.0 ** (np.arange(0, rot, 2) / rot)
    c, s = np.cos(theta), np.sin(theta)
    rotd = x.copy()
    rotd[:, :heads + kv, 0:rot:2] = c * x[:, :heads + kv, 0:rot:2] - s * x[:, :heads + kv, 1:rot:2]
    rotd[:, :heads + kv, 1:rot:2] = c * x[:, :heads + kv, 1:rot:2] + s * x[:, :heads + kv, 0:rot:2]
    K, V = kc[0].astype(np.float64).copy(), vc[0].astype(np.float64).copy()
    K[:, :, step - 1], V[:, :, step - 1] = rotd[:, heads:heads + kv], rotd[:, heads + kv:]
    assert np.allclose(nk[0], K, rtol=1e-5, atol=1e-6) and np.allclose(nv[0], V, rtol=1e-6, atol=1e-7)
    for b in range(batch):
        for h in range(heads):
            g = h // group
            logits = K[b, g, :step] @ rotd[b, h] / np.sqrt(d)
            p = np.exp(logits - logits.max())
            want = (p / (p.sum() + 1e-6)) @ V[b, g, :step]
            assert np.allclose(out[b, h], want, rtol=2e-5, atol=2e-6)
