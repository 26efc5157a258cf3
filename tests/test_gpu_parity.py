"""CUDA kernels vs the oracle, through the C ABI.  Marked gpu.

Bit-exact where the op is a copy or an index selection (embedding, KV concat,
top-K ids and values); 1e-5 relative for fp32 outputs; 2e-3 absolute against
the oracle's fp32-accumulated value for fp16 outputs (tests/_util.py).
"""
import numpy as np
import pytest
import torch

from _util import assert_close_f16, assert_close_f32, dev, host, randn16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda):
    from inferspore_b200 import ops as _ops

    return _ops


@pytest.fixture(autouse=True)
def _clean_status(cuda):
    from inferspore_b200 import capi

    capi.device_status(clear=True)
    yield
    torch.cuda.synchronize()


# ---- residual add + RMSNorm ---------------------------------------------------------------------

NORM_SHAPES = [(64, 4096), (2, 32), (5, 8), (3, 1000), (300, 4096), (7, 5120), (4, 8192), (3, 11008), (2, 16384),
               (3, 100), (2, 4100), (1, 1), (1200, 256), (2, 20000)]


@pytest.mark.parametrize("tokens,hidden", NORM_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_add_residual_rmsnorm_f32(ops, orc, rng, tokens, hidden, with_bias):
    x = rng.standard_normal((tokens, hidden), dtype=np.float32)
    r = rng.standard_normal((tokens, hidden), dtype=np.float32)
    g = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    b = (rng.standard_normal(hidden) * 0.1).astype(np.float32) if with_bias else None
    dx, dr, dg = dev(x), dev(r), dev(g)
    ops.launchFusedAddBiasResidualRMSNorm(dr, dx, None if b is None else dev(b), dg, 1e-6)
    want_x, want_r, _ = orc.add_residual_rmsnorm(x, r, b, g, 1e-6)
    assert np.array_equal(host(dr), want_r)  # one IEEE add: exact
    assert_close_f32(host(dx), want_x, what="rmsnorm f32")


@pytest.mark.parametrize("tokens,hidden", NORM_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_add_residual_rmsnorm_f16(ops, orc, rng, tokens, hidden, with_bias):
    x, r = randn16(rng, (tokens, hidden)), randn16(rng, (tokens, hidden))
    g = rng.uniform(0.5, 1.5, hidden).astype(np.float16)
    b = randn16(rng, hidden, 0.1) if with_bias else None
    dx, dr = dev(x), dev(r)
    ops.launchFusedAddBiasResidualRMSNorm(dr, dx, None if b is None else dev(b), dev(g), 1e-6)
    want_x, want_r, want32 = orc.add_residual_rmsnorm(x, r, b, g, 1e-6)
    assert np.array_equal(host(dr).view(np.uint16), want_r.view(np.uint16))
    _, _, same = assert_close_f16(host(dx), want32, want_x, "rmsnorm f16")
    assert same > 0.99


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("tokens,hidden", [(64, 4096), (9, 40), (3, 12288)])
def test_plain_rmsnorm_and_null_residual(ops, orc, rng, dtype, tokens, hidden):
    x = rng.standard_normal((tokens, hidden), dtype=np.float32).astype(dtype)
    g = rng.uniform(0.5, 1.5, hidden).astype(dtype)
    want, want_copy, want32 = orc.rmsnorm(x, g, 1e-6, want_copy=True)
    # (1) launchRMSNorm with a residual copy
    dx, dc = dev(x), torch.empty_like(dev(x))
    ops.launchRMSNorm(dx, dc, dev(g), 1e-6)
    assert np.array_equal(host(dc).view(np.uint8), x.view(np.uint8))
    # (2) launchRMSNorm without, (3) the reference's route: fused launcher with a NULL residual
    dx2, dx3 = dev(x), dev(x)
    ops.launchRMSNorm(dx2, None, dev(g), 1e-6)
    ops.launchFusedAddBiasResidualRMSNorm(None, dx3, None, dev(g), 1e-6)
    for d in (dx, dx2, dx3):
        if dtype == np.float32:
            assert_close_f32(host(d), want, what="plain rmsnorm")
        else:
            assert_close_f16(host(d), want32, want, "plain rmsnorm f16")
    # the two routes to the plain norm are the same kernel
    assert np.array_equal(host(dx2).view(np.uint8), host(dx3).view(np.uint8))


def test_rmsnorm_unaligned_views_take_the_scalar_path(ops, orc, rng):
    big = rng.standard_normal(3 * 64 + 1, dtype=np.float32)
    d = dev(big)
    x = d[1:].view(3, 64)  # 4-byte aligned only
    g = rng.uniform(0.5, 1.5, 64).astype(np.float32)
    ops.launchFusedAddBiasResidualRMSNorm(None, x, None, dev(g), 1e-6)
    want, _, _ = orc.add_residual_rmsnorm(big[1:].reshape(3, 64), None, None, g, 1e-6)
    assert_close_f32(host(x), want, what="unaligned rmsnorm")
    assert host(d)[0] == big[0]


def test_rmsnorm_empty(ops, cuda):
    x = torch.empty((0, 128), device=cuda)
    ops.launchFusedAddBiasResidualRMSNorm(torch.empty_like(x), x, None, torch.ones(128, device=cuda), 1e-6)


def test_prepared_launch_is_the_same_call_without_the_checks(ops, rng):
    x = rng.standard_normal((33, 1024), dtype=np.float32)
    g = rng.uniform(0.5, 1.5, 1024).astype(np.float32)
    a, b, dg = dev(x), dev(x), dev(g)
    ops.launchRMSNorm(a, None, dg, 1e-6)
    launch = ops.prepare(ops.launchRMSNorm, b, None, dg, 1e-6)
    assert np.array_equal(host(b), x)  # preparing validates and binds, it does not launch
    launch()
    assert np.array_equal(host(a), host(b))
    with pytest.raises(ValueError):  # the checks run at prepare time
        ops.prepare(ops.launchRMSNorm, b, None, dev(g[:100]), 1e-6)


# ---- embedding -----------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("tokens,hidden,vocab", [(4096, 4096, 32000), (64, 4096, 32000), (33, 100, 50), (1, 8, 3),
                                                 (257, 1000, 777), (19, 7, 11)])
def test_input_embedding_bit_exact(ops, orc, rng, dtype, tokens, hidden, vocab):
    table = (rng.standard_normal((vocab, hidden), dtype=np.float32) * 0.02).astype(dtype)
    ids = rng.integers(0, vocab, tokens).astype(np.int32)
    ids[0], ids[-1] = vocab - 1, 0
    out = torch.empty((tokens, hidden), dtype=dev(table[:1]).dtype, device="cuda:0")
    ops.launchInputEmbedding(dev(ids), out, dev(table))
    assert np.array_equal(host(out).view(np.uint8), orc.input_embedding(ids, table).view(np.uint8))


def test_input_embedding_bad_id_is_flagged_not_faulted(ops, orc, rng):
    from inferspore_b200 import capi

    table = rng.standard_normal((10, 64), dtype=np.float32)
    ids = np.array([1, 10, -1, 9], np.int32)
    out = torch.full((4, 64), 5.0, device="cuda:0")
    ops.launchInputEmbedding(dev(ids), out, dev(table))
    torch.cuda.synchronize()
    assert capi.device_status(clear=True) & capi.DEV_BAD_TOKEN_ID
    assert np.array_equal(host(out), orc.input_embedding(ids, table))
    assert capi.device_status() == 0


# ---- QKV bias + RoPE + transpose --------------------------------------------------------------------------

def _rope_inputs(rng, dtype, batch, seq, heads, kv_heads, d, lens, hist):
    lens = np.asarray(lens)
    token_num = int(lens.sum())
    padding_offset = np.concatenate([np.full(n, b * seq - lens[:b].sum(), np.int32) for b, n in enumerate(lens)])
    QKV = rng.standard_normal((token_num, heads + 2 * kv_heads, d), dtype=np.float32).astype(dtype)
    bias = (rng.standard_normal((heads + 2 * kv_heads) * d) * 0.02).astype(dtype)
    return QKV, bias, padding_offset.astype(np.int32), np.asarray(hist, np.int32), lens.astype(np.int32)


def _pair_magnitude(QKV, bias, padding_offset, batch, seq, heads, kv_heads):
    """|x0| + |x1| of every rotation pair, scattered like the outputs: the scale the fp32
    rounding error of c*x0 - s*x1 is proportional to when the two terms cancel."""
    x = QKV.astype(np.float32)
    if bias is not None:
        x = x + bias.astype(np.float32).reshape(1, -1, x.shape[2])
    half = x.shape[2] // 2
    mag = np.abs(x[..., :half]) + np.abs(x[..., half:])
    mag = np.concatenate([mag, mag], -1)
    dst = np.arange(x.shape[0]) + padding_offset
    out_q = np.zeros((batch, heads, seq, x.shape[2]), np.float32)
    out_k = np.zeros((batch, kv_heads, seq, x.shape[2]), np.float32)
    out_q[dst // seq, :, dst % seq] = mag[:, :heads]
    out_k[dst // seq, :, dst % seq] = mag[:, heads:heads + kv_heads]
    return out_q, out_k


ROPE_CASES = [
    # batch, seq, heads, kv_heads, d, rot, lens, hist
    (1, 32, 32, 32, 128, 128, [32], [0]),
    (3, 5, 2, 2, 8, 8, [3, 3, 3], [0, 0, 0]),
    (2, 16, 8, 2, 128, 128, [16, 9], [7, 4000]),      # GQA, history, ragged
    (2, 7, 4, 4, 64, 32, [7, 1], [0, 5]),             # partial rotary dim
    (4, 33, 5, 1, 128, 128, [33, 1, 17, 2], [1, 2, 3, 4095]),
    (2, 6, 3, 3, 20, 20, [6, 5], [0, 1]),             # head size not a multiple of the vector width
]


@pytest.mark.parametrize("case", ROPE_CASES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_qkv_rope_transpose_f32(ops, orc, rng, case, with_bias):
    batch, seq, heads, kv_heads, d, rot, lens, hist = case
    QKV, bias, po, hl, il = _rope_inputs(rng, np.float32, batch, seq, heads, kv_heads, d, lens, hist)
    bias = bias if with_bias else None
    sentinel = 777.0
    q = torch.full((batch, heads, seq, d), sentinel, device="cuda:0")
    k = torch.full((batch, kv_heads, seq, d), sentinel, device="cuda:0")
    v = torch.full((batch, kv_heads, seq, d), sentinel, device="cuda:0")
    ops.launchAddFusedQKVBiasTransposeAndRoPE(q, k, v, dev(QKV), None if bias is None else dev(bias), dev(po), dev(hl),
                                              dev(il), rot, 10000.0)
    wq, wk, wv, _, _ = orc.qkv_bias_rope_transpose(QKV, bias, po, hl, batch, seq, heads, kv_heads, rot, 10000.0,
                                                   fill=sentinel)
    mq, mk = _pair_magnitude(QKV, bias, po, batch, seq, heads, kv_heads)
    # c*x0 - s*x1 can cancel: the error is relative to |x0| + |x1| (an fma on one side and two
    # roundings on the other already differ by an ulp of the larger term), hence the floor.
    assert_close_f32(host(q), wq, floor=0.1 * mq, what="q")
    assert_close_f32(host(k), wk, floor=0.1 * mk, what="k")
    assert np.array_equal(host(v), wv)  # copy, or one IEEE add with the bias


@pytest.mark.parametrize("case", ROPE_CASES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_qkv_rope_transpose_f16(ops, orc, rng, case, with_bias):
    batch, seq, heads, kv_heads, d, rot, lens, hist = case
    QKV, bias, po, hl, il = _rope_inputs(rng, np.float16, batch, seq, heads, kv_heads, d, lens, hist)
    bias = bias if with_bias else None
    mk16 = lambda *s: torch.full(s, 777.0, dtype=torch.float16, device="cuda:0")
    q, k, v = mk16(batch, heads, seq, d), mk16(batch, kv_heads, seq, d), mk16(batch, kv_heads, seq, d)
    ops.launchAddFusedQKVBiasTransposeAndRoPE(q, k, v, dev(QKV), None if bias is None else dev(bias), dev(po), dev(hl),
                                              dev(il), rot, 10000.0)
    wq, wk, wv, q32, k32 = orc.qkv_bias_rope_transpose(QKV, bias, po, hl, batch, seq, heads, kv_heads, rot, 10000.0,
                                                       fill=777.0)
    assert_close_f16(host(q), q32, wq, "q f16")
    assert_close_f16(host(k), k32, wk, "k f16")
    assert np.array_equal(host(v).view(np.uint16), wv.view(np.uint16))


def test_qkv_rope_norm_preserved_and_llama_shape(ops, orc, rng):
    """Llama-2-7B prefill shape (one sequence of 512): rotation preserves every pair's norm."""
    batch, seq, H, d = 1, 512, 32, 128
    QKV, _, po, hl, il = _rope_inputs(rng, np.float32, batch, seq, H, H, d, [seq], [0])
    q = torch.empty((batch, H, seq, d), device="cuda:0")
    k, v = torch.empty_like(q), torch.empty_like(q)
    ops.launchAddFusedQKVBiasTransposeAndRoPE(q, k, v, dev(QKV), None, dev(po), dev(hl), dev(il), 128, 10000.0)
    qh = host(q).astype(np.float64)
    got = qh[..., :64] ** 2 + qh[..., 64:] ** 2
    x = QKV[:, :H].astype(np.float64).reshape(seq, H, d).transpose(1, 0, 2)[None]
    want = x[..., :64] ** 2 + x[..., 64:] ** 2
    assert np.allclose(got, want, rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("batch,heads,kv_heads,d,rot,step", [(1, 32, 32, 128, 128, 17), (5, 8, 2, 64, 32, 4096),
                                                             (2, 3, 3, 10, 10, 1)])
def test_rope_decode(ops, orc, rng, dtype, batch, heads, kv_heads, d, rot, step):
    qkv = rng.standard_normal((batch, heads + 2 * kv_heads, d), dtype=np.float32).astype(dtype)
    dq = dev(qkv)
    ops.launchRoPE(dq, step, heads, kv_heads, rot, 10000.0)
    want, unr = orc.rope_decode(qkv, heads, kv_heads, step, rot, 10000.0)
    if dtype == np.float32:
        half = d // 2
        x = qkv.astype(np.float32)
        mag = np.abs(x[..., :half]) + np.abs(x[..., half:])
        assert_close_f32(host(dq), want, floor=0.1 * np.concatenate([mag, mag], -1), what="decode rope")
    else:
        assert_close_f16(host(dq), unr, want, "decode rope f16")
    # v heads untouched
    assert np.array_equal(host(dq)[:, heads + kv_heads:].view(np.uint8), qkv[:, heads + kv_heads:].view(np.uint8))


# ---- SiLU * up ---------------------------------------------------------------------------------------------------

ACT_SHAPES = [(16, 11008), (1, 8), (3, 7), (5, 1001), (64, 4096), (1, 27648), (130, 344)]


@pytest.mark.parametrize("rows,inter", ACT_SHAPES)
def test_silu_mul_f32(ops, orc, rng, rows, inter):
    inp = (rng.standard_normal((rows, 2, inter), dtype=np.float32) * 3)
    inp.flat[:6] = [0.0, -0.0, 30.0, -30.0, 80.0, -80.0][: min(6, inp.size)]
    out = torch.empty((rows, inter), device="cuda:0")
    ops.launchAct(dev(inp), out)
    want, _ = orc.silu_mul(inp)
    assert_close_f32(host(out), want, floor=1e-30, what="silu*up f32")


@pytest.mark.parametrize("rows,inter", ACT_SHAPES)
def test_silu_mul_f16(ops, orc, rng, rows, inter):
    inp = randn16(rng, (rows, 2, inter), 2.0)
    out = torch.empty((rows, inter), dtype=torch.float16, device="cuda:0")
    ops.launchAct(dev(inp), out)
    want, want32 = orc.silu_mul(inp)
    _, _, same = assert_close_f16(host(out), want32, want, "silu*up f16")
    assert same > 0.99


# ---- KV concat ------------------------------------------------------------------------------------------------------

CONCAT_CASES = [
    # layers, batch, heads, max_q, max_seq, d, layer
    (1, 1, 2, 16, 32, 8, 0),
    (3, 4, 2, 5, 40, 128, 2),
    (2, 64, 32, 1, 64, 128, 1),       # decode shape (short cache)
    (2, 3, 4, 7, 19, 20, 1),          # head size not a multiple of the vector width (fp32 ok, fp16 scalar path)
    (1, 2, 1, 9, 9, 3, 0),
]


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("case", CONCAT_CASES)
def test_concat_kv_bit_exact(ops, orc, rng, dtype, case):
    layers, batch, heads, max_q, max_seq, d, layer = case
    k_src = rng.standard_normal((batch, heads, max_q, d), dtype=np.float32).astype(dtype)
    v_src = rng.standard_normal((batch, heads, max_q, d), dtype=np.float32).astype(dtype)
    cur = rng.integers(0, max_q + 1, batch).astype(np.int32)
    cur[0] = max_q
    hist = np.array([rng.integers(0, max_seq - c + 1) for c in cur], np.int32)
    k_dst = rng.standard_normal((layers, batch, heads, max_seq, d), dtype=np.float32).astype(dtype)
    v_dst = rng.standard_normal((layers, batch, heads, max_seq, d), dtype=np.float32).astype(dtype)
    dk, dv = dev(k_dst), dev(v_dst)
    ops.launchConcatKVCache(dev(k_src), dev(v_src), layer, dev(cur), dev(hist), dk, dv)
    assert np.array_equal(host(dk).view(np.uint8), orc.concat_kv(k_dst, k_src, cur, hist, layer).view(np.uint8))
    assert np.array_equal(host(dv).view(np.uint8), orc.concat_kv(v_dst, v_src, cur, hist, layer).view(np.uint8))


def test_concat_kv_reference_fixture_4d_cache(ops, rng):
    # tests/unittests/test_concat_kv.cu: src = 1, history 1, cur 16, 4-D single-layer cache
    k_src = torch.ones((1, 2, 16, 8), device="cuda:0")
    kd = torch.full((1, 2, 32, 8), -7.0, device="cuda:0")
    vd = torch.full((1, 2, 32, 8), -7.0, device="cuda:0")
    ops.launchConcatKVCache(k_src, k_src, 0, dev(np.array([16], np.int32)), dev(np.array([1], np.int32)), kd, vd)
    for t in (host(kd), host(vd)):
        assert np.all(t[0, :, 1:17] == 1.0) and np.all(t[0, :, 0] == -7.0) and np.all(t[0, :, 17:] == -7.0)


def test_concat_kv_overrun_is_flagged_and_clamped(ops, orc, rng):
    from inferspore_b200 import capi

    k_src = rng.standard_normal((2, 1, 4, 8), dtype=np.float32)
    k_dst = np.zeros((1, 2, 1, 6, 8), np.float32)
    cur, hist = np.array([4, 4], np.int32), np.array([4, 0], np.int32)  # batch 0 would write rows 4..7 of 6
    dk, dv = dev(k_dst), dev(k_dst)
    ops.launchConcatKVCache(dev(k_src), dev(k_src), 0, dev(cur), dev(hist), dk, dv)
    torch.cuda.synchronize()
    assert capi.device_status(clear=True) & capi.DEV_KV_OVERRUN
    assert np.array_equal(host(dk), orc.concat_kv(k_dst, k_src, cur, hist, 0))


def test_qkv_rope_beyond_the_three_way_split(ops, orc, rng):
    """Launches of up to 16384 tokens run three CTAs per token (its q, its k and its v heads); longer
    ones one CTA per token.  17000 tokens of small grouped heads (8 q, 2 kv, size 64) with a bias and
    ragged sequences take the latter, against the oracle."""
    batch, seq, heads, kv_heads, d = 40, 512, 8, 2, 64
    lens = rng.integers(300, seq + 1, batch)
    lens[: 17000 // seq + 1] = seq
    while lens.sum() < 17000:
        lens[rng.integers(0, batch)] = seq
    tokens = int(lens.sum())
    assert tokens > 16384
    pad = np.concatenate([np.full(n, i * seq - lens[:i].sum(), np.int32) for i, n in enumerate(lens)])
    hist = rng.integers(0, 100, batch).astype(np.int32)
    qkv = randn16(rng, (tokens, heads + 2 * kv_heads, d))
    bias = randn16(rng, ((heads + 2 * kv_heads) * d,), 0.1)
    q = torch.zeros((batch, heads, seq, d), dtype=torch.float16, device="cuda:0")
    k = torch.zeros((batch, kv_heads, seq, d), dtype=torch.float16, device="cuda:0")
    v = torch.zeros_like(k)
    ops.launchAddFusedQKVBiasTransposeAndRoPE(q, k, v, dev(qkv), dev(bias), dev(pad), dev(hist), _i32(lens), d, 10000.0)
    wq, wk, wv, q32, k32 = orc.qkv_bias_rope_transpose(qkv, bias, pad, hist, batch, seq, heads, kv_heads, d, 10000.0)
    assert_close_f16(host(q), q32, wq, "q beyond the split")
    assert_close_f16(host(k), k32, wk, "k beyond the split")
    assert np.array_equal(host(v).view(np.uint16), wv.view(np.uint16))


# ---- softmax --------------------------------------------------------------------------------------------------------------

SOFTMAX_CASES = [
    # batch, heads, q_len, k_len
    (1, 2, 8, 8), (2, 3, 5, 64), (2, 4, 16, 512), (1, 2, 3, 1000), (4, 8, 1, 4096), (1, 1, 2, 8192),
    (1, 2, 3, 33), (2, 2, 2, 1), (1, 1, 1, 16384), (1, 3, 7, 264), (1, 1, 2, 20000),
]


def _causal_mask(rng, batch, q_len, k_len, dtype):
    lens = rng.integers(1, k_len + 1, batch)
    mask = np.zeros((batch, q_len, k_len), dtype)
    for b in range(batch):
        for qi in range(q_len):
            mask[b, qi, : max(1, lens[b] - (q_len - 1 - qi))] = 1
    return mask


@pytest.mark.parametrize("case", SOFTMAX_CASES)
def test_softmax_f32(ops, orc, rng, case):
    batch, heads, q_len, k_len = case
    qk = rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32) * 3
    mask = _causal_mask(rng, batch, q_len, k_len, np.float32)
    out = torch.empty(qk.shape, device="cuda:0")
    ops.launchScaleMaskAndSoftmax(dev(qk), dev(mask), out, 1.0 / np.sqrt(128.0))
    want, _ = orc.scale_mask_softmax(qk, mask, np.float32(1.0 / np.sqrt(128.0)))
    got = host(out)
    assert_close_f32(got, want, floor=1e-30, what="softmax f32")
    assert np.all(got[np.broadcast_to(mask[:, None] == 0, got.shape)] == 0.0)


@pytest.mark.parametrize("case", SOFTMAX_CASES)
def test_softmax_f16(ops, orc, rng, case):
    batch, heads, q_len, k_len = case
    qk = randn16(rng, (batch, heads, q_len, k_len), 3.0)
    mask = _causal_mask(rng, batch, q_len, k_len, np.float16)
    out = torch.empty(qk.shape, dtype=torch.float16, device="cuda:0")
    ops.launchScaleMaskAndSoftmax(dev(qk), dev(mask), out, 1.0 / np.sqrt(128.0))
    want, want32 = orc.scale_mask_softmax(qk, mask, np.float32(1.0 / np.sqrt(128.0)))
    err, over, same = assert_close_f16(host(out), want32, want, "softmax f16")
    assert over == 0 and err < 3e-4  # outputs are in [0, 1]: half spacing is at most 2^-11 there
    rows = host(out).astype(np.float64).sum(-1)
    assert np.all(np.abs(rows - 1.0) < 5e-3)


def test_softmax_fully_masked_rows_are_zero_and_in_place(ops, orc, rng):
    qk = rng.standard_normal((2, 2, 4, 128), dtype=np.float32)
    mask = np.ones((2, 4, 128), np.float32)
    mask[1, 2] = 0
    d = dev(qk)
    ops.launchScaleMaskAndSoftmax(d, dev(mask), d, 0.5)  # attn_score aliases qk
    want, _ = orc.scale_mask_softmax(qk, mask, 0.5)
    assert_close_f32(host(d), want, floor=1e-30, what="in-place softmax")
    assert np.all(host(d)[1, :, 2] == 0.0)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("case", SOFTMAX_CASES)
def test_causal_softmax_equals_mask_then_softmax(ops, orc, rng, case, dtype):
    # the fused call must reproduce the two calls it replaces and match the oracle run on the
    # oracle's mask
    batch, heads, q_len, k_len = case
    qk = (rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32) * 3).astype(dtype)
    ql = rng.integers(0, q_len + 1, batch)
    kl = np.minimum(ql + rng.integers(0, k_len + 1, batch), k_len)
    ql[0], kl[0] = min(q_len, k_len), min(q_len, k_len)
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    dqk, dql, dkl = dev(qk), _i32(ql), _i32(kl)
    mask = torch.empty((batch, q_len, k_len), dtype=tdt, device="cuda:0")
    two, fused = torch.empty(qk.shape, dtype=tdt, device="cuda:0"), torch.empty(qk.shape, dtype=tdt, device="cuda:0")
    scale = 1.0 / np.sqrt(128.0)
    ops.launchBuildCausalMasks(mask, dql, dkl)
    ops.launchScaleMaskAndSoftmax(dqk, mask, two, scale)
    ops.launchScaleCausalSoftmax(dqk, dql, dkl, fused, scale)
    # (the two routes may run different kernels for one shape, each the faster one for its inputs:
    # same arithmetic per element, sums in another order)
    if dtype == np.float16:
        assert np.max(np.abs(host(fused).astype(np.float32) - host(two).astype(np.float32))) <= 2.0 ** -11
    else:
        assert np.allclose(host(fused), host(two), rtol=3e-6, atol=1e-30)
    want, want32 = orc.scale_mask_softmax(qk, orc.build_causal_mask(ql, kl, q_len, k_len, dtype), np.float32(scale))
    if dtype == np.float16:
        err, over, _ = assert_close_f16(host(fused), want32, want, "causal softmax f16")
        assert over == 0 and err < 3e-4
    else:
        assert_close_f32(host(fused), want, floor=1e-30, what="causal softmax f32")


def test_causal_softmax_in_place_and_rows_past_qlen_are_zero(ops, rng):
    qk = rng.standard_normal((2, 3, 8, 64), dtype=np.float32)
    d = dev(qk)
    ops.launchScaleCausalSoftmax(d, _i32([8, 5]), _i32([8, 20]), d, 0.3)
    got = host(d)
    assert np.all(got[1, :, 5:] == 0.0)                      # rows q >= q_len
    assert np.all(got[1, :, :5, :15] == 0.0)                 # history keys before k_len - q_len
    assert np.allclose(got[0].sum(-1), 1.0, atol=1e-5) and np.allclose(got[1, :, :5].sum(-1), 1.0, atol=1e-5)
    assert np.all(np.triu(got[0, 0], 1) == 0.0)


# ---- top-K and sampling --------------------------------------------------------------------------------------------------------

def _topk_run(ops, probs, K, slices=8, index_offset=0, uniform=None, temperature=1.0):
    rows = probs.shape[0]
    tdt = torch.float16 if probs.dtype == np.float16 else torch.float32
    sc_i = torch.full((rows, slices, K), -5, dtype=torch.int32, device="cuda:0")
    sc_v = torch.zeros((rows, slices, K), dtype=tdt, device="cuda:0")
    f_i = torch.full((rows, K), -5, dtype=torch.int32, device="cuda:0")
    f_v = torch.zeros((rows, K), dtype=tdt, device="cuda:0")
    picked = torch.full((rows,), -9, dtype=torch.int32, device="cuda:0") if uniform is not None else None
    ops.launchTopKforBeamSearch(dev(probs), sc_i, sc_v, f_i, f_v, index_offset,
                                None if uniform is None else dev(uniform), temperature, picked)
    return host(f_i), host(f_v), None if picked is None else host(picked)


TOPK_CASES = [(256, 32000, 50), (3, 32000, 5), (7, 1000, 1), (4, 50, 50), (4, 30, 50), (2, 128256, 50), (5, 4097, 64),
              (3, 32001, 50), (2, 32000, 256), (1, 7, 3), (9, 5000, 17)]


@pytest.mark.parametrize("rows,vocab,K", TOPK_CASES)
def test_topk_f32_bit_exact(ops, orc, rng, rows, vocab, K):
    probs = (rng.standard_normal((rows, vocab), dtype=np.float32) * 2)
    got_i, got_v, _ = _topk_run(ops, probs, K)
    want_i, want_v = orc.topk(probs, K)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))


@pytest.mark.parametrize("rows,vocab,K", [(16, 32000, 50), (3, 999, 10)])
def test_topk_f16_bit_exact_with_many_ties(ops, orc, rng, rows, vocab, K):
    probs = randn16(rng, (rows, vocab), 2.0)  # half has few distinct values near the top: ties everywhere
    got_i, got_v, _ = _topk_run(ops, probs, K)
    want_i, want_v = orc.topk(probs, K)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(np.uint16), want_v.view(np.uint16))


@pytest.mark.parametrize("fill", ["zeros", "const", "two_values", "neg_zero_mix", "inf", "ramp_down", "ramp_up"])
def test_topk_adversarial_rows(ops, orc, rng, fill):
    rows, vocab, K = 3, 32000, 50
    probs = np.zeros((rows, vocab), np.float32)
    if fill == "const":
        probs[:] = 1.25
    elif fill == "two_values":
        probs[:] = rng.integers(0, 2, (rows, vocab)).astype(np.float32)
    elif fill == "neg_zero_mix":
        probs[:] = np.where(rng.integers(0, 2, (rows, vocab)) == 1, 0.0, -0.0).astype(np.float32)
    elif fill == "inf":
        probs[:] = rng.standard_normal((rows, vocab))
        probs[:, 100:140] = np.inf
        probs[:, 7] = -np.inf
    elif fill == "ramp_down":
        probs[:] = -np.arange(vocab, dtype=np.float32)
    elif fill == "ramp_up":
        probs[:] = np.arange(vocab, dtype=np.float32)
    got_i, got_v, _ = _topk_run(ops, probs, K)
    want_i, want_v = orc.topk(probs, K)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))


def test_topk_k_too_large_is_an_error(ops, rng):
    from inferspore_b200 import capi

    with pytest.raises(capi.IsporeError):
        _topk_run(ops, rng.standard_normal((2, 100), dtype=np.float32), 257)


@pytest.mark.parametrize("slices", [1, 2, 3, 8, 40])
@pytest.mark.parametrize("rows,vocab,K", [(3, 400000, 5), (2, 32000, 50), (300, 32000, 50), (5, 9000, 64)])
def test_topk_any_scratch_size(ops, orc, rng, slices, rows, vocab, K):
    """The scratch the caller brings only bounds how many slices a row is cut in: with one slice a CTA
    walks the whole row tile by tile and the merge round is skipped."""
    probs = (rng.standard_normal((rows, vocab), dtype=np.float32) * 2)
    probs[:, ::5] = np.round(probs[:, ::5])  # ties across tiles and slices
    u = rng.random(rows, dtype=np.float32)
    got_i, got_v, picked = _topk_run(ops, probs, K, slices=slices, uniform=u)
    want_i, want_v = orc.topk(probs, K)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))
    want_pick, margin = orc.sampling(want_i, want_v, u, 1.0)
    assert np.all(margin[picked != want_pick] < 1e-6)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("shape", ["noise", "rising", "falling", "steps", "negative"])
@pytest.mark.parametrize("vocab,K", [(100000, 50), (65536, 256), (70001, 100), (40000, 1)])
def test_topk_one_cta_walks_a_long_row(ops, orc, rng, dtype, shape, vocab, K):
    """One slice per row, so a CTA streams 5 to 13 tiles: later tiles park their survivors behind the
    running best and are ranked every few tiles.  `rising` makes every later tile beat the running
    K-th best with many elements (parked lists overflow: exact selection per tile), `steps` does so
    for some tiles only, `falling` and `noise` leave few or no survivors, `negative` keeps the
    threshold below zero (the slower order-key compare).  70001 is not a whole number of 128-bit
    vectors: plain loads instead of the TMA ring."""
    rows = 3
    x = rng.standard_normal((rows, vocab)).astype(np.float32)
    t = np.arange(vocab, dtype=np.float32) / vocab
    if shape == "rising":
        x += 8 * t
    elif shape == "falling":
        x -= 8 * t
    elif shape == "steps":
        x += 3.0 * ((np.arange(vocab) // 8192) % 3 == 2)
    elif shape == "negative":
        x = -np.abs(x) - 1.0
    probs = x.astype(dtype)
    got_i, got_v, _ = _topk_run(ops, probs, K, slices=1)
    want_i, want_v = orc.topk(probs, K)
    bits = np.uint32 if dtype == np.float32 else np.uint16
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(bits), want_v.view(bits))


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_topk_outliers_in_the_first_tile(ops, orc, rng, dtype):
    """Rows of several tiles first take a threshold from the first tile alone and rank once at the
    end.  Here the first tile holds 16 huge values, two under each warp (thread t of a CTA looks at
    the 128-bit vectors t, t + 256, ... of a tile), so that threshold is huge and only those 16
    elements of the whole row reach it — fewer than K: the row must still come out exact."""
    rows, vocab, K = 3, 32000, 50
    x = rng.standard_normal((rows, vocab)).astype(np.float32)
    E = 4 if dtype == np.float32 else 8
    for w in range(8):
        for t in (32 * w, 32 * w + 1):
            x[:, t * E] = 1000.0 + t  # first element of vector t of the first tile
    probs = x.astype(dtype)
    for slices in (1, 8):
        got_i, got_v, _ = _topk_run(ops, probs, K, slices=slices)
        want_i, want_v = orc.topk(probs, K)
        bits = np.uint32 if dtype == np.float32 else np.uint16
        assert np.array_equal(got_i, want_i)
        assert np.array_equal(got_v.view(bits), want_v.view(bits))


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("shape", ["noise", "rising", "steps", "flat", "negative"])
@pytest.mark.parametrize("vocab,K", [(20000, 50), (8192, 64), (17001, 5)])
def test_topk_more_rows_than_one_wave(ops, orc, rng, dtype, shape, vocab, K):
    """More rows than three CTAs per SM hold at once (CTA slots are reused within the launch), one
    slice per row, a round of 64 KB (two fp32 tiles, four fp16 tiles).  `flat` rows hold one
    value only (every vector of a tile survives the threshold: the per-warp lists overflow and the
    tile is selected exactly), `rising` and `steps` overflow the parked survivors of later tiles,
    `negative` keeps the threshold below zero, 17001 is not a whole number of 128-bit vectors."""
    rows = 600
    x = rng.standard_normal((rows, vocab)).astype(np.float32)
    t = np.arange(vocab, dtype=np.float32) / vocab
    if shape == "rising":
        x += 8 * t
    elif shape == "steps":
        x += 3.0 * ((np.arange(vocab) // 8192) % 2 == 1)
    elif shape == "flat":
        x[:] = 0.75
        x[::7, 100] = 2.0
    elif shape == "negative":
        x = -np.abs(x) - 1.0
    probs = x.astype(dtype)
    u = rng.random(rows, dtype=np.float32)
    got_i, got_v, picked = _topk_run(ops, probs, K, uniform=u)
    want_i, want_v = orc.topk(probs, K)
    bits = np.uint32 if dtype == np.float32 else np.uint16
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_v.view(bits), want_v.view(bits))
    want_pick, margin = orc.sampling(want_i, want_v, u, 1.0)
    assert np.all(margin[picked != want_pick] < 1e-6)


def test_topk_without_scratch(ops, orc, rng):
    probs = (rng.standard_normal((4, 20000), dtype=np.float32))
    f_i = torch.empty((4, 10), dtype=torch.int32, device="cuda:0")
    f_v = torch.empty((4, 10), dtype=torch.float32, device="cuda:0")
    from inferspore_b200 import capi
    capi.check(capi.load().ispore_topk_f32(dev(probs).data_ptr(), 4, 20000, 10, None, None, 0, f_i.data_ptr(),
                                           f_v.data_ptr(), 0, None, 1.0, None, None))
    want_i, want_v = orc.topk(probs, 10)
    assert np.array_equal(host(f_i), want_i) and np.array_equal(host(f_v), want_v)


def test_topk_merge_accepts_unsorted_lists(ops, orc, rng):
    rows, lists, K = 7, 5, 16
    ids = np.stack([rng.permutation(100000)[: lists * K] for _ in range(rows)]).astype(np.int32).reshape(rows, lists, K)
    vals = rng.integers(-3, 4, (rows, lists, K)).astype(np.float32)  # heavy ties, arbitrary order
    ids[:, 1, 3:] = -1  # a short list
    f_i = torch.empty((rows, K), dtype=torch.int32, device="cuda:0")
    f_v = torch.empty((rows, K), dtype=torch.float32, device="cuda:0")
    ops.launchTopKMerge(dev(ids), dev(vals), f_i, f_v)
    want_i, want_v = orc.topk_merge(ids, vals, K)
    assert np.array_equal(host(f_i), want_i) and np.array_equal(host(f_v), want_v)


def test_topk_vocab_sharded_merge_equals_unsharded(ops, orc, rng):
    rows, vocab, K, shards = 32, 32000, 50, 8
    probs = (rng.standard_normal((rows, vocab), dtype=np.float32) * 2)
    probs[:, ::97] = probs[:, 5:6]  # ties across shards
    want_i, want_v = orc.topk(probs, K)
    per = vocab // shards
    cand_i, cand_v = [], []
    for s in range(shards):
        i, v, _ = _topk_run(ops, np.ascontiguousarray(probs[:, s * per:(s + 1) * per]), K, index_offset=s * per)
        cand_i.append(i), cand_v.append(v)
    ci, cv = np.stack(cand_i, 1), np.stack(cand_v, 1)  # [rows, shards, K]: what an all-gather delivers
    f_i = torch.empty((rows, K), dtype=torch.int32, device="cuda:0")
    f_v = torch.empty((rows, K), dtype=torch.float32, device="cuda:0")
    ops.launchTopKMerge(dev(ci), dev(cv), f_i, f_v)
    assert np.array_equal(host(f_i), want_i) and np.array_equal(host(f_v), want_v)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,K,shards", [(32, 50, 8), (7, 5, 3), (3, 1, 2)])
def test_topk_merge_of_gathered_records_in_place(ops, orc, rng, dtype, rows, K, shards):
    """The merge reads an all-gather's output where it lies: one packed record per rank
    ([rows, K] int32 ids | [rows, K] values, padded to 16 bytes), list stride = record size."""
    vocab = 4000 * shards
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    probs = (rng.standard_normal((rows, vocab), dtype=np.float32) * 2).astype(dtype)
    probs[:, ::97] = probs[:, 5:6]  # ties across shards
    want_i, want_v = orc.topk(probs, K)
    per = vocab // shards
    record = ops.packed_record_bytes(rows, K, tdt)
    gathered = np.full((shards, record), 0xAB, np.uint8)
    for s in range(shards):
        i, v, _ = _topk_run(ops, np.ascontiguousarray(probs[:, s * per:(s + 1) * per]), K, index_offset=s * per)
        gathered[s, :rows * K * 4] = i.view(np.uint8).reshape(-1)
        gathered[s, rows * K * 4:rows * K * (4 + v.itemsize)] = v.view(np.uint8).reshape(-1)
    u = rng.random(rows, dtype=np.float32)
    f_i = torch.empty((rows, K), dtype=torch.int32, device="cuda:0")
    f_v = torch.empty((rows, K), dtype=tdt, device="cuda:0")
    picked = torch.empty(rows, dtype=torch.int32, device="cuda:0")
    ops.launchTopKMergeGathered(dev(gathered), shards, rows, K, f_i, f_v, dev(u), 0.9, picked)
    assert np.array_equal(host(f_i), want_i)
    assert np.array_equal(host(f_v).view(np.uint8), want_v.view(np.uint8))
    want_pick, margin = orc.sampling(want_i, want_v, u, 0.9)
    assert np.all(margin[host(picked) != want_pick] < 1e-6)


@pytest.mark.parametrize("temperature", [1.0, 0.7, 2.5])
def test_sampling_fused_and_standalone(ops, orc, rng, temperature):
    rows, vocab, K = 256, 32000, 50
    probs = (rng.standard_normal((rows, vocab), dtype=np.float32) * 2)
    u = rng.random(rows, dtype=np.float32)
    got_i, got_v, picked = _topk_run(ops, probs, K, uniform=u, temperature=temperature)
    want_i, want_v = orc.topk(probs, K)
    assert np.array_equal(got_i, want_i)
    want_pick, margin = orc.sampling(want_i, want_v, u, temperature)
    # a draw may legitimately differ only if u*S sits on a CDF boundary (expf differs in the last ulp)
    differ = picked != want_pick
    assert np.all(margin[differ] < 1e-6), f"{differ.sum()} picks differ away from a CDF boundary"
    assert differ.sum() <= 2
    out = torch.empty(rows, dtype=torch.int32, device="cuda:0")
    ops.launchSampling(dev(got_i), dev(got_v), dev(u), out, temperature)
    assert np.array_equal(host(out), picked)


# ---- layout kernels either side of attention: all bit-exact ----------------------------------------------

def _i32(a):
    return dev(np.ascontiguousarray(a, np.int32))


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("batch,max_q,max_k", [(1, 5, 5), (3, 7, 13), (4, 64, 128), (2, 1, 300), (5, 33, 40),
                                                (2, 512, 1024)])
def test_build_causal_mask(ops, orc, rng, dtype, batch, max_q, max_k):
    ql = rng.integers(0, max_q + 1, batch)
    kl = np.minimum(ql + rng.integers(0, max_k, batch), max_k)
    ql[0], kl[0] = min(max_q, max_k), min(max_q, max_k)  # the reference fixture's case: no history
    mask = torch.full((batch, max_q, max_k), 7.0, dtype=torch.float16 if dtype == np.float16 else torch.float32,
                      device="cuda:0")
    ops.launchBuildCausalMasks(mask, _i32(ql), _i32(kl))
    assert np.array_equal(host(mask), orc.build_causal_mask(ql, kl, max_q, max_k, dtype))


def test_build_causal_mask_fixture(ops):
    # tests/unittests/test_casual_mask.cu:45-68
    mask = torch.empty((1, 5, 5), device="cuda:0")
    ops.launchBuildCausalMasks(mask, _i32([3]), _i32([3]))
    want = np.zeros((1, 5, 5), np.float32)
    want[0, :3, :3] = np.tril(np.ones((3, 3)))
    assert np.array_equal(host(mask), want)


def test_build_causal_mask_unaligned_view(ops, orc):
    buf = torch.zeros(1 + 2 * 6 * 8, device="cuda:0")
    mask = buf[1:].view(2, 6, 8)  # 4-byte aligned only: scalar path
    ops.launchBuildCausalMasks(mask, _i32([6, 2]), _i32([8, 5]))
    assert np.array_equal(host(mask), orc.build_causal_mask([6, 2], [8, 5], 6, 8))
    assert float(buf[0]) == 0.0


@pytest.mark.parametrize("lens,max_q", [([3, 3, 3], 5), ([2, 0, 4, 1], 4), ([1], 1), ([4096] * 16, 4096),
                                        (None, 37)])
def test_cal_padding_offset(ops, orc, rng, lens, max_q):
    if lens is None:  # more sequences than one scan chunk holds
        lens = rng.integers(0, max_q + 1, 2500)
    batch = len(lens)
    po = torch.full((batch, max_q), -5, dtype=torch.int32, device="cuda:0")
    cum = torch.full((batch + 1,), -5, dtype=torch.int32, device="cuda:0")
    ops.launchCalPaddingoffset(po, cum, _i32(lens))
    want_po, want_cum = orc.cal_padding_offset(lens, max_q, fill=-5)
    assert np.array_equal(host(cum), want_cum)
    assert np.array_equal(host(po), want_po)  # entries past the total stay untouched


def test_cal_padding_offset_clamps_bad_lengths(ops, orc):
    po = torch.full((3, 4), -1, dtype=torch.int32, device="cuda:0")
    cum = torch.empty(4, dtype=torch.int32, device="cuda:0")
    ops.launchCalPaddingoffset(po, cum, _i32([9, -2, 3]))
    want_po, want_cum = orc.cal_padding_offset([9, -2, 3], 4)
    assert host(cum).tolist() == [0, 4, 4, 7] == want_cum.tolist()
    assert np.array_equal(host(po), want_po)


def test_cal_padding_offset_empty_batch(ops):
    po = torch.empty((0, 4), dtype=torch.int32, device="cuda:0")
    cum = torch.full((1,), -1, dtype=torch.int32, device="cuda:0")
    ops.launchCalPaddingoffset(po, cum, torch.empty(0, dtype=torch.int32, device="cuda:0"))
    assert host(cum).tolist() == [0]


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("lens,seq,heads,d", [([2, 3], 4, 2, 2), ([5, 1, 8], 8, 4, 128), ([7], 7, 3, 20),
                                              ([0, 6, 2], 6, 32, 64), ([100, 37], 100, 8, 128)])
def test_transpose_remove_padding(ops, orc, rng, dtype, lens, seq, heads, d):
    po, cum = orc.cal_padding_offset(lens, seq)
    tokens = int(cum[-1])
    offs = po.reshape(-1)[:tokens]
    inp = rng.standard_normal((len(lens), heads, seq, d), dtype=np.float32).astype(dtype)
    out = torch.full((tokens, heads, d), 3.0, dtype=torch.float16 if dtype == np.float16 else torch.float32,
                     device="cuda:0")
    ops.launchTransposeOutRemovePadding(dev(inp), _i32(offs), out)
    assert np.array_equal(host(out), orc.transpose_remove_padding(inp, offs, tokens))


def test_transpose_remove_padding_fixture(ops):
    # tests/unittests/test_fused_trans_remv_pad.cu:7-38
    inp = np.arange(32, dtype=np.float32).reshape(2, 2, 4, 2)
    out = torch.empty((5, 2, 2), device="cuda:0")
    ops.launchTransposeOutRemovePadding(dev(inp), _i32([0, 0, 2, 2, 2]), out)
    assert host(out).reshape(-1).tolist() == [0, 1, 8, 9, 2, 3, 10, 11, 16, 17, 24, 25, 18, 19, 26, 27, 20, 21, 28, 29]


def test_transpose_remove_padding_flags_bad_offset(ops):
    from inferspore_b200 import capi

    inp = torch.ones((1, 2, 4, 8), device="cuda:0")
    out = torch.zeros((3, 2, 8), device="cuda:0")
    ops.launchTransposeOutRemovePadding(inp, _i32([0, 50, 0]), out)
    torch.cuda.synchronize()
    assert capi.device_status(clear=True) & capi.DEV_BAD_PADDING
    got = host(out)
    assert (got[0] == 1).all() and (got[1] == 0).all() and (got[2] == 1).all()  # the bad token is skipped


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("layers,batch,kv,heads,max_seq,max_k,d", [(2, 1, 2, 2, 4, 2, 2), (3, 2, 2, 8, 64, 40, 128),
                                                                    (1, 3, 1, 5, 16, 16, 20), (2, 4, 8, 32, 128, 100, 64)])
def test_repeat_kv(ops, orc, rng, dtype, layers, batch, kv, heads, max_seq, max_k, d):
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    ksrc = rng.standard_normal((layers, batch, kv, max_seq, d), dtype=np.float32).astype(dtype)
    vsrc = rng.standard_normal((layers, batch, kv, max_seq, d), dtype=np.float32).astype(dtype)
    ctx = rng.integers(0, max_k + 1, batch)
    ctx[0] = max_k
    layer = layers - 1
    kd = torch.full((batch, heads, max_k, d), -9.0, dtype=tdt, device="cuda:0")
    vd = torch.full((batch, heads, max_k, d), -9.0, dtype=tdt, device="cuda:0")
    ops.launchRepeatKVCache(dev(ksrc), dev(vsrc), _i32(ctx), layer, kd, vd)
    fill = np.full((batch, heads, max_k, d), -9.0, dtype)
    assert np.array_equal(host(kd), orc.repeat_kv(fill, ksrc, ctx, layer, heads))
    assert np.array_equal(host(vd), orc.repeat_kv(fill, vsrc, ctx, layer, heads))


def test_repeat_kv_fixture(ops):
    # tests/unittests/test_repeat_kv.cu:14-56
    src = dev(np.arange(32, dtype=np.float32).reshape(2, 1, 2, 4, 2))
    kd, vd = torch.zeros((1, 2, 2, 2), device="cuda:0"), torch.zeros((1, 2, 2, 2), device="cuda:0")
    ops.launchRepeatKVCache(src, src, _i32([2]), 0, kd, vd)
    assert host(kd).reshape(-1).tolist() == [0, 1, 2, 3, 8, 9, 10, 11] == host(vd).reshape(-1).tolist()


def test_layout_ops_reject_bad_shapes(ops):
    with pytest.raises(Exception):
        ops.launchCalPaddingoffset(torch.empty((2, 4), dtype=torch.int32, device="cuda:0"),
                                   torch.empty(2, dtype=torch.int32, device="cuda:0"), _i32([1, 2]))
    src = torch.zeros((1, 1, 3, 4, 8), device="cuda:0")
    with pytest.raises(Exception):  # 4 heads over 3 kv heads
        ops.launchRepeatKVCache(src, src, _i32([1]), 0, torch.zeros((1, 4, 4, 8), device="cuda:0"),
                                torch.zeros((1, 4, 4, 8), device="cuda:0"))
    with pytest.raises(Exception):  # layer out of range
        ops.launchRepeatKVCache(src, src, _i32([1]), 1, torch.zeros((1, 3, 4, 8), device="cuda:0"),
                                torch.zeros((1, 3, 4, 8), device="cuda:0"))


# ---- decode-time fused masked multi-head attention ---------------------------------------------------

MHA_CASES = [
    # batch, heads, kv_heads, d, max_seq, step, rot_dim, bias, workspace
    (1, 2, 2, 128, 8, 4, 128, False, False),
    (2, 8, 8, 128, 64, 64, 128, True, False),
    (3, 8, 2, 128, 300, 257, 128, True, True),      # GQA, 4 q heads per CTA
    (2, 16, 2, 64, 128, 100, 32, False, True),      # 8 q heads per CTA, partial rotation
    (1, 6, 2, 128, 40, 33, 128, False, False),      # 3 q heads per kv head: one head per CTA
    (1, 4, 4, 128, 5000, 4100, 128, False, True),   # long context split over many CTAs
    (1, 4, 4, 128, 5000, 4100, 128, True, False),   # the same in one CTA per head
    (2, 4, 4, 32, 70, 1, 0, False, False),          # first token: the cache holds nothing yet
    (2, 2, 1, 256, 50, 50, 256, True, True),
    (2, 16, 2, 128, 200, 131, 128, True, True),     # 8 q heads per kv head on rows of 128
    (1, 8, 1, 128, 2100, 2049, 128, False, True),   # the same, chunks that end inside a 64-row tile
    (1, 8, 1, 128, 700, 650, 64, True, False),      # the same in one CTA, partial rotation
    (2, 8, 1, 128, 20, 1, 128, False, False),       # the same, first token
    (1, 24, 3, 128, 90, 17, 128, False, True),      # fewer rows than one warp's share of a tile
]


def _mha_inputs(rng, dtype, batch, heads, kv, d, max_seq, step, bias):
    layers = 2
    cast = (lambda a: a.astype(np.float16)) if dtype == np.float16 else (lambda a: a)
    qkv = cast(rng.standard_normal((batch, heads + 2 * kv, d), dtype=np.float32))
    kc = cast(rng.standard_normal((layers, batch, kv, max_seq, d), dtype=np.float32))
    vc = cast(rng.standard_normal((layers, batch, kv, max_seq, d), dtype=np.float32))
    b = cast((rng.standard_normal((heads + 2 * kv) * d) * 0.1).astype(np.float32)) if bias else None
    return qkv, kc, vc, b


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("case", MHA_CASES)
def test_decoder_masked_mha(ops, orc, rng, case, dtype):
    batch, heads, kv, d, max_seq, step, rot_dim, bias, use_ws = case
    if dtype == np.float32 and d > 128:
        pytest.skip("f32 rows are limited to 32 vectors of 4")
    qkv, kc, vc, b = _mha_inputs(rng, dtype, batch, heads, kv, d, max_seq, step, bias)
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    dk, dv = dev(kc), dev(vc)
    out = torch.full((batch, heads, d), 9.0, dtype=tdt, device="cuda:0")
    ws = None
    if use_ws:
        nbytes = ops.decoderMaskedMHAWorkspaceBytes(batch, heads, kv, d, step)
        ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device="cuda:0")
    ops.launchDecoderMaskedMHA(dev(qkv), None if b is None else dev(b), 1, dk, dv, None, step, out, rot_dim, 10000.0, ws)
    want, want_k, want_v, want32 = orc.decoder_masked_mha(qkv, b, kc, vc, 1, step, rot_dim, 10000.0)
    got_k, got_v = host(dk), host(dv)
    # everything but the new row is untouched; v of the new row is a copy (+ one rounded add)
    keep = np.ones(max_seq, bool)
    keep[step - 1] = False
    assert np.array_equal(got_k[0], kc[0]) and np.array_equal(got_v[0], vc[0])
    assert np.array_equal(got_k[1][:, :, keep], kc[1][:, :, keep]) and np.array_equal(got_v[1][:, :, keep], vc[1][:, :, keep])
    assert np.array_equal(got_v[1][:, :, step - 1], want_v[1][:, :, step - 1])
    if dtype == np.float16:
        # k of the new row: device and host sin/cos differ in the last bits, which can move a half rounding
        assert np.max(np.abs(got_k[1][:, :, step - 1].astype(np.float32) - want_k[1][:, :, step - 1].astype(np.float32))) <= 4e-3
        err, over, _ = assert_close_f16(host(out), want32, want, "decoder mha f16")
        assert over == 0
    else:
        # both are sums of O(1) terms that cancel: the relative bound is taken at magnitude 1
        assert_close_f32(got_k[1][:, :, step - 1], want_k[1][:, :, step - 1], floor=1.0, what="new k row")
        assert_close_f32(host(out), want32, floor=1.0, what="decoder mha f32")


def test_decoder_masked_mha_split_equals_unsplit(ops, rng):
    batch, heads, kv, d, max_seq, step = 1, 8, 8, 128, 3000, 2900
    qkv, kc, vc, _ = _mha_inputs(rng, np.float16, batch, heads, kv, d, max_seq, step, False)
    outs = []
    for use_ws in (False, True):
        nbytes = ops.decoderMaskedMHAWorkspaceBytes(batch, heads, kv, d, step)
        assert nbytes > 0  # a single sequence of 8 heads cannot fill the GPU unsplit
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0") if use_ws else None
        out = torch.empty((batch, heads, d), dtype=torch.float16, device="cuda:0")
        ops.launchDecoderMaskedMHA(dev(qkv), None, 0, dev(kc), dev(vc), None, step, out, 128, 10000.0, ws)
        outs.append(host(out).astype(np.float32))
    assert np.max(np.abs(outs[0] - outs[1])) <= 1e-3


def test_decoder_masked_mha_rejects_bad_shapes(ops):
    qkv = torch.zeros((1, 6, 24), device="cuda:0")  # 24 floats = 6 vectors: not a power of two
    kc = torch.zeros((1, 1, 2, 8, 24), device="cuda:0")
    out = torch.zeros((1, 2, 24), device="cuda:0")
    with pytest.raises(Exception):
        ops.launchDecoderMaskedMHA(qkv, None, 0, kc, kc.clone(), None, 1, out, 0, 10000.0)
    qkv = torch.zeros((1, 6, 32), device="cuda:0")
    kc = torch.zeros((1, 1, 2, 8, 32), device="cuda:0")
    out = torch.zeros((1, 2, 32), device="cuda:0")
    with pytest.raises(Exception):  # step beyond the cache
        ops.launchDecoderMaskedMHA(qkv, None, 0, kc, kc.clone(), None, 9, out, 0, 10000.0)
    with pytest.raises(Exception):  # layer out of range
        ops.launchDecoderMaskedMHA(qkv, None, 1, kc, kc.clone(), None, 1, out, 0, 10000.0)


# ---- stream capture: a decode step replayed from a CUDA graph ------------------------------------------

def test_decode_step_in_a_cuda_graph(ops, rng):
    """Every launcher of a decode step is captured into one CUDA graph (after one eager warm-up
    call, which performs the per-kernel attribute calls) and replayed on fresh inputs; the replay
    must reproduce the eager results bit for bit."""
    batch, heads, d, hidden, inter, step, max_seq, K = 8, 8, 128, 1024, 2816, 200, 256, 20
    g = torch.Generator(device="cuda:0")
    g.manual_seed(3)
    rnd = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda:0") * sc).half()
    x0, gamma = rnd(batch, hidden), (torch.rand(hidden, generator=g, device="cuda:0") + 0.5).half()
    qkv0 = rnd(batch, 3 * heads, d)
    kc0, vc0 = rnd(1, batch, heads, max_seq, d), rnd(1, batch, heads, max_seq, d)
    act0 = rnd(batch, 2, inter)
    logits0 = rnd(batch, 32000, sc=2.0).float()
    u = torch.rand(batch, generator=g, device="cuda:0")
    # working buffers the graph owns
    x, res, qkv, kc, vc, act = (t.clone() for t in (x0, x0, qkv0, kc0, vc0, act0))
    attn = torch.empty((batch, heads, d), dtype=torch.float16, device="cuda:0")
    act_out = torch.empty((batch, inter), dtype=torch.float16, device="cuda:0")
    ws = torch.empty(max(4, ops.decoderMaskedMHAWorkspaceBytes(batch, heads, heads, d, step)), dtype=torch.uint8,
                     device="cuda:0")
    top_i = torch.empty((batch, K), dtype=torch.int32, device="cuda:0")
    top_v = torch.empty((batch, K), device="cuda:0")
    sc_i = torch.empty((batch, 8, K), dtype=torch.int32, device="cuda:0")
    sc_v = torch.empty((batch, 8, K), device="cuda:0")
    picked = torch.empty(batch, dtype=torch.int32, device="cuda:0")

    def reset():
        for dst, src in ((x, x0), (qkv, qkv0), (kc, kc0), (vc, vc0), (act, act0)):
            dst.copy_(src)

    def decode_step():
        ops.launchRMSNorm(x, res, gamma, 1e-6)
        ops.launchDecoderMaskedMHA(qkv, None, 0, kc, vc, None, step, attn, d, 10000.0, ws)
        ops.launchFusedAddBiasResidualRMSNorm(res, x, None, gamma, 1e-6)
        ops.launchAct(act, act_out)
        ops.launchTopKforBeamSearch(logits0, sc_i, sc_v, top_i, top_v, 0, u, 1.0, picked)

    outputs = lambda: [t.clone() for t in (x, res, kc, vc, attn, act_out, top_i, top_v, picked)]
    reset()
    decode_step()
    torch.cuda.synchronize()
    eager = outputs()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    reset()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            decode_step()
    for _ in range(2):
        reset()
        graph.replay()
        torch.cuda.synchronize()
        for got, want in zip(outputs(), eager):
            assert torch.equal(got, want)


def test_softmax_many_short_sequences(ops, orc, rng):
    # 70,000 sequences of one 8-key row: more units than any single grid axis but x could index
    batch, heads, q_len, k_len = 70000, 2, 1, 8
    qk = rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32)
    mask = (rng.random((batch, q_len, k_len)) < 0.7).astype(np.float32)
    out = torch.empty(qk.shape, device="cuda:0")
    ops.launchScaleMaskAndSoftmax(dev(qk), dev(mask), out, 0.5)
    want, _ = orc.scale_mask_softmax(qk, mask, np.float32(0.5))
    assert_close_f32(host(out), want, floor=1e-30, what="softmax, many short sequences")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("case", [(2, 5, 7, 777), (1, 3, 2, 4099), (3, 4, 5, 37), (1, 2, 3, 1001)])
def test_softmax_rows_not_16_byte_aligned_in_place(ops, orc, rng, case, dtype):
    # k_len is not a multiple of the 128-bit vector: rows start at arbitrary offsets inside aligned
    # vectors, neighbouring rows share a vector, and attn_score aliases qk
    batch, heads, q_len, k_len = case
    qk = (rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32) * 3).astype(dtype)
    mask = _causal_mask(rng, batch, q_len, k_len, dtype)
    d = dev(qk)
    ops.launchScaleMaskAndSoftmax(d, dev(mask), d, 0.25)
    want, want32 = orc.scale_mask_softmax(qk, mask, np.float32(0.25))
    if dtype == np.float16:
        err, over, _ = assert_close_f16(host(d), want32, want, "unaligned softmax f16")
        assert over == 0
    else:
        assert_close_f32(host(d), want, floor=1e-30, what="unaligned softmax f32")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("k_len", [9, 15, 17, 31, 255, 263, 513, 777, 1023, 1029, 2047, 3001, 4099, 6143, 8191, 12289, 20001])
def test_softmax_any_row_length_random_mask(ops, orc, rng, k_len, dtype):
    # the mask row and the qk row of a (b, h, q) start at different offsets inside their aligned
    # vectors; 3 heads x 3 q rows x 2 sequences go through every relative shift for odd k_len, and
    # a random 0/1 mask shows any element that was paired with the wrong mask entry
    batch, heads, q_len = 2, 3, 3
    qk = (rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32) * 3).astype(dtype)
    mask = (rng.random((batch, q_len, k_len)) < 0.6).astype(dtype)
    mask[1, 1] = 0  # a fully masked row
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    out = torch.full(qk.shape, 7.0, dtype=tdt, device="cuda:0")
    ops.launchScaleMaskAndSoftmax(dev(qk), dev(mask), out, 0.3)
    want, want32 = orc.scale_mask_softmax(qk, mask, np.float32(0.3))
    if dtype == np.float16:
        err, over, _ = assert_close_f16(host(out), want32, want, "softmax f16, any row length")
        assert over == 0
    else:
        assert_close_f32(host(out), want, floor=1e-30, what="softmax f32, any row length")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("case", [(3, 5, 9, 45), (2, 3, 11, 333), (1, 2, 5, 1501), (1, 1, 3, 5003)])
def test_causal_softmax_any_row_length(ops, orc, rng, case, dtype):
    batch, heads, q_len, k_len = case
    qk = (rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32) * 3).astype(dtype)
    ql = rng.integers(1, q_len + 1, batch)
    kl = np.minimum(ql + rng.integers(0, k_len + 1, batch), k_len)
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    d = dev(qk)
    ops.launchScaleCausalSoftmax(d, _i32(ql), _i32(kl), d, 0.2)  # in place
    want, want32 = orc.scale_mask_softmax(qk, orc.build_causal_mask(ql, kl, q_len, k_len, dtype), np.float32(0.2))
    if dtype == np.float16:
        err, over, _ = assert_close_f16(host(d), want32, want, "causal softmax f16, any row length")
        assert over == 0
    else:
        assert_close_f32(host(d), want, floor=1e-30, what="causal softmax f32, any row length")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("case", [(2, 3, 5, 8192), (1, 2, 3, 8200), (2, 2, 7, 12000), (1, 3, 4, 16384), (1, 40, 9, 16384),
                                  (1, 2, 3, 20000), (1, 1, 2, 32768), (2, 3, 5, 5000), (1, 70, 9, 6008), (1, 33, 7, 3000),
                                  (2, 2, 3, 4104), (2, 5, 3, 1536), (1, 200, 11, 2560), (3, 50, 7, 1792), (1, 9, 40, 2048)])
def test_softmax_long_rows_through_the_staged_ring(ops, orc, rng, case, causal, dtype):
    """Rows of whole vectors beyond 16 KB — and rows of 8 to 16 KB that are not a power of two long
    (5000, 6008 in fp16; 3000, 4104 in fp32), four warps per row, and of 4 to 8 KB between the powers
    of two (3000, 2560 in fp16; 1536 in fp32 with a mask tensor), two warps per row — travel through a ring of
    shared-memory row buffers (bulk copies in, bulk stores out), two CTAs of 256 threads per SM or
    one of 512 for the longest; a CTA
    walks rows b, b + grid, ... — (1, 40, 9, 16384) gives every CTA several trips and wraps the
    ring — and fetches each row's mask slice a trip ahead.  In place, mask tensor and mask-free."""
    batch, heads, q_len, k_len = case
    if dtype == np.float32 and k_len > 16384:
        pytest.skip("fp32 rows beyond 4096 vectors take the generic kernel")
    qk = (rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32) * 3).astype(dtype)
    d = dev(qk)
    if causal:
        ql = rng.integers(1, q_len + 1, batch)
        kl = np.minimum(ql + rng.integers(k_len // 2, k_len + 1, batch), k_len)
        ops.launchScaleCausalSoftmax(d, _i32(ql), _i32(kl), d, 0.2)
        mask = orc.build_causal_mask(ql, kl, q_len, k_len, dtype)
    else:
        mask = (rng.random((batch, q_len, k_len)) < 0.7).astype(dtype)
        mask[0, q_len - 1] = 0  # a fully masked row
        ops.launchScaleMaskAndSoftmax(d, dev(mask), d, 0.2)
    want, want32 = orc.scale_mask_softmax(qk, mask, np.float32(0.2))
    if dtype == np.float16:
        err, over, _ = assert_close_f16(host(d), want32, want, "long-row softmax f16")
        assert over == 0
    else:
        assert_close_f32(host(d), want, floor=1e-30, what="long-row softmax f32")


@pytest.mark.parametrize("case", [(3000, 7, 3, 17), (2, 1, 4, 19), (5, 16, 1, 23), (1, 3, 1025, 9), (700, 3, 2, 35)])
def test_softmax_any_row_length_row_index_recovery(ops, orc, rng, case):
    # many rows, one head, one q row, q_len a power of two and not: (sequence, head, q) are
    # recovered from the flat row by multiply-shift division, and the mask row depends on them
    batch, heads, q_len, k_len = case
    qk = rng.standard_normal((batch, heads, q_len, k_len), dtype=np.float32)
    mask = (rng.random((batch, q_len, k_len)) < 0.5).astype(np.float32)
    out = torch.empty(qk.shape, device="cuda:0")
    ops.launchScaleMaskAndSoftmax(dev(qk), dev(mask), out, 0.7)
    want, _ = orc.scale_mask_softmax(qk, mask, np.float32(0.7))
    assert_close_f32(host(out), want, floor=1e-30, what="softmax, row index recovery")
