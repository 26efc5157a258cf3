#!/usr/bin/env python
"""Benchmark of the fused layer-kernel chain on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the per-layer fused kernels over one batch of synthetic
Llama-2-7B-shaped input (fp16 activations, seeded): embedding gather ->
plain RMSNorm -> QKV bias+RoPE+head transpose -> KV-cache concat -> scale+mask+
softmax -> residual add+RMSNorm -> SiLU(gate)*up -> top-K(50)+sampling.  Every
rank owns its own batch (token-axis sharding, no data-path collective), so
scaling is weak: per-GPU work is fixed as N grows.

Rank 0 prints ONE JSON line.  `value` is rows (tokens) per second through the
chain with inputs resident in HBM; `e2e` is the same chain driven from pinned
host buffers with the host<->device copies inside the timed region; `kernels`
gives rows/s and algorithmic GB/s per kernel; `roofline` is the kernel that
moves the most bytes (SiLU*up); `cpu_baseline` (N=1 only) is the reference's
CPU code / the oracle port timed on the host cores on a bounded sample.

--impl reference times that CPU chain alone, on the same metric and unit.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Llama-2-7B constants (reference: src/utils/model_utils.h:15-29)
HIDDEN, INTER, HEADS, KV_HEADS, HEAD_SIZE, VOCAB = 4096, 11008, 32, 32, 128, 32000
SEQ, ROT_DIM, ROT_BASE, TOPK_K, TOPK_ROWS, EPS = 512, 128, 10000.0, 50, 256, 1e-6
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
KERNELS = ["input_embedding", "rmsnorm", "qkv_bias_rope_transpose", "concat_kv", "scale_mask_softmax",
           "add_residual_rmsnorm", "silu_mul", "topk_sampling"]
LAUNCHES_PER_STEP = 8  # one per kernel (at 256 rows top-K runs one slice per row and samples in the same launch)
# DRAM traffic of the roofline kernel (SiLU*up) from the ncu capture summarised in
# profiles/silu_mul_16384tok.md: dram__bytes_read.sum + dram__bytes_write.sum of one launch at 16,384
# tokens (1,037.6 MB) over that launch's algorithmic bytes (1,082.1 MB).  The kernel is a flat
# streaming pass, so traffic grows in proportion to the rows; a full-size launch is scaled by it.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1037.6 / 1082.13


def algorithmic_bytes(tokens: int, topk_rows: int) -> dict:
    """Bytes each kernel must move per step: every input read once, every output written once (fp16;
    fp32 logits for top-K)."""
    s, T, B = 2, tokens, tokens // SEQ
    return {
        "input_embedding": T * 4 + 2 * T * HIDDEN * s,
        "rmsnorm": 3 * T * HIDDEN * s + HIDDEN * s,  # read x, write normed x and the residual copy
        "qkv_bias_rope_transpose": 2 * T * 3 * HIDDEN * s + 3 * HIDDEN * s + T * 4 + 2 * B * 4,
        "concat_kv": 2 * 2 * T * KV_HEADS * HEAD_SIZE * s + 2 * B * 4,
        "scale_mask_softmax": 2 * B * HEADS * SEQ * SEQ * s + B * SEQ * SEQ * s,
        "add_residual_rmsnorm": 4 * T * HIDDEN * s + HIDDEN * s,
        "silu_mul": 3 * T * INTER * s,
        "topk_sampling": topk_rows * VOCAB * 4 + topk_rows * TOPK_K * 8 + 2 * topk_rows * 4,
    }


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- clocks --------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz, self._stop, self._thread = None, threading.Event(), None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.reasons.update(n for n, bit in names.items() if mask & bit)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- the CPU chain (reference CPU functions where they exist, the oracle port elsewhere) ------------

class CpuChain:
    """The same chain on the host cores, fp32 (the reference's CPU functions are fp32): reference
    code from oracle/_ref/ for SiLU*up, embedding, QKV+RoPE and residual+RMSNorm
    (tests/unittests/test_{act,input_embedding,bias_and_RoPE,fused_addresidual_norm}.cu), the oracle
    port for plain RMSNorm, KV concat, softmax and top-K+sampling (the reference has no CPU code for
    those).  The reference functions are single-threaded loops over rows, so rows are split over a
    thread pool; the oracle port uses OpenMP."""

    def __init__(self, tokens: int, threads: int, seed: int = 1234):
        from oracle import binding as orc

        self.orc, self.tokens, self.threads = orc, tokens, threads
        self.batch = max(1, tokens // SEQ)
        self.seq = min(SEQ, tokens)
        self.topk_rows = max(1, TOPK_ROWS * tokens // 65536)
        rng = np.random.default_rng(seed)
        f32 = np.float32
        self.ids = rng.integers(0, VOCAB, tokens).astype(np.int32)
        self.table = (rng.standard_normal((VOCAB, HIDDEN), dtype=f32) * 0.02)
        self.gamma = rng.uniform(0.5, 1.5, HIDDEN).astype(f32)
        self.x = rng.standard_normal((tokens, HIDDEN), dtype=f32)
        self.res = rng.standard_normal((tokens, HIDDEN), dtype=f32)
        self.qkv = rng.standard_normal((tokens, 3 * HEADS, HEAD_SIZE), dtype=f32)
        self.bias = (rng.standard_normal(3 * HIDDEN, dtype=f32) * 0.02)
        self.k_src = rng.standard_normal((self.batch, KV_HEADS, self.seq, HEAD_SIZE), dtype=f32)
        self.cache = np.zeros((1, self.batch, KV_HEADS, self.seq, HEAD_SIZE), f32)
        self.qk = rng.standard_normal((self.batch, HEADS, self.seq, self.seq), dtype=f32) * 3
        self.mask = np.tril(np.ones((self.seq, self.seq), f32))[None].repeat(self.batch, 0)
        self.act_in = rng.standard_normal((tokens, 2, INTER), dtype=f32)
        self.logits = rng.standard_normal((self.topk_rows, VOCAB), dtype=f32) * 2
        self.u = rng.random(self.topk_rows, dtype=f32)
        self.zeros_h = np.zeros(HIDDEN, f32)
        self.pool = ThreadPoolExecutor(max_workers=threads)
        self.use_ref = all(orc.ref_available(n) for n in
                           ("libref_act.so", "libref_embedding.so", "libref_norm.so", "libref_rope.so"))
        orc.set_threads(threads)

    @property
    def kind(self) -> str:
        return "reference" if self.use_ref else "port"

    def _split(self, n):
        step = -(-n // self.threads)
        return [(a, min(n, a + step)) for a in range(0, n, step)]

    def step(self) -> None:
        orc, T = self.orc, self.tokens
        if self.use_ref:
            list(self.pool.map(lambda ab: orc.ref_cpu_embedding(self.ids[ab[0]:ab[1]], self.table), self._split(T)))
        else:
            orc.input_embedding(self.ids, self.table)
        orc.rmsnorm(self.x, self.gamma, EPS, want_copy=True)
        if self.use_ref:
            # CPUfunc walks [batch, seq]; a chunk of one sequence is a batch-1 call whose history
            # length is the chunk's first position, so every thread gets an equal share of tokens.
            def rope(ab):
                a, b = ab
                while a < b:
                    n = min(b, (a // self.seq + 1) * self.seq) - a
                    orc.ref_cpu_qkv_rope(self.qkv[a:a + n], self.bias, np.array([a % self.seq], np.int32), 1, n,
                                         HEADS, KV_HEADS, HEAD_SIZE, ROT_DIM, ROT_BASE)
                    a += n
            list(self.pool.map(rope, self._split(T)))
        else:
            orc.qkv_bias_rope_transpose(self.qkv, self.bias, np.zeros(T, np.int32), np.zeros(self.batch, np.int32),
                                        self.batch, self.seq, HEADS, KV_HEADS, ROT_DIM, ROT_BASE)
        cur = np.full(self.batch, self.seq, np.int32)
        hist = np.zeros(self.batch, np.int32)
        orc.concat_kv(self.cache, self.k_src, cur, hist, 0)
        orc.concat_kv(self.cache, self.k_src, cur, hist, 0)
        orc.scale_mask_softmax(self.qk, self.mask, np.float32(1.0 / np.sqrt(HEAD_SIZE)))
        if self.use_ref:
            list(self.pool.map(lambda ab: orc.ref_cpu_fused_resid_rmsnorm(self.res[ab[0]:ab[1]], self.x[ab[0]:ab[1]],
                                                                          self.zeros_h, self.gamma, EPS),
                               self._split(T)))
            list(self.pool.map(lambda ab: orc.ref_cpu_swiglu(self.act_in[ab[0]:ab[1]]), self._split(T)))
        else:
            orc.add_residual_rmsnorm(self.x, self.res, None, self.gamma, EPS)
            orc.silu_mul(self.act_in)
        ids, vals = orc.topk(self.logits, TOPK_K)
        orc.sampling(ids, vals, self.u, 1.0)

    def describe(self) -> str:
        src = ("reference CPU functions (SiLU*up, embedding, QKV+RoPE, residual+RMSNorm) + oracle port "
               "(plain RMSNorm, KV concat, softmax, top-K+sampling)") if self.use_ref else "oracle port for every kernel"
        return (f"{self.tokens} tokens ({self.batch} x {self.seq}) + {self.topk_rows} top-K rows per step, fp32, "
                f"{src}")


def time_cpu_chain(tokens: int, threads: int, steps: int, warmup: int, budget_s: float = 200.0):
    """Returns (rows/s, seconds per step, chain); shrinks the sample until steps+warmup fit the budget."""
    while True:
        chain = CpuChain(tokens, threads)
        t0 = time.perf_counter()
        chain.step()
        first = time.perf_counter() - t0
        if first * (steps + warmup) <= budget_s or tokens <= SEQ:
            break
        tokens = max(SEQ, tokens // 2)
    for _ in range(max(0, warmup - 1)):
        chain.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        chain.step()
    dt = (time.perf_counter() - t0) / steps
    return chain.tokens / dt, dt, chain


# ---- the GPU chain --------------------------------------------------------------------------------------

class GpuChain:
    def __init__(self, tokens: int, device, seed: int, topk_buffers: int = 5):
        import torch

        from inferspore_b200 import ops

        self.torch, self.ops, self.dev, self.tokens = torch, ops, device, tokens
        self.batch = tokens // SEQ
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        h = torch.float16

        def randn(*shape, dtype=h, scale=1.0):
            return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)

        T, B = tokens, self.batch
        self.ids = torch.randint(0, VOCAB, (T,), generator=g, device=device, dtype=torch.int32)
        self.table = randn(VOCAB, HIDDEN, scale=0.02)
        self.gamma = (torch.rand(HIDDEN, generator=g, device=device) + 0.5).to(h)
        self.x = torch.empty((T, HIDDEN), dtype=h, device=device)        # embedding out, normed in place
        self.res = torch.empty((T, HIDDEN), dtype=h, device=device)      # residual stream
        self.qkv = randn(T, 3 * HEADS, HEAD_SIZE)
        self.bias = randn(3 * HIDDEN, scale=0.02)
        self.pad = torch.zeros(T, dtype=torch.int32, device=device)
        self.hist = torch.zeros(B, dtype=torch.int32, device=device)
        self.inlen = torch.full((B,), SEQ, dtype=torch.int32, device=device)
        self.q = torch.empty((B, HEADS, SEQ, HEAD_SIZE), dtype=h, device=device)
        self.k = torch.empty((B, KV_HEADS, SEQ, HEAD_SIZE), dtype=h, device=device)
        self.v = torch.empty_like(self.k)
        self.k_cache = torch.zeros((1, B, KV_HEADS, SEQ, HEAD_SIZE), dtype=h, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.qk = randn(B, HEADS, SEQ, SEQ, scale=3.0)
        self.score = torch.empty_like(self.qk)
        self.mask = torch.tril(torch.ones((SEQ, SEQ), dtype=h, device=device))[None].repeat(B, 1, 1).contiguous()
        self.attn_out = randn(T, HIDDEN)                                   # stands for the o-proj GEMM output
        self.act_in = randn(T, 2, INTER)
        self.act_out = torch.empty((T, INTER), dtype=h, device=device)
        self.logits = [randn(TOPK_ROWS, VOCAB, dtype=torch.float32, scale=2.0) for _ in range(topk_buffers)]
        self.u = torch.rand(TOPK_ROWS, generator=g, device=device)
        self.sc_i = torch.empty((TOPK_ROWS, 8, TOPK_K), dtype=torch.int32, device=device)
        self.sc_v = torch.empty((TOPK_ROWS, 8, TOPK_K), dtype=torch.float32, device=device)
        self.top_i = torch.empty((TOPK_ROWS, TOPK_K), dtype=torch.int32, device=device)
        self.top_v = torch.empty((TOPK_ROWS, TOPK_K), dtype=torch.float32, device=device)
        self.picked = torch.empty(TOPK_ROWS, dtype=torch.int32, device=device)
        self.scale = 1.0 / float(np.sqrt(HEAD_SIZE))
        self.n = 0

    def launchers(self):
        """The chain as (kernel name, launch closure) pairs, in order."""
        o = self.ops
        return [
            ("input_embedding", lambda: o.launchInputEmbedding(self.ids, self.x, self.table)),
            ("rmsnorm", lambda: o.launchRMSNorm(self.x, self.res, self.gamma, EPS)),
            ("qkv_bias_rope_transpose", lambda: o.launchAddFusedQKVBiasTransposeAndRoPE(
                self.q, self.k, self.v, self.qkv, self.bias, self.pad, self.hist, self.inlen, ROT_DIM, ROT_BASE)),
            ("concat_kv", lambda: o.launchConcatKVCache(self.k, self.v, 0, self.inlen, self.hist, self.k_cache,
                                                        self.v_cache)),
            ("scale_mask_softmax", lambda: o.launchScaleMaskAndSoftmax(self.qk, self.mask, self.score, self.scale)),
            ("add_residual_rmsnorm", lambda: o.launchFusedAddBiasResidualRMSNorm(self.res, self.attn_out, None,
                                                                                 self.gamma, EPS)),
            ("silu_mul", lambda: o.launchAct(self.act_in, self.act_out)),
            ("topk_sampling", self._topk),
        ]

    def _topk(self):
        self.ops.launchTopKforBeamSearch(self.logits[self.n % len(self.logits)], self.sc_i, self.sc_v, self.top_i,
                                         self.top_v, 0, self.u, 1.0, self.picked)
        self.n += 1

    def step(self, events=None) -> None:
        """Launches the chain on the current stream; `events` (len 9) are recorded around each kernel."""
        for i, (_, launch) in enumerate(self.launchers()):
            if events is not None:
                events[i].record()
            launch()
        if events is not None:
            events[8].record()


NEXT_KERNELS = ["build_causal_mask", "scale_causal_softmax", "scale_mask_softmax_len777", "cal_padding_offset",
                "transpose_remove_padding",
                "repeat_kv", "decoder_masked_mha", "decoder_masked_mha_gqa8"]


class NextRows:
    """The kernels either side of the chain (mask build, mask-free softmax, padding offsets,
    transpose + remove padding, repeat-KV, decode-time fused attention), each at a Llama-2-7B shape
    derived from `tokens` (prefill: tokens/512 sequences of 512) and `decode_batch` sequences with
    `context` cached positions.  Timed one by one, outside the step the headline metric counts."""

    def __init__(self, tokens: int, device, seed: int = 77, decode_batch: int = 64, context: int = 4096):
        import torch

        from inferspore_b200 import ops

        self.torch, self.ops, self.dev = torch, ops, device
        self.tokens, self.batch, self.decode_batch, self.context = tokens, tokens // SEQ, decode_batch, context
        self.g = torch.Generator(device=device)
        self.g.manual_seed(seed)
        self._bufs = {}

    def _randn(self, *shape, scale=1.0):
        t = self.torch
        return (t.randn(*shape, generator=self.g, device=self.dev, dtype=t.float32) * scale).to(t.float16)

    def _i32(self, values):
        return self.torch.tensor(values, dtype=self.torch.int32, device=self.dev)

    def prepare(self, name: str):
        """Allocates the kernel's buffers; returns (launch closure, algorithmic bytes, workload text)."""
        t, o, h = self.torch, self.ops, self.torch.float16
        B, T, dev = self.batch, self.tokens, self.dev
        if name == "build_causal_mask":
            mask = t.empty((B, SEQ, SEQ), dtype=h, device=dev)
            ql = self._i32([SEQ] * B)
            return (lambda: o.launchBuildCausalMasks(mask, ql, ql)), mask.numel() * 2, f"mask [{B}, {SEQ}, {SEQ}] f16"
        if name == "scale_causal_softmax":
            qk = self._randn(B, HEADS, SEQ, SEQ, scale=3.0)
            out = t.empty_like(qk)
            ql = self._i32([SEQ] * B)
            return ((lambda: o.launchScaleCausalSoftmax(qk, ql, ql, out, 1.0 / float(np.sqrt(HEAD_SIZE)))),
                    2 * qk.numel() * 2, f"qk [{B}, {HEADS}, {SEQ}, {SEQ}] f16, no mask tensor")
        if name == "scale_mask_softmax_len777":
            # prompts of 777 tokens: rows that are not a whole number of 128-bit vectors, so every
            # row (and every mask row) starts at another offset inside its aligned vectors
            n, bs = 777, max(1, self.tokens // 4096)
            qk = self._randn(bs, HEADS, n, n, scale=3.0)
            out = t.empty_like(qk)
            mask = t.tril(t.ones((n, n), dtype=h, device=dev)).expand(bs, n, n).contiguous()
            return ((lambda: o.launchScaleMaskAndSoftmax(qk, mask, out, 1.0 / float(np.sqrt(HEAD_SIZE)))),
                    2 * qk.numel() * 2 + mask.numel() * 2, f"qk [{bs}, {HEADS}, {n}, {n}] f16 + mask [{bs}, {n}, {n}]")
        if name == "cal_padding_offset":
            lens = self._i32([SEQ] * B)
            po = t.empty((B, SEQ), dtype=t.int32, device=dev)
            cum = t.empty(B + 1, dtype=t.int32, device=dev)
            return (lambda: o.launchCalPaddingoffset(po, cum, lens)), B * SEQ * 4 + (2 * B + 1) * 4, f"{B} sequences of {SEQ}"
        if name == "transpose_remove_padding":
            x = self._randn(B, HEADS, SEQ, HEAD_SIZE)
            out = t.empty((T, HEADS, HEAD_SIZE), dtype=h, device=dev)
            po = t.zeros(T, dtype=t.int32, device=dev)
            return ((lambda: o.launchTransposeOutRemovePadding(x, po, out)), 2 * x.numel() * 2 + T * 4,
                    f"[{B}, {HEADS}, {SEQ}, {HEAD_SIZE}] f16 -> [{T}, {HEADS}, {HEAD_SIZE}]")
        if name == "repeat_kv":  # a grouped-query shape: 8 kv heads under the 32 q heads
            bs, kvh, ctx = 16, 8, 2048
            ks, vs = self._randn(1, bs, kvh, 2 * ctx, HEAD_SIZE), self._randn(1, bs, kvh, 2 * ctx, HEAD_SIZE)
            kd = t.empty((bs, HEADS, ctx, HEAD_SIZE), dtype=h, device=dev)
            vd = t.empty_like(kd)
            cl = self._i32([ctx] * bs)
            nbytes = 2 * kd.numel() * 2 + 2 * bs * kvh * ctx * HEAD_SIZE * 2
            return ((lambda: o.launchRepeatKVCache(ks, vs, cl, 0, kd, vd)), nbytes,
                    f"{bs} sequences, {kvh} -> {HEADS} heads, context {ctx}, f16")
        if name in ("decoder_masked_mha", "decoder_masked_mha_gqa8"):
            # the model's own 32/32 heads, and 64 q heads on 8 kv heads (eight q heads share each cache row)
            heads, kvh = (HEADS, KV_HEADS) if name == "decoder_masked_mha" else (64, 8)
            bs, ctx = self.decode_batch, self.context
            qkv = self._randn(bs, heads + 2 * kvh, HEAD_SIZE)
            kc, vc = self._randn(1, bs, kvh, ctx, HEAD_SIZE), self._randn(1, bs, kvh, ctx, HEAD_SIZE)
            out = t.empty((bs, heads, HEAD_SIZE), dtype=h, device=dev)
            nb = o.decoderMaskedMHAWorkspaceBytes(bs, heads, kvh, HEAD_SIZE, ctx)
            ws = t.empty(max(nb, 4), dtype=t.uint8, device=dev)
            nbytes = 2 * bs * kvh * ctx * HEAD_SIZE * 2 + qkv.numel() * 2 + out.numel() * 2
            return ((lambda: o.launchDecoderMaskedMHA(qkv, None, 0, kc, vc, None, ctx, out, ROT_DIM, ROT_BASE, ws)), nbytes,
                    f"{bs} sequences, {heads} q / {kvh} kv heads, step {ctx}, f16 caches ({nb >> 10} KiB split workspace)")
        raise KeyError(name)

    def time_one(self, name: str, steps: int, warmup: int):
        t = self.torch
        launch, nbytes, workload = self.prepare(name)
        for _ in range(max(3, warmup)):
            launch()
        t.cuda.synchronize()
        s, e = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            launch()
        e.record()
        t.cuda.synchronize()
        return s.elapsed_time(e) / steps, nbytes, workload

    def decode_small_kernels(self, iters: int = 50) -> dict:
        """The launch-bound kernels of one decode step at `decode_batch` sequences (plain RMSNorm,
        residual add + RMSNorm, SiLU*up, top-K + sampling): time per step launched one by one and
        replayed from a CUDA graph (the C ABI is capturable after one warm-up call)."""
        t, o, h, dev, bs = self.torch, self.ops, self.torch.float16, self.dev, self.decode_batch
        x, res = self._randn(bs, HIDDEN), self._randn(bs, HIDDEN)
        gamma = (t.rand(HIDDEN, generator=self.g, device=dev) + 0.5).to(h)
        act, act_out = self._randn(bs, 2, INTER), t.empty((bs, INTER), dtype=h, device=dev)
        logits = (t.randn(bs, VOCAB, generator=self.g, device=dev) * 2.0)
        u = t.rand(bs, generator=self.g, device=dev)
        sc_i = t.empty((bs, 8, TOPK_K), dtype=t.int32, device=dev)
        sc_v = t.empty((bs, 8, TOPK_K), device=dev)
        top_i, top_v = t.empty((bs, TOPK_K), dtype=t.int32, device=dev), t.empty((bs, TOPK_K), device=dev)
        picked = t.empty(bs, dtype=t.int32, device=dev)

        def step():
            o.launchRMSNorm(x, res, gamma, EPS)
            o.launchFusedAddBiasResidualRMSNorm(res, x, None, gamma, EPS)
            o.launchAct(act, act_out)
            o.launchTopKforBeamSearch(logits, sc_i, sc_v, top_i, top_v, 0, u, 1.0, picked)

        def timed(fn):
            for _ in range(3):
                fn()
            t.cuda.synchronize()
            s, e = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record()
            t.cuda.synchronize()
            return s.elapsed_time(e) / iters * 1e3

        eager_us = timed(step)
        graph, side = t.cuda.CUDAGraph(), t.cuda.Stream(dev)
        with t.cuda.stream(side):
            with t.cuda.graph(graph, stream=side):
                step()
        graph_us = timed(graph.replay)
        return {"eager_us": round(eager_us, 2), "graph_us": round(graph_us, 2), "launches_per_step": 4,
                "workload": f"{bs} sequences: RMSNorm, residual+RMSNorm [{bs}, {HIDDEN}], SiLU*up [{bs}, {INTER}], "
                            f"top-K({TOPK_K})+sampling [{bs}, {VOCAB}]"}

    def measure(self, steps: int = 20, warmup: int = 3) -> dict:
        peak, _ = measured_peak_gbs()
        out = {}
        for name in NEXT_KERNELS:
            ms, nbytes, workload = self.time_one(name, steps, warmup)
            gbs = nbytes / (ms * 1e-3) / 1e9
            out[name] = {"ms": round(ms, 5), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                         "bytes": nbytes, "workload": workload}
            self.torch.cuda.empty_cache()
        out["decode_small_kernels"] = self.decode_small_kernels()
        return out


class HostDrivenChain:
    """The same chain for a caller whose data lives in host memory: every step copies the step's
    inputs from pinned host buffers to the GPU, runs the kernels and copies every output back.

    The three phases of a step run on three streams (copy in, kernels, copy out) and consecutive
    steps alternate between two sets of device buffers, so step i's copy out and step i+1's copy
    in use the two directions of the PCIe link at the same time.  Every step still moves all of its
    inputs and outputs; events order the phases of a step and the reuse of a buffer set."""

    def __init__(self, chains):
        torch = chains[0].torch
        self.torch, self.chains = torch, chains
        dev = chains[0].dev
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.sets = []
        for c in chains:
            inputs = [c.ids, c.qkv, c.qk, c.attn_out, c.act_in, c.logits[0], c.u]
            outputs = [c.x, c.res, c.q, c.k, c.v, c.score, c.attn_out, c.act_out, c.top_i, c.top_v, c.picked]
            self.sets.append({
                "chain": c, "inputs": inputs, "outputs": outputs,
                "h_in": [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in inputs],
                "h_out": [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outputs],
                "in_ready": torch.cuda.Event(), "ran": torch.cuda.Event(), "out_done": torch.cuda.Event(),
            })
        first = self.sets[0]
        self.h2d = sum(t.numel() * t.element_size() for t in first["inputs"])
        self.d2h = sum(t.numel() * t.element_size() for t in first["outputs"])
        self.n = 0

    def begin(self) -> None:
        """The three streams start after everything already queued on the current stream."""
        cur = self.torch.cuda.current_stream()
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_stream(cur)
        for b in self.sets:
            b["out_done"].record(self.s_out)

    def step(self) -> None:
        torch, b = self.torch, self.sets[self.n % len(self.sets)]
        self.n += 1
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(b["out_done"])  # the previous user of this buffer set has been read out
            for h, d in zip(b["h_in"], b["inputs"]):
                d.copy_(h, non_blocking=True)
            b["in_ready"].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(b["in_ready"])
            b["chain"].step()
            b["ran"].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(b["ran"])
            for h, d in zip(b["h_out"], b["outputs"]):
                h.copy_(d, non_blocking=True)
            b["out_done"].record(self.s_out)

    def end(self) -> None:
        """The current stream continues after the three streams have drained."""
        cur = self.torch.cuda.current_stream()
        for st in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(st)


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the layer kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner on stdout at VERSION/INFO level; stdout carries the one JSON line.
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tokens = args.tokens
    chain = GpuChain(tokens, device, seed=1000 + rank)
    for _ in range(max(3, args.warmup)):
        chain.step()
    barrier()

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(9)] for _ in range(K)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        for i in range(K):
            chain.step(ev[i])
        barrier()
    total_ms = ev[0][0].elapsed_time(ev[-1][8])
    per_kernel_ms = [sum(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(K)) / K for j in range(8)]
    t = torch.tensor([total_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / K

    # end to end from host buffers, smaller batch (rows/s is size-normalised)
    e2e_chains = [GpuChain(args.e2e_tokens, device, seed=2000 + 10 * rank + i, topk_buffers=1) for i in range(2)]
    hd = HostDrivenChain(e2e_chains)
    e2e_steps = max(3, min(K, args.e2e_steps))
    hd.begin()
    for _ in range(3):
        hd.step()
    hd.end()
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    hd.begin()
    for _ in range(e2e_steps):
        hd.step()
    hd.end()
    e.record()
    barrier()
    t2 = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(t2.item()) / e2e_steps

    # The path's one real exchange, timed on its own when there are ranks to exchange with: top-K
    # over logits whose vocabulary axis is split across the ranks (local top-K with global ids, one
    # NCCL all-gather of the candidate lists, merge + sampling on every rank).
    sharded_topk = None
    if world > 1:
        from inferspore_b200.sharding import vocab_shard, vocab_sharded_topk

        shard = vocab_shard(VOCAB, world, rank)
        g = torch.Generator(device=device)
        g.manual_seed(4000)  # the same logits on every rank; each keeps its own columns
        full = torch.randn(TOPK_ROWS, VOCAB, generator=g, device=device) * 2.0
        local = full[:, shard.start:shard.stop].contiguous()
        uni = torch.rand(TOPK_ROWS, generator=g, device=device)
        for _ in range(3):
            vocab_sharded_topk(local, shard, TOPK_K, uniform=uni)
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(20):
            vocab_sharded_topk(local, shard, TOPK_K, uniform=uni)
        e.record()
        barrier()
        t3 = torch.tensor([s.elapsed_time(e) / 20], dtype=torch.float64, device=device)
        dist.all_reduce(t3, op=dist.ReduceOp.MAX)
        sharded_topk = {"ms": round(float(t3.item()), 4), "rows": TOPK_ROWS, "vocab_per_rank": shard.size,
                        "gathered_bytes_per_rank": TOPK_ROWS * TOPK_K * 8 * world}

    from inferspore_b200 import capi

    status = capi.device_status(clear=True)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return {}

    peak, peak_kind = measured_peak_gbs()
    bytes_per = algorithmic_bytes(tokens, TOPK_ROWS)
    rows_per = {k: (TOPK_ROWS if k == "topk_sampling" else tokens) for k in KERNELS}
    kernels = {}
    for name, ms in zip(KERNELS, per_kernel_ms):
        gbs = bytes_per[name] / (ms * 1e-3) / 1e9
        kernels[name] = {"ms": round(ms, 5), "rows_per_s": round(rows_per[name] / (ms * 1e-3), 1),
                         "gbs": round(gbs, 1), "frac_of_8TBs": round(gbs / NOMINAL_HBM_GBS, 4),
                         "frac_of_peak": round(gbs / peak, 4), "bytes": bytes_per[name]}
    dom = "silu_mul"
    out = {
        "metric": "rows/s through the fused layer-kernel chain (per-kernel GB/s in `kernels`)",
        "value": round(world * tokens / (ms_per_step * 1e-3), 1),
        "unit": "rows/s",
        "n_gpus": world,
        "steps": K,
        "warmup": max(3, args.warmup),
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"Llama-2-7B prefill layer-kernel chain, {tokens} tokens ({tokens // SEQ} x {SEQ}) per GPU "
                               f"+ top-K(50)+sampling over [{TOPK_ROWS}, {VOCAB}] fp32 logits",
                   "tokens_per_gpu": tokens, "l2": "inputs larger than L2 (top-K rotates 5 logits buffers)",
                   "sharding": f"token axis, {world} shard(s), no collective"},
        "gbs": round(world * sum(bytes_per.values()) / (ms_per_step * 1e-3) / 1e9, 1),
        "kernels": kernels,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": kernels[dom]["gbs"], "peak": peak, "unit": "GB/s",
                     "frac": round(kernels[dom]["gbs"] / peak, 4), "peak_kind": f"{peak_kind} copy bandwidth",
                     "traffic": args.traffic if args.traffic is not None
                     else round(NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_per[dom])},
        "clocks": clocks.summary(),
        "e2e": {"value": round(world * args.e2e_tokens / (e2e_ms_per_step * 1e-3), 1), "unit": "rows/s",
                "h2d_bytes_per_step": hd.h2d, "d2h_bytes_per_step": hd.d2h, "rows_per_step": args.e2e_tokens,
                "steps": e2e_steps, "ms_per_step": round(e2e_ms_per_step, 3)},
        "gpu_launches": K * LAUNCHES_PER_STEP,
        "device_status": status,
    }
    if sharded_topk is not None:
        out["vocab_sharded_topk"] = sharded_topk
    if world == 1 and not args.no_next_rows:
        del chain, e2e_chains, hd
        torch.cuda.empty_cache()
        out["next_rows"] = NextRows(tokens, device).measure()
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        rps, dt, cpu = time_cpu_chain(args.cpu_tokens, threads, steps=3, warmup=1, budget_s=40.0)
        out["cpu_baseline"] = {"value": round(rps, 1), "unit": "rows/s", "cores": threads, "kind": cpu.kind,
                               "sample": cpu.describe(), "s_per_step": round(dt, 3)}
    return out


def run_only(args) -> dict:
    """One kernel of the chain alone (for profiler captures on a small case): W warm-up launches,
    K timed launches, one JSON line with its time and algorithmic GB/s."""
    import torch

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    if args.only in NEXT_KERNELS:
        ms, nbytes, workload = NextRows(args.tokens, device, decode_batch=max(1, args.tokens // 1024)).time_one(
            args.only, args.steps, args.warmup)
        peak, kind = measured_peak_gbs()
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"kernel": args.only, "workload": workload, "ms": round(ms, 5), "bytes": nbytes, "gbs": round(gbs, 1),
                "frac_of_peak": round(gbs / peak, 4), "peak": peak, "peak_kind": kind, "steps": args.steps}
    chain = GpuChain(args.tokens, device, seed=1000)
    launch = dict(chain.launchers())[args.only]
    for _ in range(args.warmup):
        launch()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        launch()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    nbytes = algorithmic_bytes(args.tokens, TOPK_ROWS)[args.only]
    peak, kind = measured_peak_gbs()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"kernel": args.only, "tokens": args.tokens, "ms": round(ms, 5), "bytes": nbytes, "gbs": round(gbs, 1),
            "frac_of_peak": round(gbs / peak, 4), "peak": peak, "peak_kind": kind, "steps": args.steps}


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    threads = os.cpu_count() or 1
    rps, dt, cpu = time_cpu_chain(args.cpu_tokens, threads, steps=args.steps, warmup=args.warmup, budget_s=200.0)
    return {
        "impl": "reference",
        "metric": "rows/s through the fused layer-kernel chain (per-kernel GB/s in `kernels`)",
        "value": round(rps, 1), "unit": "rows/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "Llama-2-7B prefill layer-kernel chain on the host cores, bounded sample: " + cpu.describe()},
        "cpu_baseline": {"value": round(rps, 1), "unit": "rows/s", "cores": threads, "kind": cpu.kind,
                         "sample": cpu.describe()},
        "e2e": {"value": round(rps, 1), "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--tokens", type=int, default=65536, help="tokens per GPU per step (multiple of 512)")
    ap.add_argument("--e2e-tokens", type=int, default=8192, help="tokens per step of the host-driven leg")
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--cpu-tokens", type=int, default=4096, help="tokens per step of the CPU chain sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-next-rows", action="store_true",
                    help="skip the separately timed kernels either side of the chain (`next_rows`)")
    ap.add_argument("--only", choices=KERNELS + NEXT_KERNELS, default=None,
                    help="run one kernel of the chain alone at --tokens (small cases for profiler captures)")
    ap.add_argument("--traffic", type=float, default=None,
                    help="override: DRAM bytes per launch of the roofline kernel from a fresh ncu capture")
    args = ap.parse_args()
    if args.tokens % SEQ or args.e2e_tokens % SEQ or args.tokens <= 0:
        ap.error("--tokens and --e2e-tokens must be positive multiples of 512")
    # stdout carries exactly one JSON line: anything a library prints there during the run (NCCL's
    # version banner, for one) is sent to stderr instead, and the line is written to the real stdout.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        if args.only:
            out = run_only(args)
        else:
            out = run_reference(args) if args.impl == "reference" else run_ours(args)
        sys.stdout.flush()
    finally:
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    if out:
        print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
