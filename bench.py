#!/usr/bin/env python
"""Benchmark of the fused layer-kernel chain on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the per-layer fused kernels over one batch of synthetic
Llama-2-7B-shaped input (fp16 activations, seeded): embedding gather ->
plain RMSNorm -> QKV bias+RoPE+head transpose -> KV-cache concat -> scale+mask+
softmax -> residual add+RMSNorm -> SiLU(gate)*up -> top-K(50)+sampling.  The
batch is the 65,536-token sweep (128 sequences of 512) plus 256 rows of logits;
with N GPUs it is split along the token axis in whole sequences, 65,536 / N
tokens and 256 / N logits rows per rank, with no data-path collective, so
scaling is strong: total work is fixed as N grows.

Rank 0 prints ONE JSON line.  `value` is rows (tokens) per second of the whole
job through the chain with inputs resident in HBM (the steps replayed from a
CUDA graph; `--no-graph` launches them one by one, `--pdl` adds programmatic
dependent launch); `eager` is the same K steps launched one by one with CUDA events
around every kernel, which gives `kernels` (rows/s and algorithmic GB/s per
kernel) and `roofline` (SiLU*up, the kernel that moves the most bytes); `e2e`
is the chain driven from pinned host buffers with the host<->device copies
inside the timed region; `weak` (N > 1) is the per-GPU-65,536-token figure;
`vocab_sharded_topk` (N > 1) times the path's one real exchange and checks it
against the unsharded kernel bit for bit; `configs` (N = 1) times BASELINE's
configurations 1-4 as stated; `cpu_baseline` (N = 1) is the reference's CPU
code / the oracle port timed on the host cores on a bounded sample.

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
TOTAL_TOKENS = 65536
# DRAM traffic of the roofline kernel (SiLU*up): dram__bytes_read.sum + dram__bytes_write.sum of one
# launch at 16,384 tokens from an ncu capture of the current kernel (721.4 + 314.0 MB) over that
# launch's algorithmic bytes (1,082.1 MB).  The kernel is a flat streaming pass, so traffic grows in
# proportion to the rows; a full-size launch is scaled by it.  --traffic overrides it with a fresh
# capture's figure.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1035.4 / 1082.13


def launches_per_step(topk_rows: int) -> int:
    """Kernels of this library per chain step: one per op (top-K runs one slice per row at this
    vocabulary, so its merge kernel is not launched)."""
    del topk_rows
    return 8


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
    def __init__(self, tokens: int, device, seed: int, topk_buffers: int = 5, topk_rows: int = 256):
        import torch

        from inferspore_b200 import ops

        self.torch, self.ops, self.dev, self.tokens, self.topk_rows = torch, ops, device, tokens, topk_rows
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
        self.logits = [randn(topk_rows, VOCAB, dtype=torch.float32, scale=2.0) for _ in range(topk_buffers)]
        self.u = torch.rand(topk_rows, generator=g, device=device)
        self.sc_i = torch.empty((topk_rows, 8, TOPK_K), dtype=torch.int32, device=device)
        self.sc_v = torch.empty((topk_rows, 8, TOPK_K), dtype=torch.float32, device=device)
        self.top_i = torch.empty((topk_rows, TOPK_K), dtype=torch.int32, device=device)
        self.top_v = torch.empty((topk_rows, TOPK_K), dtype=torch.float32, device=device)
        self.picked = torch.empty(topk_rows, dtype=torch.int32, device=device)
        self.scale = 1.0 / float(np.sqrt(HEAD_SIZE))
        self.n = 0
        self._launchers = None

    def launchers(self):
        """The chain as (kernel name, launch closure) pairs, in order.  Every launch is validated once
        here (ops.prepare) and is a bare C-ABI call afterwards: at 8,192 tokens per GPU a kernel takes
        20-90 us, which per-call argument checks in Python would rival."""
        if self._launchers is None:
            o = self.ops
            topk = [o.prepare(o.launchTopKforBeamSearch, lg, self.sc_i, self.sc_v, self.top_i, self.top_v, 0, self.u,
                              1.0, self.picked) for lg in self.logits]

            def topk_next():
                topk[self.n % len(topk)]()
                self.n += 1

            self._launchers = [
                ("input_embedding", o.prepare(o.launchInputEmbedding, self.ids, self.x, self.table)),
                ("rmsnorm", o.prepare(o.launchRMSNorm, self.x, self.res, self.gamma, EPS)),
                ("qkv_bias_rope_transpose", o.prepare(o.launchAddFusedQKVBiasTransposeAndRoPE, self.q, self.k, self.v,
                                                      self.qkv, self.bias, self.pad, self.hist, self.inlen, ROT_DIM, ROT_BASE)),
                ("concat_kv", o.prepare(o.launchConcatKVCache, self.k, self.v, 0, self.inlen, self.hist, self.k_cache,
                                        self.v_cache)),
                ("scale_mask_softmax", o.prepare(o.launchScaleMaskAndSoftmax, self.qk, self.mask, self.score, self.scale)),
                ("add_residual_rmsnorm", o.prepare(o.launchFusedAddBiasResidualRMSNorm, self.res, self.attn_out, None,
                                                   self.gamma, EPS)),
                ("silu_mul", o.prepare(o.launchAct, self.act_in, self.act_out)),
                ("topk_sampling", topk_next),
            ]
        return self._launchers

    def step(self, events=None) -> None:
        """Launches the chain on the current stream; `events` (len 9) are recorded around each kernel."""
        for i, (_, launch) in enumerate(self.launchers()):
            if events is not None:
                events[i].record()
            launch()
        if events is not None:
            events[8].record()

    def capture(self, steps: int, pdl: bool):
        """`steps` chain steps captured into one CUDA graph (top-K walks through its logits buffers as
        in the eager loop).  With `pdl` the launches carry the programmatic-dependent-launch attribute,
        so inside the graph one kernel's ramp-up overlaps the tail of the one before."""
        return capture_graph(self.torch, self.ops, self.dev, lambda: [self.step() for _ in range(steps)], pdl)


def capture_graph(torch, ops, device, body, pdl: bool):
    """Runs `body` under stream capture (every entry point must have run once before) and returns the graph."""
    ops.set_programmatic_launch(pdl)
    try:
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream(device)
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                body()
    finally:
        ops.set_programmatic_launch(False)
    torch.cuda.current_stream(device).wait_stream(side)
    return graph


def timed_ms(torch, fn, iters: int) -> float:
    """Mean milliseconds of `fn` over `iters` back-to-back calls (CUDA events on the current stream)."""
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


NEXT_KERNELS = ["build_causal_mask", "scale_causal_softmax", "scale_mask_softmax_len777", "scale_mask_softmax_len16384",
                "cal_padding_offset", "transpose_remove_padding", "repeat_kv", "decoder_masked_mha",
                "decoder_masked_mha_gqa8", "decoder_masked_mha_32q4kv", "decoder_masked_mha_gqa8_step8192",
                "topk_sampling_4096rows"]


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
            # write-only and smaller than L2: three masks in turn, so that every launch's lines leave for HBM
            masks = [t.empty((B, SEQ, SEQ), dtype=h, device=dev) for _ in range(3)]
            ql = self._i32([SEQ] * B)
            turn = [0]

            def build():
                o.launchBuildCausalMasks(masks[turn[0] % 3], ql, ql)
                turn[0] += 1

            return build, masks[0].numel() * 2, f"mask [{B}, {SEQ}, {SEQ}] f16, three outputs in turn"
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
        if name == "scale_mask_softmax_len16384":
            # few, very long rows: 8,192 rows of 16,384 (a long-context prefill chunk of 128 queries)
            bs, q, n = 2, 128, 16384
            qk = self._randn(bs, HEADS, q, n, scale=3.0)
            out = t.empty_like(qk)
            mask = t.ones((bs, q, n), dtype=h, device=dev)
            mask[:, :, n - 100:] = 0
            return ((lambda: o.launchScaleMaskAndSoftmax(qk, mask, out, 1.0 / float(np.sqrt(HEAD_SIZE)))),
                    2 * qk.numel() * 2 + mask.numel() * 2, f"qk [{bs}, {HEADS}, {q}, {n}] f16 + mask [{bs}, {q}, {n}]")
        if name == "topk_sampling_4096rows":
            rows = 4096
            logits = [(t.randn(rows, VOCAB, generator=self.g, device=dev) * 2.0) for _ in range(2)]
            u = t.rand(rows, generator=self.g, device=dev)
            sc_i = t.empty((rows, 8, TOPK_K), dtype=t.int32, device=dev)
            sc_v = t.empty((rows, 8, TOPK_K), device=dev)
            top_i, top_v = t.empty((rows, TOPK_K), dtype=t.int32, device=dev), t.empty((rows, TOPK_K), device=dev)
            picked = t.empty(rows, dtype=t.int32, device=dev)
            state = {"n": 0}

            def launch():
                o.launchTopKforBeamSearch(logits[state["n"] & 1], sc_i, sc_v, top_i, top_v, 0, u, 1.0, picked)
                state["n"] += 1
            return launch, rows * VOCAB * 4 + rows * TOPK_K * 8 + 2 * rows * 4, f"logits [{rows}, {VOCAB}] f32, K = {TOPK_K}, + sampling"
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
        if name.startswith("decoder_masked_mha"):
            # the model's own 32/32 heads; 64 q heads on 8 kv heads (eight q heads share each cache row), also
            # at 16 sequences x step 8192; 32 q heads on 4 kv heads
            heads, kvh = {"decoder_masked_mha": (HEADS, KV_HEADS), "decoder_masked_mha_32q4kv": (32, 4)}.get(name, (64, 8))
            bs, ctx = self.decode_batch, self.context
            if name == "decoder_masked_mha_gqa8_step8192":
                bs, ctx = max(1, self.decode_batch // 4), 2 * self.context
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
            if ms < 0.04:  # a launch from Python costs as much as such a kernel: also replayed from a CUDA graph
                launch, _, _ = self.prepare(name)
                launch()
                graph = capture_graph(self.torch, self.ops, self.dev, lambda: [launch() for _ in range(steps)], False)
                graph.replay()
                gms = timed_ms(self.torch, graph.replay, 3) / steps
                out[name].update({"graph_ms": round(gms, 5), "graph_frac_of_peak": round(nbytes / (gms * 1e-3) / 1e9 / peak, 4)})
                del graph
            self.torch.cuda.empty_cache()
        out["decode_small_kernels"] = self.decode_small_kernels()
        return out


class StatedConfigs:
    """BASELINE configurations 1-4 exactly as stated (configuration 5 is the headline workload itself).
    Kernels whose tensors fit in L2 are timed one launch at a time with a buffer larger than L2
    written and then read between launches (the read pushes the dirty lines of the write out of L2
    before the timed launch starts, whose DRAM bandwidth they would otherwise share); configuration 1 (a 4 us kernel) instead walks through enough input
    sets to exceed L2, launched one by one and replayed from a CUDA graph."""

    L2_FLUSH_BYTES = 256 << 20

    def __init__(self, device):
        import torch

        from inferspore_b200 import ops

        self.torch, self.ops, self.dev = torch, ops, device
        self.g = torch.Generator(device=device)
        self.g.manual_seed(99)
        self.flush = torch.empty(self.L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
        self.flush_sink = torch.zeros(1, dtype=torch.int64, device=device)
        self.peak, _ = measured_peak_gbs()

    def _flushed_us(self, launch, iters: int = 10) -> float:
        t = self.torch
        for _ in range(3):
            launch()
        total = 0.0
        for _ in range(iters):
            self.flush.zero_()
            t.sum(self.flush.view(t.int64), dim=0, keepdim=True, out=self.flush_sink)
            s, e = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            s.record()
            launch()
            e.record()
            e.synchronize()
            total += s.elapsed_time(e)
        return total / iters * 1e3

    def _entry(self, us: float, nbytes: int, workload: str, **extra) -> dict:
        gbs = nbytes / (us * 1e-6) / 1e9
        return {"us": round(us, 2), "bytes": nbytes, "gbs": round(gbs, 1), "frac_of_peak": round(gbs / self.peak, 4),
                "frac_of_8TBs": round(gbs / NOMINAL_HBM_GBS, 4), "workload": workload, **extra}

    def config1(self) -> dict:
        t, o, dev = self.torch, self.ops, self.dev
        rows, sets = 64, 72  # 72 x (x + residual) of 1 MiB each = 151 MB > L2
        xs = [t.randn(rows, HIDDEN, generator=self.g, device=dev) for _ in range(sets)]
        rs = [t.randn(rows, HIDDEN, generator=self.g, device=dev) for _ in range(sets)]
        gamma = t.rand(HIDDEN, generator=self.g, device=dev) + 0.5

        def sweep():
            for x, r in zip(xs, rs):
                o.launchFusedAddBiasResidualRMSNorm(r, x, None, gamma, EPS)

        sweep()
        eager_us = timed_ms(t, sweep, 5) / sets * 1e3
        graph = capture_graph(t, o, dev, sweep, False)
        graph.replay()
        graph_us = timed_ms(t, graph.replay, 5) / sets * 1e3
        nbytes = 4 * rows * HIDDEN * 4 + HIDDEN * 4
        return self._entry(graph_us, nbytes, f"residual add + RMSNorm fp32 [{rows}, {HIDDEN}], {sets} input sets in turn "
                           "(past L2), per launch, replayed from a CUDA graph", eager_us=round(eager_us, 2))

    def config2(self) -> dict:
        t, o, dev = self.torch, self.ops, self.dev
        chains = [GpuChain(4096, dev, seed=11 + i, topk_buffers=1, topk_rows=16) for i in range(3)]
        las = [dict(c.launchers()) for c in chains]
        by = algorithmic_bytes(4096, 16)
        out = {}
        for k in ("input_embedding", "qkv_bias_rope_transpose"):
            us = self._flushed_us(las[0][k])

            def sweep():  # three sets of tensors in turn (200-600 MB): past L2 without a flush
                for la in las:
                    la[k]()

            sweep()
            graph = capture_graph(t, o, dev, lambda: [sweep() for _ in range(4)], False)
            graph.replay()
            graph_us = timed_ms(t, graph.replay, 5) / (4 * len(las)) * 1e3
            out[k] = self._entry(us, by[k], "fp16, 4096 tokens (8 x 512), L2 flushed between launches; graph_us: three "
                                 "sets of tensors in turn replayed from a CUDA graph", graph_us=round(graph_us, 2))
            del graph
        return out

    def config3(self) -> dict:
        chain = GpuChain(16384, self.dev, seed=12, topk_buffers=1, topk_rows=64)
        la = dict(chain.launchers())
        by = algorithmic_bytes(16384, 64)
        return {k: self._entry(self._flushed_us(la[k]), by[k], f"fp16, 16384 tokens, L2 flushed between launches")
                for k in ("add_residual_rmsnorm", "silu_mul")}

    def config4(self) -> dict:
        t, o, dev, h = self.torch, self.ops, self.dev, self.torch.float16
        bs, max_seq = 64, 4096
        per_layer = 2 * bs * KV_HEADS * max_seq * HEAD_SIZE * 2
        free, _ = t.cuda.mem_get_info(dev)
        layers = int(max(1, min(32, (free * 3 // 4) // per_layer)))
        kc = t.empty((layers, bs, KV_HEADS, max_seq, HEAD_SIZE), dtype=h, device=dev)
        vc = t.empty_like(kc)
        k = (t.randn(bs, KV_HEADS, 1, HEAD_SIZE, generator=self.g, device=dev)).to(h)
        v = (t.randn(bs, KV_HEADS, 1, HEAD_SIZE, generator=self.g, device=dev)).to(h)
        steps = t.randint(1, max_seq, (bs,), generator=self.g, device=dev, dtype=t.int32)
        cur = t.ones(bs, dtype=t.int32, device=dev)

        def all_layers():
            for layer in range(layers):
                o.launchConcatKVCache(k, v, layer, cur, steps, kc, vc)

        all_layers()
        eager_us = timed_ms(t, all_layers, 5) / layers * 1e3
        graph = capture_graph(t, o, dev, all_layers, False)
        graph.replay()
        graph_us = timed_ms(t, graph.replay, 5) / layers * 1e3
        concat_bytes = 2 * 2 * bs * KV_HEADS * HEAD_SIZE * 2 + 2 * bs * 4
        out = {"concat_kv": self._entry(graph_us, concat_bytes, f"k, v [{bs}, {KV_HEADS}, 1, {HEAD_SIZE}] f16 into caches "
                                        f"[{layers}, {bs}, {KV_HEADS}, {max_seq}, {HEAD_SIZE}] at steps ~U[1, {max_seq}), per layer, "
                                        f"{layers} layers in turn replayed from a CUDA graph", eager_us=round(eager_us, 2),
                                        layers=layers)}
        del kc, vc, graph
        t.cuda.empty_cache()
        qk = (t.randn(bs, HEADS, 1, max_seq, generator=self.g, device=dev) * 3.0).to(h)
        score = t.empty_like(qk)
        mask = (t.arange(max_seq, device=dev)[None, None, :] < steps[:, None, None]).to(h).contiguous()
        us = self._flushed_us(lambda: o.launchScaleMaskAndSoftmax(qk, mask, score, 1.0 / float(np.sqrt(HEAD_SIZE))))
        # the same launch without the host in the loop: six input sets in turn (208 MB), from a CUDA graph
        sets = [(qk, score)] + [((t.randn(bs, HEADS, 1, max_seq, generator=self.g, device=dev) * 3.0).to(h),
                                 t.empty_like(qk)) for _ in range(5)]

        def sweep():
            for a, b in sets:
                o.launchScaleMaskAndSoftmax(a, mask, b, 1.0 / float(np.sqrt(HEAD_SIZE)))

        sweep()
        graph = capture_graph(t, o, dev, sweep, False)
        graph.replay()
        graph_us = timed_ms(t, graph.replay, 5) / len(sets) * 1e3
        out["scale_mask_softmax"] = self._entry(us, 2 * qk.numel() * 2 + mask.numel() * 2,
                                                f"qk [{bs}, {HEADS}, 1, {max_seq}] f16, valid length = step, L2 flushed between launches; "
                                                "graph_us: six input sets in turn replayed from a CUDA graph", graph_us=round(graph_us, 2))
        return out

    def measure(self) -> dict:
        out = {}
        for name in ("config1", "config2", "config3", "config4"):
            out[name] = getattr(self, name)()
            self.torch.cuda.empty_cache()
        return out


def small_shard_table(device, use_pdl: bool, tokens: int = 8192, topk_rows: int = 32, steps: int = 20) -> dict:
    """The chain at the per-GPU size of the 8-way split, on this one GPU: per-kernel times launched
    one by one, and the step time replayed from a CUDA graph with and without programmatic
    dependent launch.  What limits the 1 -> 8 curve is here, not in any collective."""
    import torch

    chain = GpuChain(tokens, device, seed=5000, topk_rows=topk_rows)
    peak, _ = measured_peak_gbs()
    for _ in range(3):
        chain.step()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(9)] for _ in range(steps)]
    torch.cuda.synchronize()
    for i in range(steps):
        chain.step(ev[i])
    torch.cuda.synchronize()
    eager_ms = ev[0][0].elapsed_time(ev[-1][8]) / steps
    by = algorithmic_bytes(tokens, topk_rows)
    kernels = {}
    for j, name in enumerate(KERNELS):
        ms = sum(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(steps)) / steps
        gbs = by[name] / (ms * 1e-3) / 1e9
        kernels[name] = {"us": round(ms * 1e3, 2), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4)}
    out = {"tokens": tokens, "topk_rows": topk_rows, "eager_us_per_step": round(eager_ms * 1e3, 1), "kernels": kernels,
           "ideal_us_at_peak": round(sum(by.values()) / peak / 1e3, 1)}
    for key, pdl in (("graph_us_per_step", False), ("graph_pdl_us_per_step", True)):
        graph = chain.capture(steps, pdl)
        graph.replay()
        out[key] = round(timed_ms(torch, graph.replay, 3) / steps * 1e3, 1)
        del graph
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


def host_memory_available() -> int:
    """Bytes of host memory this process may still take (the smaller of the machine's and the
    cgroup's head-room)."""
    avail = 1 << 62
    try:
        import psutil

        avail = psutil.virtual_memory().available
    except Exception:
        pass
    for limit, used in (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
                        ("/sys/fs/cgroup/memory/memory.limit_in_bytes", "/sys/fs/cgroup/memory/memory.usage_in_bytes")):
        try:
            lim = Path(limit).read_text().strip()
            if lim != "max":
                avail = min(avail, int(lim) - int(Path(used).read_text().strip()))
        except Exception:
            pass
    return avail


def bind_to_gpu_numa_node(device_index: int) -> str:
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, before any pinned host
    buffer exists: pinned pages are placed where the allocating thread runs, and copies from the
    other socket's memory cross the inter-socket link, which all ranks of a node then share.
    Best effort: returns what was done (the bench line carries it)."""
    try:
        import torch

        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        pci = f"{dom:04x}:{bus:02x}:{dev:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{pci}/numa_node").read_text().strip())
        if node < 0:
            return f"unchanged (GPU {pci} reports no NUMA node)"
        cpus = set()
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return f"unchanged (no allowed CPU on NUMA node {node} of GPU {pci})"
        os.sched_setaffinity(0, allowed)
        return f"NUMA node {node} of GPU {pci} ({len(allowed)} CPUs)"
    except Exception as exc:  # no sysfs, no such attribute, not permitted ...
        return f"unchanged ({type(exc).__name__})"


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from inferspore_b200 import capi, ops
    from inferspore_b200.sharding import shard_range, shard_sequences

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the layer kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    all_cpus = os.sched_getaffinity(0)
    host_affinity = bind_to_gpu_numa_node(local_rank)
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

    def max_over_ranks(ms: float) -> float:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # This rank's share of the job: whole sequences of the 65,536-token batch, and rows of the logits.
    if args.tokens is not None:  # per-GPU override (small cases for development and profiling)
        tokens, total_tokens = args.tokens, args.tokens * world
        topk_rows = args.topk_rows if args.topk_rows is not None else max(1, TOPK_ROWS * tokens // TOTAL_TOKENS)
        total_topk_rows = topk_rows * world
    else:
        total_tokens, total_topk_rows = TOTAL_TOKENS, TOPK_ROWS
        _, tok = shard_sequences(total_tokens // SEQ, SEQ, world, rank)
        tokens, topk_rows = tok.size, shard_range(total_topk_rows, world, rank).size
    use_graph, use_pdl = not args.no_graph, args.pdl
    K, W = args.steps, max(3, args.warmup)

    chain = GpuChain(tokens, device, seed=1000 + rank, topk_rows=topk_rows)
    for _ in range(W):
        chain.step()
    barrier()

    # Timed region 1 (`value`): exactly K steps, one graph launch (or K eager steps with --no-graph).
    graph = None
    if use_graph:
        try:
            graph = chain.capture(K, use_pdl)
            graph.replay()  # one more warm-up pass, through the graph
        except Exception as exc:  # capture refused: fall back to plain launches and say so
            print(f"bench: graph capture failed ({exc}); timing plain launches", file=sys.stderr)
            graph = None
    if graph is None and use_pdl:
        ops.set_programmatic_launch(True)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        s.record()
        if graph is not None:
            graph.replay()
        else:
            for _ in range(K):
                chain.step()
        e.record()
        barrier()
    ops.set_programmatic_launch(False)
    ms_per_step = max_over_ranks(s.elapsed_time(e)) / K
    launch_mode = ("graph" if graph is not None else "eager") + ("+pdl" if use_pdl else "")

    # Timed region 2 (`eager`, `kernels`, `roofline`): the same K steps launched one by one, CUDA events
    # around every kernel.
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(9)] for _ in range(K)]
    barrier()
    for i in range(K):
        chain.step(ev[i])
    barrier()
    eager_ms_per_step = max_over_ranks(ev[0][0].elapsed_time(ev[-1][8])) / K
    per_kernel_ms = [sum(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(K)) / K for j in range(8)]
    del graph

    # Weak scaling beside the strong figure: every rank runs the whole 65,536-token batch.
    weak = None
    if world > 1 and args.tokens is None and not args.no_weak:
        wchain = GpuChain(TOTAL_TOKENS, device, seed=3000 + rank, topk_rows=TOPK_ROWS)
        wk = max(3, min(K, 10))
        for _ in range(3):
            wchain.step()
        wgraph = wchain.capture(wk, use_pdl) if use_graph else None
        if wgraph is not None:
            wgraph.replay()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        if wgraph is not None:
            wgraph.replay()
        else:
            for _ in range(wk):
                wchain.step()
        e.record()
        barrier()
        wms = max_over_ranks(s.elapsed_time(e)) / wk
        weak = {"value": round(world * TOTAL_TOKENS / (wms * 1e-3), 1), "unit": "rows/s", "ms_per_step": round(wms, 4),
                "tokens_per_gpu": TOTAL_TOKENS, "topk_rows_per_gpu": TOPK_ROWS, "steps": wk, "scaling": "weak"}
        del wchain, wgraph
        torch.cuda.empty_cache()

    # End to end from host buffers: this rank's share of the same batch, unless the host cannot pin
    # that much (two buffer sets of inputs and outputs); rows/s is size-normalised either way.
    e2e_tokens = args.e2e_tokens if args.e2e_tokens is not None else tokens
    per_token_pinned = 2 * (930 + 852) * (1 << 20) // 8192  # both directions, two buffer sets
    budget = host_memory_available() // (3 * max(1, world if args.e2e_tokens is None else 1))
    while e2e_tokens > SEQ and e2e_tokens * per_token_pinned > budget:
        e2e_tokens = max(SEQ, (e2e_tokens // 2) // SEQ * SEQ)
    e2e_topk = max(1, topk_rows * e2e_tokens // tokens)
    del chain
    torch.cuda.empty_cache()
    e2e_chains = [GpuChain(e2e_tokens, device, seed=2000 + 10 * rank + i, topk_buffers=1, topk_rows=e2e_topk) for i in range(2)]
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
    e2e_ms_per_step = max_over_ranks(s.elapsed_time(e)) / e2e_steps
    e2e = {"value": round(world * e2e_tokens / (e2e_ms_per_step * 1e-3), 1), "unit": "rows/s",
           "h2d_bytes_per_step": hd.h2d, "d2h_bytes_per_step": hd.d2h, "rows_per_step": e2e_tokens,
           "rows_per_step_all_gpus": world * e2e_tokens, "steps": e2e_steps, "ms_per_step": round(e2e_ms_per_step, 3)}
    del e2e_chains, hd
    os.sched_setaffinity(0, all_cpus)  # the CPU baseline below runs on every core again
    torch.cuda.empty_cache()

    sharded_topk = vocab_sharded_leg(torch, dist, ops, device, rank, world, barrier, max_over_ranks) if world > 1 else None

    status = capi.device_status(clear=True)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        if sharded_topk is not None and not sharded_topk["matches_unsharded"]:
            raise SystemExit(3)
        return {}

    peak, peak_kind = measured_peak_gbs()
    bytes_per = algorithmic_bytes(tokens, topk_rows)
    rows_per = {k: (topk_rows if k == "topk_sampling" else tokens) for k in KERNELS}
    kernels = {}
    for name, ms in zip(KERNELS, per_kernel_ms):
        gbs = bytes_per[name] / (ms * 1e-3) / 1e9
        kernels[name] = {"ms": round(ms, 5), "rows_per_s": round(rows_per[name] / (ms * 1e-3), 1),
                         "gbs": round(gbs, 1), "frac_of_8TBs": round(gbs / NOMINAL_HBM_GBS, 4),
                         "frac_of_peak": round(gbs / peak, 4), "bytes": bytes_per[name]}
    dom = "silu_mul"
    total_bytes = sum(algorithmic_bytes(total_tokens, total_topk_rows).values())
    out = {
        "metric": "rows/s through the fused layer-kernel chain (per-kernel GB/s in `kernels`)",
        "value": round(total_tokens / (ms_per_step * 1e-3), 1),
        "unit": "rows/s",
        "n_gpus": world,
        "steps": K,
        "warmup": W,
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"Llama-2-7B prefill layer-kernel chain over {total_tokens} tokens ({total_tokens // SEQ} x {SEQ}) "
                               f"+ top-K(50)+sampling over [{total_topk_rows}, {VOCAB}] fp32 logits, split over {world} GPU(s)",
                   "tokens_per_gpu": tokens, "topk_rows_per_gpu": topk_rows,
                   "l2": "inputs larger than L2 (2.4 GB of tensors per step even at 8,192 tokens per GPU; top-K rotates 5 "
                         "logits buffers)",
                   "sharding": f"token axis, whole sequences, {world} shard(s), no collective",
                   "launch": launch_mode, "host_affinity": host_affinity},
        "gbs": round(total_bytes / (ms_per_step * 1e-3) / 1e9, 1),
        "eager": {"ms_per_step": round(eager_ms_per_step, 4), "value": round(total_tokens / (eager_ms_per_step * 1e-3), 1),
                  "note": "the same K steps launched one by one with CUDA events around every kernel; source of `kernels` "
                          "and `roofline`"},
        "kernels": kernels,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": kernels[dom]["gbs"], "peak": peak, "unit": "GB/s",
                     "frac": round(kernels[dom]["gbs"] / peak, 4), "peak_kind": f"{peak_kind} copy bandwidth",
                     "traffic": args.traffic if args.traffic is not None
                     else round(NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_per[dom])},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": K * launches_per_step(topk_rows),
        "device_status": status,
    }
    if weak is not None:
        out["weak"] = weak
    if sharded_topk is not None:
        out["vocab_sharded_topk"] = sharded_topk
    if world == 1 and not args.no_next_rows:
        torch.cuda.empty_cache()
        out["next_rows"] = NextRows(total_tokens, device).measure()
        out["configs"] = StatedConfigs(device).measure()
        out["small_shard"] = small_shard_table(device, use_pdl)
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        rps, dt, cpu = time_cpu_chain(args.cpu_tokens, threads, steps=3, warmup=1, budget_s=40.0)
        out["cpu_baseline"] = {"value": round(rps, 1), "unit": "rows/s", "cores": threads, "kind": cpu.kind,
                               "sample": cpu.describe(), "s_per_step": round(dt, 3)}
    if sharded_topk is not None and not sharded_topk["matches_unsharded"]:
        print(json.dumps(out), file=sys.stderr)
        raise SystemExit(3)
    return out


def vocab_sharded_leg(torch, dist, ops, device, rank, world, barrier, max_over_ranks) -> dict:
    """The path's one real exchange, timed on its own and checked: top-K over logits whose vocabulary
    axis is split across the ranks (local top-K with global ids, one NCCL all-gather of the packed
    candidate records, merge + sampling on every rank, reading the gathered records in place).
    Outside the timed loops the unsharded kernel runs on the full logits and its ids, values and
    sampled ids must equal the sharded result bit for bit on every rank."""
    from inferspore_b200.sharding import VocabShardedTopK, vocab_shard

    shard = vocab_shard(VOCAB, world, rank)
    g = torch.Generator(device=device)
    g.manual_seed(4000)  # the same logits on every rank; each keeps its own columns
    full = torch.randn(TOPK_ROWS, VOCAB, generator=g, device=device) * 2.0
    full[:, ::97] = full[:, 5:6]  # equal values in different shards: the tie rule has to hold across ranks
    local = full[:, shard.start:shard.stop].contiguous()
    uni = torch.rand(TOPK_ROWS, generator=g, device=device)
    op = VocabShardedTopK(TOPK_ROWS, TOPK_K, torch.float32, device)
    iters = 20

    def whole():
        return op(local, shard, uni, 1.0)

    for _ in range(3):
        whole()
    barrier()
    total = max_over_ranks(timed_ms(torch, whole, iters))
    barrier()
    local_ms = max_over_ranks(timed_ms(torch, lambda: op.local(local, shard), iters))
    barrier()
    gather_ms = max_over_ranks(timed_ms(torch, op.exchange, iters))
    barrier()
    merge_ms = max_over_ranks(timed_ms(torch, lambda: op.merge(uni, 1.0), iters))
    barrier()

    # parity, outside the timed loops
    ids, vals, picked = whole()
    sc_i = torch.empty((TOPK_ROWS, 8, TOPK_K), dtype=torch.int32, device=device)
    sc_v = torch.empty((TOPK_ROWS, 8, TOPK_K), device=device)
    f_i = torch.empty((TOPK_ROWS, TOPK_K), dtype=torch.int32, device=device)
    f_v = torch.empty((TOPK_ROWS, TOPK_K), device=device)
    f_p = torch.empty(TOPK_ROWS, dtype=torch.int32, device=device)
    ops.launchTopKforBeamSearch(full, sc_i, sc_v, f_i, f_v, 0, uni, 1.0, f_p)
    torch.cuda.synchronize()
    same = bool(torch.equal(ids, f_i) and torch.equal(vals.view(torch.int32), f_v.view(torch.int32)) and torch.equal(picked, f_p))
    flag = torch.tensor([1 if same else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)

    # Last, the three steps replayed from one CUDA graph (NCCL collectives can be captured).  Every
    # rank replays only if every rank captured, so that no rank waits in the all-gather for one
    # that has nothing to replay.
    graph, graph_ms = None, None
    try:
        graph = capture_graph(torch, ops, device, whole, False)
    except Exception as exc:
        print(f"bench: capture of the sharded top-K failed on rank {rank} ({exc})", file=sys.stderr)
    captured = torch.tensor([0 if graph is None else 1], dtype=torch.int32, device=device)
    dist.all_reduce(captured, op=dist.ReduceOp.MIN)
    if captured.item() == 1:
        graph.replay()
        barrier()
        graph_ms = max_over_ranks(timed_ms(torch, graph.replay, iters))
        barrier()
        g_same = bool(torch.equal(op.out_i, f_i) and torch.equal(op.picked, f_p))
        flag2 = torch.tensor([1 if g_same else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag2, op=dist.ReduceOp.MIN)
        flag = torch.minimum(flag, flag2)
    del graph
    return {"ms": round(total, 4), "local_topk_us": round(local_ms * 1e3, 2), "allgather_us": round(gather_ms * 1e3, 2),
            "merge_us": round(merge_ms * 1e3, 2), "graph_us": None if graph_ms is None else round(graph_ms * 1e3, 2),
            "rows": TOPK_ROWS, "vocab_per_rank": shard.size, "record_bytes_per_rank": op.record_bytes,
            "gathered_bytes_per_rank": op.record_bytes * world, "matches_unsharded": bool(flag.item() == 1),
            "checked": "ids, value bits and sampled ids of every rank against launchTopKforBeamSearch on the full logits"}


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
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
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
    ap.add_argument("--tokens", type=int, default=None,
                    help="tokens per GPU per step (multiple of 512); default: 65536 split over the GPUs")
    ap.add_argument("--topk-rows", type=int, default=None, help="logits rows per GPU (default: 256 split over the GPUs)")
    ap.add_argument("--e2e-tokens", type=int, default=None,
                    help="tokens per GPU per step of the host-driven leg (default: this GPU's share of the batch, "
                         "halved until two pinned buffer sets fit the host)")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of from a CUDA graph")
    ap.add_argument("--pdl", action="store_true",
                    help="programmatic dependent launch in the timed steps (measured neutral inside a graph; off by default)")
    ap.add_argument("--no-weak", action="store_true", help="N > 1: skip the extra 65,536-tokens-per-GPU (weak scaling) leg")
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
    for v in (args.tokens, args.e2e_tokens):
        if v is not None and (v % SEQ or v <= 0):
            ap.error("--tokens and --e2e-tokens must be positive multiples of 512")
    if args.only and args.tokens is None:
        args.tokens = 16384
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
