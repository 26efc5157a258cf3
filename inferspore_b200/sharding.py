"""Token-axis and vocab-axis partitioning for multi-GPU runs (one process per GPU).

Every layer kernel is row-local, so the token/batch axis shards with no
data-path collective: each rank runs the same kernels on its own block of whole
sequences.  The one exchange on the path is optional: vocab-sharded top-K, where
each rank reduces its vocab slice to K candidates with GLOBAL ids, the
candidates are all-gathered (rows * K * 8 bytes per rank) and every rank merges
them with the same (value desc, index asc) order — bit-identical to the
unsharded kernel.  The gathered candidates sit in local HBM before the merge
kernel reads them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    start: int
    stop: int

    @property
    def size(self) -> int:
        return self.stop - self.start


def shard_range(total: int, world_size: int, rank: int) -> Shard:
    """Contiguous block of `total` units for `rank`: sizes differ by at most one,
    the first total % world_size ranks take the extra unit."""
    if world_size < 1 or not 0 <= rank < world_size or total < 0:
        raise ValueError(f"bad shard request total={total} world={world_size} rank={rank}")
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return Shard(start, start + base + (1 if rank < extra else 0))


def shard_sequences(batch: int, seq_len: int, world_size: int, rank: int) -> Tuple[Shard, Shard]:
    """Shards whole sequences (so [b, h, s, d] outputs and padding offsets stay rank-local).
    Returns (sequence range, token range) for packed, un-padded sequences of equal length."""
    seqs = shard_range(batch, world_size, rank)
    return seqs, Shard(seqs.start * seq_len, seqs.stop * seq_len)


def vocab_shard(vocab: int, world_size: int, rank: int, align: int = 8) -> Shard:
    """Column block of the logits for `rank`, boundaries rounded to `align` elements so every
    shard starts on a 16-byte boundary for both fp32 and fp16."""
    if vocab < 0 or align < 1:
        raise ValueError("bad vocab shard request")
    units = -(-vocab // align)
    u = shard_range(units, world_size, rank)
    return Shard(min(u.start * align, vocab), min(u.stop * align, vocab))


def gather_candidates(local_ids: torch.Tensor, local_vals: torch.Tensor,
                      group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gathers per-rank top-K lists [rows, K] into [rows, world, K] (rank-major lists per row).
    Works on CUDA tensors over NCCL and on CPU tensors over gloo."""
    if local_ids.shape != local_vals.shape or local_ids.dim() != 2:
        raise ValueError("candidates must be [rows, K] ids and values of equal shape")
    world = dist.get_world_size(group)
    rows, K = local_ids.shape
    # Output is the ranks' inputs concatenated along dim 0: [world * rows, K].
    ids = torch.empty((world * rows, K), dtype=local_ids.dtype, device=local_ids.device)
    vals = torch.empty((world * rows, K), dtype=local_vals.dtype, device=local_vals.device)
    dist.all_gather_into_tensor(ids, local_ids.contiguous(), group=group)
    dist.all_gather_into_tensor(vals, local_vals.contiguous(), group=group)
    return (ids.view(world, rows, K).permute(1, 0, 2).contiguous(),
            vals.view(world, rows, K).permute(1, 0, 2).contiguous())


def vocab_sharded_topk(local_logits: torch.Tensor, shard: Shard, K: int,
                       uniform: Optional[torch.Tensor] = None, temperature: float = 1.0,
                       group: Optional[dist.ProcessGroup] = None):
    """Top-K (and optional sampling) over logits whose vocab axis is split across ranks.
    local_logits [rows, shard.size] on this rank's GPU.  Returns (ids [rows, K], vals [rows, K],
    sampled [rows] or None), identical on every rank."""
    from . import ops

    rows = local_logits.shape[0]
    dev, dt = local_logits.device, local_logits.dtype
    slices = 8
    sc_i = torch.empty((rows, slices, K), dtype=torch.int32, device=dev)
    sc_v = torch.empty((rows, slices, K), dtype=dt, device=dev)
    loc_i = torch.empty((rows, K), dtype=torch.int32, device=dev)
    loc_v = torch.empty((rows, K), dtype=dt, device=dev)
    ops.launchTopKforBeamSearch(local_logits, sc_i, sc_v, loc_i, loc_v, index_offset=shard.start)
    cand_i, cand_v = gather_candidates(loc_i, loc_v, group)
    out_i = torch.empty((rows, K), dtype=torch.int32, device=dev)
    out_v = torch.empty((rows, K), dtype=dt, device=dev)
    picked = torch.empty((rows,), dtype=torch.int32, device=dev) if uniform is not None else None
    ops.launchTopKMerge(cand_i, cand_v, out_i, out_v, uniform, temperature, picked)
    return out_i, out_v, picked
