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


class VocabShardedTopK:
    """Top-K (and optional sampling) over logits whose vocab axis is split across ranks, with
    every buffer allocated once: local top-K with global ids written straight into this rank's
    packed record ([rows, K] int32 ids | [rows, K] values, padded to 16 bytes), ONE all-gather of
    the records, and a merge (+ sampling) on every rank that reads the gathered buffer in place
    (ispore_topk_merge_strided_*: one list per rank, list stride = record size).  Three launches
    per call — local top-K, the collective, the merge — and no re-layout copy."""

    def __init__(self, rows: int, K: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, slices: int = 8):
        from . import ops

        self.rows, self.K, self.group = rows, K, group
        self.world = dist.get_world_size(group)
        esize = torch.empty((), dtype=dtype).element_size()
        ids_bytes, vals_bytes = rows * K * 4, rows * K * esize
        self.record_bytes = ops.packed_record_bytes(rows, K, dtype)
        self.packed = torch.zeros(self.record_bytes, dtype=torch.uint8, device=device)
        self.loc_i = self.packed[:ids_bytes].view(torch.int32).view(rows, K)
        self.loc_v = self.packed[ids_bytes:ids_bytes + vals_bytes].view(dtype).view(rows, K)
        self.gathered = torch.empty((self.world, self.record_bytes), dtype=torch.uint8, device=device)
        self.sc_i = torch.empty((rows, slices, K), dtype=torch.int32, device=device)
        self.sc_v = torch.empty((rows, slices, K), dtype=dtype, device=device)
        self.out_i = torch.empty((rows, K), dtype=torch.int32, device=device)
        self.out_v = torch.empty((rows, K), dtype=dtype, device=device)
        self.picked = torch.empty((rows,), dtype=torch.int32, device=device)

    def local(self, local_logits: torch.Tensor, shard: Shard) -> None:
        """Step 1: this rank's candidates (global ids) into its packed record."""
        from . import ops

        if local_logits.shape != (self.rows, shard.size):
            raise ValueError("local logits must be [rows, shard.size]")
        ops.launchTopKforBeamSearch(local_logits, self.sc_i, self.sc_v, self.loc_i, self.loc_v,
                                    index_offset=shard.start)

    def exchange(self) -> None:
        """Step 2: every rank's record to every rank (the path's only collective)."""
        dist.all_gather_into_tensor(self.gathered.view(-1), self.packed, group=self.group)

    def merge(self, uniform: Optional[torch.Tensor] = None, temperature: float = 1.0):
        """Step 3: merge the gathered lists where they lie; optionally draw one id per row."""
        from . import ops

        picked = self.picked if uniform is not None else None
        ops.launchTopKMergeGathered(self.gathered, self.world, self.rows, self.K, self.out_i, self.out_v, uniform,
                                    temperature, picked)
        return self.out_i, self.out_v, picked

    def __call__(self, local_logits: torch.Tensor, shard: Shard, uniform: Optional[torch.Tensor] = None,
                 temperature: float = 1.0):
        self.local(local_logits, shard)
        self.exchange()
        return self.merge(uniform, temperature)


_SHARDED_TOPK_CACHE: dict = {}


def vocab_sharded_topk(local_logits: torch.Tensor, shard: Shard, K: int,
                       uniform: Optional[torch.Tensor] = None, temperature: float = 1.0,
                       group: Optional[dist.ProcessGroup] = None):
    """Top-K (and optional sampling) over logits whose vocab axis is split across ranks.
    local_logits [rows, shard.size] on this rank's GPU.  Returns (ids [rows, K], vals [rows, K],
    sampled [rows] or None), identical on every rank; the returned tensors are reused by the next
    call of the same shape."""
    key = (local_logits.shape[0], K, local_logits.dtype, local_logits.device, id(group))
    op = _SHARDED_TOPK_CACHE.get(key)
    if op is None:
        op = _SHARDED_TOPK_CACHE[key] = VocabShardedTopK(local_logits.shape[0], K, local_logits.dtype,
                                                         local_logits.device, group)
    return op(local_logits, shard, uniform, temperature)
