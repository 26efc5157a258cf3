"""Multi-rank host logic on CPU: shard planning, and the vocab-sharded top-K exchange run as two
gloo ranks (the all-gather layout feeds the same merge the GPU path uses; the oracle stands in
for the per-rank kernels, which need a GPU)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from inferspore_b200.sharding import shard_range, shard_sequences, vocab_shard  # noqa: E402


@pytest.mark.parametrize("total,world", [(65536, 8), (128, 8), (10, 4), (3, 8), (0, 2), (7, 1)])
def test_shard_range_partitions_exactly(total, world):
    shards = [shard_range(total, world, r) for r in range(world)]
    assert shards[0].start == 0 and shards[-1].stop == total
    assert all(a.stop == b.start for a, b in zip(shards, shards[1:]))
    sizes = [s.size for s in shards]
    assert max(sizes) - min(sizes) <= 1 and sum(sizes) == total


def test_shard_errors():
    for bad in [(10, 0, 0), (10, 2, 2), (10, 2, -1), (-1, 2, 0)]:
        with pytest.raises(ValueError):
            shard_range(*bad)


def test_shard_sequences_keeps_whole_sequences():
    seqs, toks = shard_sequences(128, 512, 8, 3)
    assert (seqs.start, seqs.stop) == (48, 64) and (toks.start, toks.stop) == (48 * 512, 64 * 512)


@pytest.mark.parametrize("vocab,world", [(32000, 8), (32001, 8), (128256, 4), (50, 8), (7, 2)])
def test_vocab_shard_is_aligned_and_covers(vocab, world):
    shards = [vocab_shard(vocab, world, r) for r in range(world)]
    assert shards[0].start == 0 and shards[-1].stop == vocab
    assert all(a.stop == b.start for a, b in zip(shards, shards[1:]))
    assert all(s.start % 8 == 0 or s.size == 0 for s in shards)


def _rank_main(rank, world, port, rows, vocab, K, seed, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from inferspore_b200.sharding import gather_candidates
        from oracle import binding as orc

        rng = np.random.default_rng(seed)  # same logits on every rank; each keeps its own columns
        logits = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
        logits[:, ::13] = logits[:, 1:2]  # ties that straddle shard boundaries
        sh = vocab_shard(vocab, world, rank)
        loc_i, loc_v = orc.topk(np.ascontiguousarray(logits[:, sh.start:sh.stop]), K, index_offset=sh.start)
        cand_i, cand_v = gather_candidates(torch.from_numpy(loc_i), torch.from_numpy(loc_v))
        assert cand_i.shape == (rows, world, K)
        assert np.array_equal(cand_i[:, rank].numpy(), loc_i)  # rank-major lists per row
        got_i, got_v = orc.topk_merge(cand_i.numpy(), cand_v.numpy(), K)
        want_i, want_v = orc.topk(logits, K)
        assert np.array_equal(got_i, want_i) and np.array_equal(got_v, want_v)
        np.save(Path(out_dir) / f"ids{rank}.npy", got_i)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_vocab_sharded_topk_two_gloo_ranks(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.start_processes(_rank_main, args=(2, port, 6, 1003, 20, 99, str(tmp_path)), nprocs=2, join=True,
                       start_method="spawn")
    a, b = np.load(tmp_path / "ids0.npy"), np.load(tmp_path / "ids1.npy")
    assert np.array_equal(a, b)  # every rank ends with the same answer


def _mismatch_main(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from inferspore_b200.sharding import gather_candidates

        with pytest.raises(ValueError):  # ids / values of different shapes never reach the collective
            gather_candidates(torch.zeros((4, 5), dtype=torch.int32), torch.zeros((4, 6)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_bad_candidate_shapes_fail_on_the_host(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    mp.start_processes(_mismatch_main, args=(2, port), nprocs=2, join=True, start_method="spawn")
