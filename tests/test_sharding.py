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


def _packed_main(rank, world, port, rows, vocab, K, seed, out_dir):
    """The exchange the GPU path uses, on gloo: each rank packs [rows, K] ids | [rows, K] values into
    one record, one all_gather_into_tensor, and the merge reads list l of row r at
    record l, offset r*K (ids) and rows*K*4 + r*K*itemsize (values)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from inferspore_b200.ops import packed_record_bytes
        from oracle import binding as orc

        rng = np.random.default_rng(seed)
        logits = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
        logits[:, ::13] = logits[:, 1:2]
        sh = vocab_shard(vocab, world, rank)
        loc_i, loc_v = orc.topk(np.ascontiguousarray(logits[:, sh.start:sh.stop]), K, index_offset=sh.start)
        record = packed_record_bytes(rows, K, torch.float32)
        assert record % 16 == 0 and record >= rows * K * 8
        packed = np.zeros(record, np.uint8)
        packed[:rows * K * 4] = loc_i.view(np.uint8).reshape(-1)
        packed[rows * K * 4:rows * K * 8] = loc_v.view(np.uint8).reshape(-1)
        gathered = torch.empty(world * record, dtype=torch.uint8)
        dist.all_gather_into_tensor(gathered, torch.from_numpy(packed))
        g = gathered.numpy().reshape(world, record)
        cand_i = np.stack([g[l, :rows * K * 4].view(np.int32).reshape(rows, K) for l in range(world)], 1)
        cand_v = np.stack([g[l, rows * K * 4:rows * K * 8].view(np.float32).reshape(rows, K) for l in range(world)], 1)
        got_i, got_v = orc.topk_merge(cand_i, cand_v, K)
        want_i, want_v = orc.topk(logits, K)
        assert np.array_equal(got_i, want_i) and np.array_equal(got_v, want_v)
        np.save(Path(out_dir) / f"packed{rank}.npy", got_i)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_packed_record_exchange_two_gloo_ranks(tmp_path):
    port = 30500 + (os.getpid() % 2000)
    mp.start_processes(_packed_main, args=(2, port, 5, 1003, 7, 99, str(tmp_path)), nprocs=2, join=True,
                       start_method="spawn")
    assert np.array_equal(np.load(tmp_path / "packed0.npy"), np.load(tmp_path / "packed1.npy"))


# ---- failure modes, on the host: a rank that never joins, a rank that leaves between two steps ----

def _lonely_main(rank, world, port, out_dir):
    """Rank 0 of a two-rank group whose other rank never starts: the rendezvous must give up within
    the timeout and raise, not hang."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    t0 = time.monotonic()
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=5))
        outcome = "joined"
    except Exception as e:  # DistStoreError / DistNetworkError / RuntimeError, by torch version
        outcome = "raised " + type(e).__name__
    (Path(out_dir) / "lonely.txt").write_text(f"{outcome} {time.monotonic() - t0:.1f}")


@pytest.mark.timeout(120)
def test_init_with_a_missing_rank_times_out(tmp_path):
    port = 32500 + (os.getpid() % 2000)
    mp.start_processes(_lonely_main, args=(2, port, str(tmp_path)), nprocs=1, join=True, start_method="spawn")
    outcome, seconds = (tmp_path / "lonely.txt").read_text().split(" ", 1)[0], float((tmp_path / "lonely.txt").read_text().rsplit(" ", 1)[1])
    assert outcome == "raised" and seconds < 60


def _leaver_main(rank, world, port, out_dir):
    """Two ranks exchange candidates once; then rank 1 fails on the host between two steps (no
    collective of its own in flight) and leaves.  Rank 0's next exchange must end with an error
    within the group's short timeout instead of waiting forever."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from inferspore_b200.sharding import gather_candidates

    ids = torch.full((4, 5), rank, dtype=torch.int32)
    vals = torch.full((4, 5), float(rank))
    cand_i, _ = gather_candidates(ids, vals)  # step 1: both ranks take part
    assert cand_i[:, 1].eq(1).all()
    if rank == 1:
        os._exit(0)  # leaves between steps: no destroy, no further collective
    t0 = time.monotonic()
    try:
        gather_candidates(ids, vals)  # step 2: the peer is gone
        outcome = "completed"
    except Exception as e:
        outcome = "raised " + type(e).__name__
    (Path(out_dir) / "survivor.txt").write_text(f"{outcome} {time.monotonic() - t0:.1f}")
    os._exit(0)  # the group is broken: skip the orderly shutdown, which would wait for the peer


@pytest.mark.timeout(180)
def test_a_rank_that_leaves_between_steps_fails_the_survivor_quickly(tmp_path):
    port = 33900 + (os.getpid() % 2000)
    mp.start_processes(_leaver_main, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    text = (tmp_path / "survivor.txt").read_text()
    assert text.startswith("raised"), text
    assert float(text.rsplit(" ", 1)[1]) < 60


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
