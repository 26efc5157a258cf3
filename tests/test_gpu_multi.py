"""Vocab-sharded top-K over NCCL: one process per GPU, each rank reduces its own column slice with
the CUDA kernel, one all-gather of the candidate lists, every rank merges.  The result must be
bit-identical to the unsharded kernel and to the oracle.  Needs two GPUs; skipped otherwise."""
import os
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, rows, vocab, K, seed, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_DEBUG="WARN")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from inferspore_b200 import ops
        from inferspore_b200.sharding import vocab_shard, vocab_sharded_topk

        rng = np.random.default_rng(seed)  # the same logits on every rank; each keeps its own columns
        logits = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
        logits[:, ::13] = logits[:, 1:2]  # ties that straddle shard boundaries
        u = rng.random(rows).astype(np.float32)
        sh = vocab_shard(vocab, world, rank)
        local = torch.from_numpy(np.ascontiguousarray(logits[:, sh.start:sh.stop])).to(device)
        ids, vals, picked = vocab_sharded_topk(local, sh, K, uniform=torch.from_numpy(u).to(device), temperature=0.8)
        # the unsharded kernel on this rank's GPU
        full = torch.from_numpy(logits).to(device)
        sc_i = torch.empty((rows, 8, K), dtype=torch.int32, device=device)
        sc_v = torch.empty((rows, 8, K), device=device)
        f_i = torch.empty((rows, K), dtype=torch.int32, device=device)
        f_v = torch.empty((rows, K), device=device)
        f_p = torch.empty(rows, dtype=torch.int32, device=device)
        ops.launchTopKforBeamSearch(full, sc_i, sc_v, f_i, f_v, 0, torch.from_numpy(u).to(device), 0.8, f_p)
        torch.cuda.synchronize()
        assert torch.equal(ids, f_i) and torch.equal(vals, f_v) and torch.equal(picked, f_p)
        np.savez(Path(out_dir) / f"rank{rank}.npz", ids=ids.cpu().numpy(), vals=vals.cpu().numpy(),
                 picked=picked.cpu().numpy(), logits=logits)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("rows,vocab,K", [(256, 32000, 50), (7, 1003, 5)])
def test_vocab_sharded_topk_over_nccl(cuda, orc, tmp_path, rows, vocab, K):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = 33500 + (os.getpid() % 2000)
    mp.start_processes(_rank_main, args=(world, port, rows, vocab, K, 4242, str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    got = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    want_i, want_v = orc.topk(got[0]["logits"], K)
    for g in got:  # every rank holds the same answer, and it is the oracle's
        assert np.array_equal(g["ids"], want_i) and np.array_equal(g["vals"], want_v)
        assert np.array_equal(g["picked"], got[0]["picked"])
