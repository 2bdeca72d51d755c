"""Multi-GPU host logic: contiguous window shards, stable participant placement, host gather over gloo (2 ranks)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from shield_sisa_b200 import sharding


@pytest.mark.parametrize("total,world", [(0, 1), (1, 2), (7, 2), (4096, 8), (4097, 8), (5, 8), (32768, 4)])
def test_shards_partition_the_windows(total, world):
    bounds = [sharding.shard_bounds(total, world, r) for r in range(world)]
    assert bounds[0][0] == 0 and bounds[-1][1] == total
    for (a, b), (c, d) in zip(bounds, bounds[1:]):
        assert b == c and a <= b and c <= d
    sizes = [b - a for a, b in bounds]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        sharding.shard_bounds(total, world, world)


def test_participant_placement_is_stable_and_spread():
    ids = [f"participant-{i}" for i in range(4000)]
    place = [sharding.device_of_participant(p, 8) for p in ids]
    assert place == [sharding.device_of_participant(p, 8) for p in ids]
    counts = np.bincount(place, minlength=8)
    assert counts.min() > 400 and counts.max() < 600


def _scorer(tokens):
    """Stand-in for one GPU's engine: any deterministic per-window function."""
    return torch.from_numpy(np.asarray(tokens, np.float64).reshape(len(tokens), -1).sum(1).astype(np.float32))


def _rank_main(rank, world, port, total, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)
        tokens = rng.standard_normal((total, 8)).astype(np.float32)       # every rank sees the same job list
        lo, hi = sharding.shard_bounds(total, world, rank)
        local = _scorer(tokens[lo:hi])
        dist.barrier()
        full = sharding.gather_logits(local, total, world, rank)
        if rank == 0:
            np.save(out_path, full.numpy())
        else:
            assert full is None
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [9, 64])
def test_two_rank_gather_matches_single_rank(tmp_path, total):
    out = tmp_path / "gathered.npy"
    port = 29000 + (os.getpid() + total) % 2000
    mp.spawn(_rank_main, args=(2, port, total, str(out)), nprocs=2, join=True)
    rng = np.random.default_rng(11)
    tokens = rng.standard_normal((total, 8)).astype(np.float32)
    np.testing.assert_array_equal(np.load(out), _scorer(tokens).numpy())


def test_single_rank_gather_is_identity():
    x = torch.arange(5, dtype=torch.float32)
    assert torch.equal(sharding.gather_logits(x, 5, 1, 0), x)
    with pytest.raises(ValueError):
        sharding.gather_logits(x, 6, 1, 0)
