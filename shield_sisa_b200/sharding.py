"""Splitting windows across the GPUs of one box: contiguous shards, one engine per GPU, host gather of logits.

Windows are independent (row independence is part of the C ABI's contract, reference engine/include/shv_cuda.h:31-34)
and every session's state is private, so the sequence path needs no data-path collective: rank r of n scores windows
[shard(r)) with its own model on its own device and the B floats are gathered on the host.  For the live service a
participant's token ring must stay on one device, so participants (not windows) are the unit that is placed.
"""
from __future__ import annotations

import zlib


def shard_bounds(total: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of rank's contiguous shard; sizes differ by at most one, earlier ranks take the extra window."""
    if world < 1 or not 0 <= rank < world or total < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def device_of_participant(participant_id: str, world: int) -> int:
    """Stable placement of a participant (and its device token slots) on one of `world` GPUs."""
    if world < 1:
        raise ValueError("world must be >= 1")
    return zlib.crc32(participant_id.encode()) % world


def gather_logits(local, total: int, world: int, rank: int, group=None):
    """All ranks pass their shard's logits (1-D float32 torch tensor on CPU); rank 0 gets the [total] vector in window
    order, the others None.  Host-side gather through torch.distributed (gloo or NCCL-independent object of the
    default group); nothing on the GPU data path."""
    import torch
    import torch.distributed as dist

    lo, hi = shard_bounds(total, world, rank)
    if local.numel() != hi - lo:
        raise ValueError(f"rank {rank} holds {local.numel()} logits, shard is {hi - lo}")
    if world == 1:
        return local.clone()
    sizes = [shard_bounds(total, world, r)[1] - shard_bounds(total, world, r)[0] for r in range(world)]
    pad = max(sizes)
    buf = torch.full((pad,), float("nan"), dtype=torch.float32)
    buf[: local.numel()] = local
    out = [torch.empty(pad, dtype=torch.float32) for _ in range(world)] if rank == 0 else None
    dist.gather(buf, out, dst=0, group=group)
    if rank != 0:
        return None
    return torch.cat([o[:n] for o, n in zip(out, sizes)])
