"""Batch sharding across the GPUs of one box: the only multi-GPU logic of this path.

Every sample of every configuration is independent, so a batch is split into contiguous shards of
ceil(B / G) samples, weights are replicated (each rank builds its own Session) and no collective
runs on the data path. This mirrors the reference's one-Session-per-slot idiom
(src/SOFIE_core/inc/SOFIE/SOFIEHelpers.hxx:23-49). torch.distributed is used for the barrier and
for reducing timings only.
"""
from __future__ import annotations

import numpy as np


def shard_bounds(batch: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the rank's contiguous shard; the last shards may be short or empty."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    per = -(-batch // world)
    begin = min(batch, rank * per)
    return begin, min(batch, begin + per)


def shard(x: np.ndarray, world: int, rank: int) -> np.ndarray:
    b, e = shard_bounds(x.shape[0], world, rank)
    return x[b:e]


def max_over_ranks(value: float, device="cpu") -> float:
    """The slowest rank's time: what a whole-job throughput has to be computed from."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def gather_rows(local: np.ndarray, batch: int):
    """All ranks' output rows in rank order (test / verification helper; not on the data path)."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(), dist.get_rank()
    per = -(-batch // world)
    pad = np.zeros((per,) + local.shape[1:], local.dtype)
    pad[: local.shape[0]] = local
    out = [torch.empty_like(torch.from_numpy(pad)) for _ in range(world)]
    dist.all_gather(out, torch.from_numpy(pad))
    rows = []
    for r, t in enumerate(out):
        b, e = shard_bounds(batch, world, r)
        rows.append(t.numpy()[: e - b])
    return np.concatenate(rows, axis=0)
