"""Scale-out by independent replicas: a stream never shards, so each GPU runs its
own engine on a disjoint set of streams and nothing crosses GPUs in the data
path (the reference has no multi-GPU mode at all).  A process group is used only
to line up the timed window and to combine per-rank counters."""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_streams(n_streams: int, rank: int, world: int) -> list[int]:
    """Global stream ids owned by `rank`: stream s lives on rank s mod world."""
    return [s for s in range(n_streams) if s % world == rank]


def aggregate_rate(units: float, elapsed_ms: float, device=None) -> tuple[float, float]:
    """Whole-job throughput over all ranks: (sum of units) / (max elapsed time).
    Returns (units_per_second, max_elapsed_ms).  Works without a process group."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return units / (elapsed_ms * 1e-3), elapsed_ms
    dev = device if device is not None else "cpu"
    tot = torch.tensor([units], dtype=torch.float64, device=dev)
    mx = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    return tot.item() / (mx.item() * 1e-3), mx.item()
