"""Partitioning of attention work across the GPUs of one box.

Attention rows of different (batch, head) pairs never interact, so the path shards with no
data-path collective: each rank (one process per GPU) takes a contiguous block of the
flattened batch x KV-head units and runs the same kernel on its own slice.  Query heads
follow their KV head (grouped-query attention keeps a KV head and its query heads on one
rank).  The reference is single-GPU; this is the multi-GPU story of the B200 build.
"""
from __future__ import annotations

from typing import List, Tuple


def shard_units(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block [start, stop) of `total` units for `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch_kvheads(B: int, Hkv: int, world: int, rank: int) -> List[Tuple[int, int, int]]:
    """This rank's units as (batch, kv_head_start, kv_head_stop) runs, so that each run is a
    plain view ``t[b, h0:h1]`` of a [B, H, S, D] tensor."""
    start, stop = shard_units(B * Hkv, world, rank)
    runs = []
    u = start
    while u < stop:
        b, h0 = divmod(u, Hkv)
        h1 = min(Hkv, h0 + (stop - u))
        runs.append((b, h0, h1))
        u += h1 - h0
    return runs


def aggregate_tflops(flops_per_rank: List[float], ms_per_rank: List[float]) -> float:
    """Whole-job throughput: all ranks' algorithmic FLOPs over the slowest rank's time."""
    if not ms_per_rank or max(ms_per_rank) <= 0:
        raise ValueError("need positive per-rank times")
    return sum(flops_per_rank) / (max(ms_per_rank) * 1e-3) / 1e12
