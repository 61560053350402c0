"""Sequence-sharded replicas: how a decode batch spreads over the GPUs of a box.

The path has no exchange step. Each GPU owns its sequences' pages, block tables
and graphs, exactly as the reference's per-GPU engine replicas do
(runtime/router.py:30-77, benchmarks/runners/phase18_replicas.py:226-308), so
going from 1 to N GPUs needs a partition of the sequences and, for
measurement, a barrier and a max over ranks — nothing on the data path.
"""

from __future__ import annotations

import heapq
from typing import Sequence


def partition_by_tokens(lens: Sequence[int], world: int) -> list[list[int]]:
    """Indices of `lens` for each of `world` replicas, balanced by outstanding
    tokens (longest first onto the lightest replica) — the refinement the
    reference's notes ask of its least-loaded routing (docs/phase18_multigpu.md:147-153).
    Deterministic: ties go to the lower rank, then the lower index."""
    if world <= 0:
        raise ValueError("world must be positive")
    shards: list[list[int]] = [[] for _ in range(world)]
    heap = [(0, r) for r in range(world)]
    heapq.heapify(heap)
    for i in sorted(range(len(lens)), key=lambda j: (-int(lens[j]), j)):
        load, r = heapq.heappop(heap)
        shards[r].append(i)
        heapq.heappush(heap, (load + int(lens[i]), r))
    for s in shards:
        s.sort()
    return shards


def max_over_ranks(value, dist=None, device=None):
    """The slowest rank's time: what a multi-replica number must be quoted on.
    A float, or a list of times reduced element by element."""
    many = isinstance(value, (list, tuple))
    values = [float(v) for v in value] if many else [float(value)]
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        import torch

        t = torch.tensor(values, dtype=torch.float64, device=device or "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        values = [float(x) for x in t.tolist()]
    return values if many else values[0]


def aggregate_throughput(units_per_rank: float, seconds: float, world: int) -> float:
    """Whole-job throughput when every rank processed `units_per_rank` in
    `seconds` (the max over ranks): weak scaling, no shared work."""
    return world * units_per_rank / seconds
