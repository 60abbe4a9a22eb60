"""Batch sharding of independent sequences over the GPUs of one node.

Sequences never interact (the reference would serve N sequences as N clones of `Gpt2Model` over
shared weights, puppygrad src/models/gpt2/rust.rs:142-148), so multi-GPU is replicas only: every
rank holds all weights and a disjoint slice of the sequences; nothing crosses GPUs on the token
path. The only collectives are a barrier and the reductions of the timing, plus an optional
gather of the finished token streams. Works with any `torch.distributed` backend (NCCL on GPUs,
gloo on CPU for tests).
"""
from __future__ import annotations

from typing import Dict, List, Sequence


def partition(n_items: int, world: int, rank: int) -> List[int]:
    """Sequence i goes to rank i mod world."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    return list(range(rank, n_items, world))


def gather_streams(local: Dict[int, Sequence[int]], n_items: int) -> List[List[int]]:
    """Collects {sequence index: token stream} from every rank into one list ordered by index."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        parts = [dict(local)]
    else:
        parts = [None] * dist.get_world_size()
        dist.all_gather_object(parts, {int(k): [int(t) for t in v] for k, v in local.items()})
    merged: Dict[int, List[int]] = {}
    for p in parts:
        for k, v in p.items():
            if k in merged:
                raise ValueError(f"sequence {k} was produced by two ranks")
            merged[k] = list(v)
    missing = [i for i in range(n_items) if i not in merged]
    if missing:
        raise ValueError(f"sequences {missing[:8]} were produced by no rank")
    return [merged[i] for i in range(n_items)]


def max_over_ranks(value: float, device=None) -> float:
    """Slowest rank's time: multi-GPU throughput is total work over the maximum device time."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
