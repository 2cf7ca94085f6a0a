"""Rank plumbing for multi-GPU runs: one process per GPU, independent scheduler replicas.

The path has no cross-GPU tensor traffic, so there is no data-path collective; ranks only meet
at a barrier around the timed region and to take the maximum of their device times.  The
rendezvous uses torch.distributed with the gloo backend (host tensors).
"""
from __future__ import annotations

import os


def init(world: int, rank: int):
    """Returns an opaque group handle (None for a single process)."""
    if world <= 1:
        return None
    import datetime

    import torch.distributed as td

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if not td.is_initialized():
        td.init_process_group("gloo", rank=rank, world_size=world,
                              timeout=datetime.timedelta(seconds=600))
    return td


def barrier(group) -> None:
    if group is not None:
        group.barrier()


def max_over_ranks(group, value: float) -> float:
    if group is None:
        return float(value)
    import torch

    t = torch.tensor([float(value)], dtype=torch.float64)
    group.all_reduce(t, op=group.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(group, value: float) -> float:
    if group is None:
        return float(value)
    import torch

    t = torch.tensor([float(value)], dtype=torch.float64)
    group.all_reduce(t, op=group.ReduceOp.SUM)
    return float(t.item())


def shard(items: list, world: int, rank: int) -> list:
    """Round-robin assignment of independent clients to ranks (one scheduler per GPU)."""
    return [it for i, it in enumerate(items) if i % max(world, 1) == rank]


def finish(group) -> None:
    if group is not None and group.is_initialized():
        group.destroy_process_group()
