"""Multi-GPU: independent data-parallel replicas.

The activation path has no exchange step: every tensor belongs to one GPU's
replica, each replica owns its pool, streams and pinned slab, and nothing on the
data path is a collective.  What N processes share is only the measurement
protocol: start together, time on the device, take the slowest rank, add up the
units.  ``torch.distributed`` carries those three scalars (NCCL on GPUs, gloo in
the CPU tests); it never carries activation bytes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class ReplicaEnv:
    rank: int
    world: int
    local_rank: int

    @staticmethod
    def from_env() -> "ReplicaEnv":
        return ReplicaEnv(int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
                          int(os.environ.get("LOCAL_RANK", "0")))


def workload_seed(rank: int, base: int = 0) -> int:
    """Each replica offloads its own data (seed = rank), so no two replicas send identical bytes."""
    return base + rank


def barrier(world: int) -> None:
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def max_over_ranks(value: float, world: int, device=None) -> float:
    """The job is as slow as its slowest replica."""
    if world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, world: int, device=None) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def aggregate_gbs(bytes_per_rank: float, world: int, slowest_ms: float, device=None) -> float:
    """Whole-job GB/s: bytes all replicas moved divided by the slowest replica's time."""
    total = sum_over_ranks(bytes_per_rank, world, device)
    return total / (slowest_ms * 1e-3) * 1e-9


def gather_over_ranks(value: float, world: int, device=None) -> list:
    """The same scalar from every rank, in rank order (for per-replica link rates)."""
    if world == 1:
        return [value]
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(o.item()) for o in out]
