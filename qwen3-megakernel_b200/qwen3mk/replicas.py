"""Data-parallel replicas: one process and one engine per GPU, requests partitioned, no inter-GPU traffic
on the data path.  The reference is single-GPU (qwen3mk/kernel.py:120-131 binds one device); this module
is the layer a multi-GPU deployment adds on top of `Megakernel`.

Only the bookkeeping needs a process group (any torch.distributed backend: NCCL on GPUs, gloo on CPUs):
which requests a rank serves, the slowest rank's time, and the job's aggregate throughput.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def world() -> tuple[int, int]:
    """(rank, world_size); (0, 1) without an initialised process group."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def partition(n_requests: int, rank: int | None = None, size: int | None = None) -> list[int]:
    """Indices of the requests rank `rank` serves: round-robin, so that lengths sorted by the caller stay balanced."""
    r, s = world()
    rank = r if rank is None else rank
    size = s if size is None else size
    if not 0 <= rank < size:
        raise ValueError(f"rank {rank} outside a world of {size}")
    return list(range(rank, n_requests, size))


def max_over_ranks(value: float, device=None) -> float:
    """The largest `value` over all ranks (the job is as slow as its slowest replica)."""
    _, size = world()
    if size == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def sum_over_ranks(value: float, device=None) -> float:
    _, size = world()
    if size == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t[0])


def aggregate_throughput(units_this_rank: float, seconds_this_rank: float, device=None) -> dict:
    """Whole-job throughput of a replicated run: all units over the slowest rank's time."""
    total = sum_over_ranks(units_this_rank, device)
    slowest = max_over_ranks(seconds_this_rank, device)
    return {"units": total, "seconds": slowest, "per_second": total / slowest if slowest > 0 else float("inf")}


def gather_tokens(tokens: torch.Tensor, indices: list[int], n_requests: int) -> torch.Tensor:
    """Reassemble per-request results (int64 [len(indices), ...]) from all ranks into request order on every rank."""
    _, size = world()
    out = torch.full((n_requests,) + tuple(tokens.shape[1:]), -1, dtype=tokens.dtype, device=tokens.device)
    out[torch.as_tensor(indices, dtype=torch.int64, device=tokens.device)] = tokens
    if size > 1:
        dist.all_reduce(out, op=dist.ReduceOp.MAX)   # unserved slots are -1 on every other rank
    return out
