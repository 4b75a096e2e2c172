"""Batch sharding of backbone inference across the GPUs of one box.

Every (image, route, channel) row of the SS2D core is an independent recurrence and no layer of the
backbone mixes images, so the path shards by batch with no data-path exchange: one process per GPU,
each with a full weight replica and its own contiguous slice of the global batch.  The only
communication is the host-side bookkeeping below (a max over the per-rank times, a gather of the
per-rank image counts), done with torch.distributed on whatever backend the job initialised.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(global_batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [start, start+count) of a global batch for `rank`; the first
    `global_batch % world` ranks take one extra image.  Empty slices are allowed."""
    if world < 1 or not (0 <= rank < world) or global_batch < 0:
        raise ValueError(f"bad shard request: batch {global_batch}, world {world}, rank {rank}")
    base, extra = divmod(global_batch, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def max_over_ranks(value: float, device: str = "cpu") -> float:
    """The slowest rank's value (the time a multi-GPU step really took)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device: str = "cpu") -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def aggregate_throughput(images_this_rank: int, elapsed_ms_this_rank: float, device: str = "cpu") -> float:
    """Whole-job images per second: all ranks' images over the slowest rank's time."""
    total = sum_over_ranks(float(images_this_rank), device)
    ms = max_over_ranks(float(elapsed_ms_this_rank), device)
    return total / (ms * 1e-3)


class ShardFailure(RuntimeError):
    """A rank of the job did not take part in the host-side bookkeeping (it exited or hung): the
    whole-job number of this step is void.  Raised on the surviving ranks instead of a backend error."""


def aggregate_throughput_or_fail(images_this_rank: int, elapsed_ms_this_rank: float, device: str = "cpu") -> float:
    """`aggregate_throughput`, with any failure of the collective (a peer that closed its connection,
    the process group's timeout running out) reported as ShardFailure naming this rank.  The data path
    has no collective, so a lost rank cannot leave a kernel of another rank waiting: the survivors'
    GPUs finish their own step; only the bookkeeping fails, on the host, between steps."""
    try:
        return aggregate_throughput(images_this_rank, elapsed_ms_this_rank, device)
    except Exception as e:  # noqa: BLE001 - gloo / nccl raise backend-specific RuntimeErrors
        rank = dist.get_rank() if dist.is_initialized() else 0
        raise ShardFailure(f"rank {rank}: a peer left the job during the step bookkeeping ({type(e).__name__}: {e})") from e
