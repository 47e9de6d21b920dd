"""NCCL collectives with the calling conventions of ``rocshmem_b200.ops.collectives`` (for benchmarks)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def allreduce(dest: torch.Tensor, source: torch.Tensor, group=None) -> torch.Tensor:
    """``dist.all_reduce`` (sum) of ``source`` into ``dest``."""
    if dest.data_ptr() != source.data_ptr():
        dest.copy_(source)
    dist.all_reduce(dest, group=group)
    return dest


def allgather(dest: torch.Tensor, source: torch.Tensor, group=None) -> torch.Tensor:
    """``dist.all_gather_into_tensor``."""
    dist.all_gather_into_tensor(dest, source, group=group)
    return dest


def alltoall(dest: torch.Tensor, source: torch.Tensor, group=None) -> torch.Tensor:
    """``dist.all_to_all_single`` with equal splits."""
    dist.all_to_all_single(dest, source, group=group)
    return dest


def broadcast(buf: torch.Tensor, root: int, group=None) -> torch.Tensor:
    """``dist.broadcast`` of ``buf`` from ``root``."""
    dist.broadcast(buf, src=root, group=group)
    return buf
