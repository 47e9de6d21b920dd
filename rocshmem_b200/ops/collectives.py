"""Collectives on symmetric tensors.

Two flavours of every operation:

* host-blocking (``broadcast``, ``reduce``, ``fcollect``, ``alltoall``): the OpenSHMEM host API, which
  returns when the collective has completed on this PE (reference: the host collectives of
  ``include/rocshmem/rocshmem_COLL.hpp``, implemented there with MPI);
* stream-ordered (``*_async``): the library's multi-block kernels enqueued on a CUDA stream, for use
  next to other GPU work. They need the CUDA backend.

All tensors must come from :func:`rocshmem_b200.empty` / :func:`rocshmem_b200.zeros` (symmetric heap).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt


def _team(team: Optional[rt.Team]) -> int:
    return (team or rt.team_world()).handle


def _check(dest: torch.Tensor, source: torch.Tensor, dest_elems: int, what: str) -> None:
    """Both buffers symmetric and contiguous, same element type, ``dest`` large enough."""
    rt.require_symmetric(dest=dest, source=source)
    if dest.dtype != source.dtype:
        raise ValueError(f"{what}: dest is {dest.dtype}, source is {source.dtype}")
    if dest.numel() < dest_elems:
        raise ValueError(f"{what}: dest holds {dest.numel()} elements, {dest_elems} are needed")


def _stream(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


# ---- host-blocking -----------------------------------------------------------------------------------

def broadcast(dest: torch.Tensor, source: torch.Tensor, root: int, team: Optional[rt.Team] = None) -> int:
    """``dest`` on every member except the root receives the root's ``source``."""
    _check(dest, source, source.numel(), "broadcast")
    return rt._C().broadcast(_team(team), dest.data_ptr(), source.data_ptr(), rt._nbytes(source), root)


def reduce(dest: torch.Tensor, source: torch.Tensor, op: int = rt.OP_SUM,
           team: Optional[rt.Team] = None) -> int:
    """All-reduce: every member's ``dest`` receives the element-wise reduction of all ``source``s."""
    _check(dest, source, source.numel(), "reduce")
    return rt._C().reduce(_team(team), dest.data_ptr(), source.data_ptr(), source.numel(),
                          rt.dtype_code(source.dtype), op)


def fcollect(dest: torch.Tensor, source: torch.Tensor, team: Optional[rt.Team] = None) -> int:
    """All-gather: member *i*'s ``source`` lands at ``dest[i * source.numel():]`` on every member."""
    _check(dest, source, source.numel() * (team or rt.team_world()).n_pes(), "fcollect")
    return rt._C().fcollect(_team(team), dest.data_ptr(), source.data_ptr(), rt._nbytes(source))


def alltoall(dest: torch.Tensor, source: torch.Tensor, team: Optional[rt.Team] = None) -> int:
    """Member *i* sends chunk *j* of ``source`` to member *j*, which stores it as chunk *i* of ``dest``."""
    n = (team or rt.team_world()).n_pes()
    if source.numel() % n:
        raise ValueError(f"alltoall: source has {source.numel()} elements, not a multiple of {n} members")
    _check(dest, source, source.numel(), "alltoall")
    return rt._C().alltoall(_team(team), dest.data_ptr(), source.data_ptr(), rt._nbytes(source) // n)


def reduce_scatter(dest: torch.Tensor, source: torch.Tensor, op: int = rt.OP_SUM,
                   team: Optional[rt.Team] = None) -> int:
    """Member *i*'s ``dest`` (``source.numel() / n`` elements) receives block *i* of the element-wise reduction of
    all members' ``source``. Host-blocking; built from the host API (every member pulls block *i* of each peer and
    reduces it locally), so it runs on every backend. The fused GEMM -> reduce-scatter kernel is the fast path for
    tensor parallelism; this is the general-purpose form (sharded optimiser states and the like)."""
    t = team or rt.team_world()
    n, me = t.n_pes(), t.my_pe()
    if me < 0:
        return rt.ERROR
    if source.numel() % n or dest.numel() < source.numel() // n or dest.dtype != source.dtype:
        raise ValueError("reduce_scatter: source must hold n equal blocks of dest's type, dest one block")
    rt.require_symmetric(dest=dest, source=source)
    if op not in (rt.OP_SUM, rt.OP_MIN, rt.OP_MAX, rt.OP_PROD):
        raise ValueError("reduce_scatter supports sum, min, max and prod")
    blk = source.numel() // n
    world = rt.team_world()
    if t.sync() != rt.SUCCESS:                         # every member's source is complete
        return rt.ERROR
    mine = source.view(-1)[me * blk:(me + 1) * blk]
    wide = torch.float64 if source.dtype.is_floating_point else torch.int64
    acc = mine.to(wide).clone()
    tmp = torch.empty(blk, dtype=source.dtype, device=source.device)
    for d in range(1, n):
        peer = (me + d) % n
        rt.getmem(tmp, mine, t.translate_pe(peer, world))
        v = tmp.to(wide)
        acc = {rt.OP_SUM: torch.add, rt.OP_PROD: torch.mul, rt.OP_MIN: torch.minimum, rt.OP_MAX: torch.maximum}[op](acc, v)
    dest.view(-1)[:blk].copy_(acc.to(dest.dtype))
    return t.sync()                                    # nobody overwrites its source while a peer still reads it


def allgather(dest: torch.Tensor, source: torch.Tensor, team: Optional[rt.Team] = None) -> int:
    """Alias of :func:`fcollect` under its usual name."""
    return fcollect(dest, source, team)


# ---- stream-ordered ---------------------------------------------------------------------------------------

def barrier_async(team: Optional[rt.Team] = None, stream=None) -> None:
    """Team barrier as one kernel on ``stream`` (the current stream by default)."""
    rt._C().k_barrier(_team(team), _stream(stream))


def allreduce_async(dest: torch.Tensor, source: torch.Tensor, op: int = rt.OP_SUM,
                    team: Optional[rt.Team] = None, algo: int = rt.ALLREDUCE_AUTO, stream=None) -> None:
    """Allreduce as one kernel on ``stream``; ``algo`` picks one-shot, two-shot or NVLS (``ALLREDUCE_AUTO`` by size)."""
    _check(dest, source, source.numel(), "allreduce_async")
    rt._C().k_allreduce(_team(team), dest.data_ptr(), source.data_ptr(), source.numel(),
                        rt.dtype_code(source.dtype), op, algo, _stream(stream))


def broadcast_async(dest: torch.Tensor, source: torch.Tensor, root: int, team: Optional[rt.Team] = None,
                    stream=None, pre_sync: bool = True) -> None:
    """Broadcast from ``root`` as one kernel on ``stream``; the root's ``dest`` is left untouched."""
    _check(dest, source, source.numel(), "broadcast_async")
    rt._C().k_broadcast(_team(team), dest.data_ptr(), source.data_ptr(), rt._nbytes(source), root,
                        _stream(stream), rt.COLL_PRE_SYNC if pre_sync else 0)


def fcollect_async(dest: torch.Tensor, source: torch.Tensor, team: Optional[rt.Team] = None, stream=None,
                   pre_sync: bool = True) -> None:
    """All-gather as one kernel on ``stream``: block ``i`` of ``dest`` receives PE ``i``'s ``source``."""
    _check(dest, source, source.numel() * (team or rt.team_world()).n_pes(), "fcollect_async")
    rt._C().k_fcollect(_team(team), dest.data_ptr(), source.data_ptr(), rt._nbytes(source),
                       _stream(stream), rt.COLL_PRE_SYNC if pre_sync else 0)


def alltoall_async(dest: torch.Tensor, source: torch.Tensor, team: Optional[rt.Team] = None, stream=None,
                   pre_sync: bool = True) -> None:
    """All-to-all as one kernel on ``stream``: block ``j`` of ``source`` goes to PE ``j``, stored at block ``my_pe``."""
    n = (team or rt.team_world()).n_pes()
    if source.numel() % n:
        raise ValueError(f"alltoall_async: source has {source.numel()} elements, not a multiple of {n} members")
    _check(dest, source, source.numel(), "alltoall_async")
    rt._C().k_alltoall(_team(team), dest.data_ptr(), source.data_ptr(), rt._nbytes(source) // n,
                       _stream(stream), rt.COLL_PRE_SYNC if pre_sync else 0)
