"""Snapshot and restore of symmetric-heap tensors.

The runtime itself holds only transient communication state (like the reference, which has no checkpoint
support); what an application may want to keep across a restart is the content of its heap-resident tensors.
These helpers copy named symmetric tensors of this PE to host memory and back. Restoring is collective in
spirit: every PE restores its own copy, then all synchronise before anybody reads a peer.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import runtime as rt


def snapshot(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Host copies of this PE's view of the given symmetric tensors (synchronises the device)."""
    if rt.is_cuda():
        torch.cuda.synchronize()
    return {name: t.detach().to("cpu", copy=True) for name, t in tensors.items()}


def restore(tensors: Dict[str, torch.Tensor], saved: Dict[str, torch.Tensor], barrier: bool = True) -> None:
    """Writes ``saved`` back into the symmetric tensors of the same names; shapes and dtypes must match."""
    for name, t in tensors.items():
        if name not in saved:
            raise KeyError(f"no saved tensor named {name!r}")
        s = saved[name]
        if tuple(s.shape) != tuple(t.shape) or s.dtype != t.dtype:
            raise ValueError(f"{name}: saved {tuple(s.shape)} {s.dtype} does not match {tuple(t.shape)} {t.dtype}")
        t.copy_(s.to(t.device))
    if rt.is_cuda():
        torch.cuda.synchronize()
    if barrier:
        rt.barrier_all()


def save(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """:func:`snapshot` written with ``torch.save`` (one file per PE: the caller chooses the path)."""
    torch.save(snapshot(tensors), path)


def load(path: str, tensors: Dict[str, torch.Tensor], barrier: bool = True) -> None:
    """Read a file written by ``save`` and ``restore`` it into the given symmetric tensors."""
    restore(tensors, torch.load(path, map_location="cpu"), barrier=barrier)
