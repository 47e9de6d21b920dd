"""Sequence-parallel attention re-sharding with all-to-all (the DeepSpeed-Ulysses pattern).

Outside attention every rank of the team holds a slice of the sequence with all heads, ``[S / n, H, D]``; attention
wants whole sequences, so it runs on a slice of the heads, ``[S, H / n, D]``. The two layouts are one all-to-all
apart in each direction. The reference has no sequence dimension anywhere; what it provides is the fixed-size
block-level ``alltoall`` (``src/ipc/context_ipc_tmpl_device.hpp:474-501``), which is exactly the primitive used
here: block ``j`` of the send buffer goes to member ``j`` and lands there as block ``my_pe``.

    sp = UlyssesResharder(seq_len=S, heads=H, head_dim=D, dtype=torch.bfloat16, team=layout.inner_team)
    q_heads = sp.seq_to_heads(q_seq)        # [S / n, H, D] -> [S, H / n, D]
    o_seq = sp.heads_to_seq(o_heads)        # [S, H / n, D] -> [S / n, H, D]

On GPUs the exchange is the library's stream-ordered all-to-all kernel; on the CPU backend the host-blocking form.
The packing before and after it is a permute of the local tensor.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt
from ..ops import collectives as coll


class UlyssesResharder:
    """Symmetric send / receive buffers for one (sequence length, heads, head dimension, dtype) shape; collective
    to create and to destroy."""

    def __init__(self, seq_len: int, heads: int, head_dim: int, dtype: torch.dtype = torch.bfloat16,
                 team: Optional[rt.Team] = None):
        self.team = team or rt.team_world()
        n = self.team.n_pes()
        if seq_len % n or heads % n:
            raise ValueError("sequence length and number of heads must be divisible by the team size")
        self.n, self.S, self.H, self.D, self.dtype = n, seq_len, heads, head_dim, dtype
        self.s_local, self.h_local = seq_len // n, heads // n
        numel = self.s_local * heads * head_dim          # == seq_len * h_local * head_dim
        self.send = rt.zeros(numel, dtype)
        self.recv = rt.zeros(numel, dtype)
        self._cuda = rt.is_cuda()

    def destroy(self) -> None:
        """Collective: free the two buffers."""
        if self._cuda:
            torch.cuda.synchronize()
        rt.free_all([self.send, self.recv])
        self.send = self.recv = None

    def _exchange(self, stream) -> None:
        if self._cuda:
            coll.alltoall_async(self.recv, self.send, team=self.team, stream=stream)
        elif coll.alltoall(self.recv, self.send, self.team) != rt.SUCCESS:
            raise RuntimeError("all-to-all failed")

    def seq_to_heads(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        """``x [S / n, H, D]`` (my part of the sequence, all heads) -> ``[S, H / n, D]`` (whole sequence, my heads).
        Returns a new tensor. Runs on the current stream unless ``stream`` is given (then the caller orders the
        packing copy, which runs on the current stream, before it)."""
        n, sl, hl, D = self.n, self.s_local, self.h_local, self.D
        if tuple(x.shape) != (sl, self.H, D) or x.dtype != self.dtype:
            raise ValueError(f"expected [{sl}, {self.H}, {D}] {self.dtype}")
        # block j: my sequence slice, heads of member j
        self.send.view(n, sl, hl, D).copy_(x.view(sl, n, hl, D).permute(1, 0, 2, 3))
        self._exchange(stream)
        # block i of recv: member i's sequence slice, my heads -> already in sequence order
        return self.recv.view(self.S, hl, D).clone()

    def heads_to_seq(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        """``x [S, H / n, D]`` (whole sequence, my heads) -> ``[S / n, H, D]`` (my part of the sequence, all heads).
        Returns a new tensor."""
        n, sl, hl, D = self.n, self.s_local, self.h_local, self.D
        if tuple(x.shape) != (self.S, hl, D) or x.dtype != self.dtype:
            raise ValueError(f"expected [{self.S}, {hl}, {D}] {self.dtype}")
        # block j: sequence slice of member j, my heads
        self.send.view(self.S, hl, D).copy_(x)
        self._exchange(stream)
        # block i of recv: my sequence slice, heads of member i
        return self.recv.view(n, sl, hl, D).permute(1, 0, 2, 3).reshape(sl, self.H, D)
