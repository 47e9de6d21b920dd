"""Ring exchange for context parallelism (ring attention): every member passes a block to its right-hand neighbour
and receives one from the left, once per step.

The reference has no attention code; the building block it offers is a put followed by a remote flag update and a
``wait_until`` on the receiver (its ring allreduce is built the same way, ``src/ipc/context_ipc_tmpl_device.hpp:
282-359``). Here one step is: put the block into the neighbour's buffer for this step's parity, complete it, bump
the neighbour's arrival counter; wait until the own arrival counter reaches the step; take the block; tell the left
neighbour that the buffer of this parity is free again. Two buffers make the next step's put overlap the
consumption of this step's block.

:func:`ring_attention` uses it for exact attention over a sequence that is sharded across the team: keys and
values travel around the ring while every member accumulates its queries' output with a running maximum and sum
(the online-softmax recurrence), so no member ever holds more than two blocks of keys and values.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt


class RingExchange:
    """Collective to create and to destroy; every member calls :meth:`shift` the same number of times."""

    def __init__(self, shape, dtype: torch.dtype, team: Optional[rt.Team] = None):
        self.team = team or rt.team_world()
        self.n, self.me = self.team.n_pes(), self.team.my_pe()
        world = rt.team_world()
        self.right = self.team.translate_pe((self.me + 1) % self.n, world)
        self.left = self.team.translate_pe((self.me - 1) % self.n, world)
        self.buf = rt.zeros((2,) + tuple(shape), dtype)
        self.arrived = rt.zeros(1, torch.int64)      # blocks delivered to me
        self.released = rt.zeros(1, torch.int64)     # blocks of mine that my right-hand neighbour has taken
        self.step = 0

    def destroy(self) -> None:
        """Collective: free the buffers and counters."""
        rt.free_all([self.buf, self.arrived, self.released])
        self.buf = self.arrived = self.released = None

    def shift(self, block: torch.Tensor) -> torch.Tensor:
        """Send ``block`` to the right, return the block that arrived from the left (a new tensor)."""
        self.step += 1
        parity = self.step & 1
        # The buffer of this parity on the right was last used two steps ago: wait until that block was taken.
        if self.step > 2 and rt.wait_until(self.released, rt.CMP_GE, self.step - 2) != rt.SUCCESS:
            raise TimeoutError(f"ring: PE {self.right} did not take block {self.step - 2}")
        rt.putmem(self.buf[parity], block.contiguous(), self.right)
        rt.quiet()
        rt.atomic_fetch_add(self.arrived, 1, self.right)
        if rt.wait_until(self.arrived, rt.CMP_GE, self.step) != rt.SUCCESS:
            raise TimeoutError(f"ring: block {self.step} from PE {self.left} did not arrive")
        out = self.buf[parity].clone()
        rt.atomic_fetch_add(self.released, 1, self.left)
        return out


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ring_k: RingExchange, ring_v: RingExchange,
                   causal: bool = False) -> torch.Tensor:
    """Exact attention for this member's queries over the whole (sharded) sequence.

    ``q``, ``k``, ``v``: ``[S / n, H, D]``, member ``r`` holding positions ``[r S / n, (r + 1) S / n)``. Keys and
    values make one trip around the ring; the result is ``[S / n, H, D]`` in fp32.
    """
    n, me = ring_k.n, ring_k.me
    sl, H, D = q.shape
    qf = q.float()
    out = torch.zeros((sl, H, D), dtype=torch.float32, device=q.device)
    row_max = torch.full((H, sl), float("-inf"), device=q.device)
    row_sum = torch.zeros((H, sl), device=q.device)
    kb, vb = k, v
    for step in range(n):
        src = (me - step) % n                     # whose keys and values are here now
        if not causal or src <= me:
            scores = torch.einsum("shd,thd->hst", qf, kb.float()) / D ** 0.5
            if causal and src == me:
                scores = scores.masked_fill(torch.triu(torch.ones(sl, sl, dtype=torch.bool, device=q.device), 1),
                                            float("-inf"))
            new_max = torch.maximum(row_max, scores.amax(dim=-1))
            scale_old = torch.exp(row_max - new_max)
            p = torch.exp(scores - new_max.unsqueeze(-1))
            row_sum = row_sum * scale_old + p.sum(dim=-1)
            out = out * scale_old.t().unsqueeze(-1) + torch.einsum("hst,thd->shd", p, vb.float())
            row_max = new_max
        if step + 1 < n:
            kb, vb = ring_k.shift(kb), ring_v.shift(vb)
    return out / row_sum.t().unsqueeze(-1)
