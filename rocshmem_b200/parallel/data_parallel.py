"""Data-parallel gradient averaging on the symmetric heap.

Gradients are packed into a few large symmetric buckets and all-reduced over the data-parallel team with the
library's allreduce kernel. Through NVSwitch the cost of an allreduce does not depend on the number of links, so
buckets are sized for launch latency and overlap (tens of MiB), not for link count; each bucket's allreduce is
enqueued on a communication stream as soon as its last gradient has been produced, so it overlaps the rest of the
backward pass. The reference offers the primitive this is built on, the block-level ``*_wg_reduce``
(``include/rocshmem/rocshmem_COLL.hpp:333-603``), and nothing above it.

    dp = GradientBuckets(model.parameters(), team=layout.dp_team, bucket_bytes=64 << 20)
    loss.backward()            # hooks copy each gradient into its bucket and start full buckets
    dp.finish()                # wait, average, copy back into p.grad

On the CPU backend the same packing runs with the host-blocking reduction, which is what the multi-process CPU
tests exercise.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from .. import runtime as rt
from ..ops import collectives as coll


class _Bucket:
    def __init__(self, dtype: torch.dtype, numel: int):
        self.send = rt.zeros(numel, dtype)
        self.recv = rt.zeros(numel, dtype)
        self.params: List[torch.nn.Parameter] = []
        self.offsets: List[int] = []
        self.pending = 0
        self.launched = False


class GradientBuckets:
    """Collective to create and to destroy: every member passes parameters of the same shapes in the same order,
    and in every step the same parameters receive gradients on every member (buckets are reduced in the order in
    which they fill up, which must agree across the team)."""

    def __init__(self, params: Iterable[torch.nn.Parameter], team: Optional[rt.Team] = None,
                 bucket_bytes: int = 64 << 20, average: bool = True, register_hooks: bool = True):
        self.team = team or rt.team_world()
        self.n = self.team.n_pes()
        self.average = average
        self.params = [p for p in params if p.requires_grad]
        self.buckets: List[_Bucket] = []
        self._where = {}
        # Parameters are packed in reverse order: the backward pass produces the last layers' gradients first.
        groups: List[List[torch.nn.Parameter]] = []
        cur: List[torch.nn.Parameter] = []
        cur_bytes, cur_dtype = 0, None
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if cur and (p.dtype != cur_dtype or cur_bytes + nbytes > bucket_bytes):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            groups.append(cur)
        for g in groups:
            # 16-byte aligned slots so that the vector paths of the kernels apply to every gradient
            align = 16 // g[0].element_size()
            offs, total = [], 0
            for p in g:
                offs.append(total)
                total += (p.numel() + align - 1) // align * align
            b = _Bucket(g[0].dtype, max(total, align))
            b.params, b.offsets = g, offs
            for p, o in zip(g, offs):
                self._where[id(p)] = (b, o)
            self.buckets.append(b)
        self._cuda = rt.is_cuda()
        self._stream = torch.cuda.Stream() if self._cuda else None
        self._hooks = []
        if register_hooks:
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
        self.reset()

    # ---- one step ------------------------------------------------------------------------------------------------

    def reset(self) -> None:
        """Forget the state of the previous step (called by :meth:`finish`)."""
        for b in self.buckets:
            b.pending = len(b.params)
            b.launched = False

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        b, off = self._where[id(p)]
        b.send[off:off + p.numel()].copy_(p.grad.reshape(-1))
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    def _launch(self, b: _Bucket) -> None:
        b.launched = True
        if self._cuda:
            # The copies into the bucket ran on the current stream; the allreduce follows them on its own stream.
            self._stream.wait_stream(torch.cuda.current_stream())
            coll.allreduce_async(b.recv, b.send, rt.OP_SUM, team=self.team, stream=self._stream)
        else:
            if coll.reduce(b.recv, b.send, rt.OP_SUM, self.team) != rt.SUCCESS:
                raise RuntimeError("gradient allreduce failed")

    def finish(self) -> None:
        """Start what has not started (parameters without hooks or without a gradient count as zeros), wait for all
        buckets and write the averaged gradients back into ``p.grad``."""
        for b in self.buckets:
            if not b.launched:
                for p, off in zip(b.params, b.offsets):
                    view = b.send[off:off + p.numel()]
                    if p.grad is None:
                        view.zero_()
                    else:                       # hooks off, or the bucket is incomplete: (re)copy what is there
                        view.copy_(p.grad.reshape(-1))
                self._launch(b)
        if self._cuda:
            torch.cuda.current_stream().wait_stream(self._stream)
        scale = 1.0 / self.n if self.average else 1.0
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                g = b.recv[off:off + p.numel()].view_as(p)
                if p.grad is None:
                    p.grad = torch.empty_like(p)
                if scale != 1.0:
                    torch.mul(g, scale, out=p.grad)
                else:
                    p.grad.copy_(g)
        self.reset()

    def destroy(self) -> None:
        """Collective: remove the hooks and free the buckets."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self._cuda:
            torch.cuda.synchronize()
        rt.free_all([t for b in self.buckets for t in (b.send, b.recv)])
        self.buckets = []
        self._where = {}
