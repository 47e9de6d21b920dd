"""Expert-parallel dispatch / combine over ``torch.distributed`` all-to-all (NCCL on GPUs, gloo on CPUs): the
library baseline that :class:`rocshmem_b200.ops.moe.EpDispatcher` is measured against.

Same traffic as the fused kernels: a token travels once to every rank that hosts one of its experts (not once per
expert), as e4m3 with one fp32 scale per 128 elements plus its routing record, and results come back as bf16 and
are summed per token with the gate weights. What the baseline cannot do is fuse: quantisation, packing by
destination, the count exchange, three payload exchanges and the weighted sum are separate kernels and separate
collectives, and the host has to read the counts before it can size the receive buffers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import moe


@dataclass
class NcclDispatchResult:
    recv_x: torch.Tensor          # [R, hidden] float8_e4m3fn (bf16 without quantisation)
    recv_scales: torch.Tensor     # [R, hidden / 128] fp32
    local_expert_idx: torch.Tensor  # [R, K] int32, -1 where the expert lives elsewhere
    gate_weights: torch.Tensor    # [R, K] fp32
    src_token: torch.Tensor       # [R] int32 (index on the source rank)
    recv_counts: list             # rows per source rank


class NcclEpDispatcher:
    """Dispatch / combine with the traffic of ``EpDispatcher`` over ``all_to_all_single``."""

    def __init__(self, num_experts: int, top_k: int, hidden: int, group=None, quantize: bool = True):
        self.group = group
        self.P, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if num_experts % self.P or hidden % 128:
            raise ValueError("num_experts must divide by the world size and hidden by 128")
        self.E, self.K, self.hidden = num_experts, top_k, hidden
        self.epr = num_experts // self.P
        self.quantize = quantize
        self.collectives = 0              # all-to-all calls issued so far
        self._tok: Optional[torch.Tensor] = None
        self._dst: Optional[torch.Tensor] = None
        self._sc: Optional[list] = None
        self._rc: Optional[list] = None

    def _a2a(self, out: torch.Tensor, inp: torch.Tensor, out_split=None, in_split=None) -> None:
        dist.all_to_all_single(out, inp, out_split, in_split, group=self.group)
        self.collectives += 1

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> NcclDispatchResult:
        """Count exchange, then rows, scales and routing records in three all-to-all calls."""
        P, K, epr, dev = self.P, self.K, self.epr, x.device
        idx = topk_idx.long()
        rank_of = torch.where(idx >= 0, idx // epr, torch.full_like(idx, -1))                  # [T, K]
        goes = (rank_of.unsqueeze(2) == torch.arange(P, device=dev).view(1, 1, P)).any(dim=1)   # [T, P]
        pairs = goes.t().nonzero()                    # (destination, token), sorted by destination then token
        dst, tok = pairs[:, 0], pairs[:, 1]
        send_counts = goes.sum(dim=0)
        recv_counts = torch.empty_like(send_counts)
        self._a2a(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()      # the host must know the sizes: one sync
        R = sum(rc)
        # payload
        if self.quantize:
            q, scales = moe.ref_quantize_1x128(x)
            send_x = q.view(torch.uint8)[tok].contiguous()
            recv_x = torch.empty((R, self.hidden), dtype=torch.uint8, device=dev)
        else:
            scales = torch.zeros((x.shape[0], self.hidden // 128), dtype=torch.float32, device=dev)
            send_x = x[tok].contiguous()
            recv_x = torch.empty((R, self.hidden), dtype=x.dtype, device=dev)
        self._a2a(recv_x, send_x, rc, sc)
        recv_s = torch.empty((R, self.hidden // 128), dtype=torch.float32, device=dev)
        self._a2a(recv_s, scales.float()[tok].contiguous(), rc, sc)
        # routing record: K local expert ids, K gate weights (bit pattern), source token
        local = torch.where(rank_of[tok] == dst.unsqueeze(1), idx[tok] % epr, torch.full_like(idx[tok], -1))
        rec = torch.empty((tok.numel(), 2 * K + 1), dtype=torch.int32, device=dev)
        rec[:, :K] = local.to(torch.int32)
        rec[:, K:2 * K] = topk_weights.float()[tok].contiguous().view(torch.int32)
        rec[:, 2 * K] = tok.to(torch.int32)
        recv_rec = torch.empty((R, 2 * K + 1), dtype=torch.int32, device=dev)
        self._a2a(recv_rec, rec, rc, sc)
        self._tok, self._dst, self._sc, self._rc = tok, dst, sc, rc
        rx = recv_x.view(torch.float8_e4m3fn) if self.quantize else recv_x
        return NcclDispatchResult(rx, recv_s, recv_rec[:, :K], recv_rec[:, K:2 * K].contiguous().view(torch.float32),
                                  recv_rec[:, 2 * K], rc)

    def combine(self, y: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, num_tokens: int,
                weighted: bool = True) -> torch.Tensor:
        """``y``: one bf16 result row per received row, in the order of the dispatch. Returns [num_tokens, hidden]."""
        if self._tok is None:
            raise RuntimeError("combine before dispatch")
        tok, dst = self._tok, self._dst
        back = torch.empty((tok.numel(), self.hidden), dtype=y.dtype, device=y.device)
        self._a2a(back, y[:sum(self._rc)].contiguous(), self._sc, self._rc)
        if weighted:
            idx = topk_idx.long()
            rank_of = torch.where(idx >= 0, idx // self.epr, torch.full_like(idx, -1))
            gate = ((rank_of[tok] == dst.unsqueeze(1)).float() * topk_weights.float()[tok]).sum(dim=1, keepdim=True)
        else:
            gate = torch.ones((tok.numel(), 1), dtype=torch.float32, device=y.device)
        out = torch.zeros((num_tokens, self.hidden), dtype=torch.float32, device=y.device)
        out.index_add_(0, tok, back.float() * gate)
        return out.to(torch.bfloat16)
