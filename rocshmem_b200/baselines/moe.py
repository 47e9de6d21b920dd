"""NCCL all-to-all version of :class:`rocshmem_b200.models.MoEFeedForward` (same weights): tokens are
replicated per selected expert, sorted by destination rank, exchanged with ``all_to_all_single`` (bf16, no
de-duplication per rank), run through per-expert cuBLAS GEMMs, sent back and summed with the gate weights."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.moe_ffn import expert_weights


class NcclMoEFeedForward:
    """The MoE feed-forward layer over NCCL all-to-all and per-expert cuBLAS GEMMs (same weights)."""

    def __init__(self, num_experts: int, top_k: int, hidden: int, inter: int, seed: int = 0, group=None):
        self.group = group
        self.P, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.K, self.hidden, self.inter = num_experts, top_k, hidden, inter
        self.e_local = num_experts // self.P
        dev = torch.device("cuda", torch.cuda.current_device())
        ws = [expert_weights(self.rank * self.e_local + e, hidden, inter, seed) for e in range(self.e_local)]
        self.w13 = [w[0].to(dev) for w in ws]
        self.w2 = [w[1].to(dev) for w in ws]

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """Replicate tokens per expert, exchange, per-expert SwiGLU feed-forward, exchange back, weighted sum."""
        T = x.shape[0]
        flat_e = topk_idx.reshape(-1).long()
        valid = flat_e >= 0
        tok = torch.arange(T, device=x.device).repeat_interleave(self.K)[valid]
        e = flat_e[valid]
        w = topk_weights.reshape(-1)[valid]
        order = torch.argsort(e, stable=True)                     # by global expert = by rank, then expert
        tok, e, w = tok[order], e[order], w[order]
        send_counts = torch.bincount(e // self.e_local, minlength=self.P)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv_x = torch.empty((sum(rc), self.hidden), dtype=x.dtype, device=x.device)
        recv_e = torch.empty(sum(rc), dtype=torch.long, device=x.device)
        dist.all_to_all_single(recv_x, x[tok].contiguous(), rc, sc, group=self.group)
        dist.all_to_all_single(recv_e, e.contiguous(), rc, sc, group=self.group)
        local_e = recv_e - self.rank * self.e_local
        y = torch.empty_like(recv_x)
        for le in range(self.e_local):
            rows = (local_e == le).nonzero(as_tuple=True)[0]
            if rows.numel() == 0:
                continue
            hc = recv_x[rows] @ self.w13[le].t()
            h = torch.nn.functional.silu(hc[:, :self.inter]) * hc[:, self.inter:]
            y[rows] = h @ self.w2[le].t()
        back = torch.empty((tok.numel(), self.hidden), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(back, y, sc, rc, group=self.group)
        out = torch.zeros((T, self.hidden), dtype=torch.float32, device=x.device)
        out.index_add_(0, tok, back.float() * w.unsqueeze(1))
        return out.to(x.dtype)

    __call__ = forward
