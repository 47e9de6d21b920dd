"""NCCL + cuBLAS version of :class:`rocshmem_b200.models.TensorParallelMLP` (same weights, same shapes)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.tp_mlp import mlp_weights


class NcclTensorParallelMLP:
    """The tensor-parallel SwiGLU MLP with NCCL all-gather / reduce-scatter and cuBLAS GEMMs (same weights)."""

    def __init__(self, d_model: int, d_ff: int, m_shard: int, seed: int = 0, group=None):
        self.group = group
        P, r = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.ff = d_ff // P
        self.w_gate_up, self.w_down = mlp_weights(r, P, d_model, d_ff, seed, dev)
        self.gathered = torch.empty((P * m_shard, d_model), dtype=torch.bfloat16, device=dev)
        self.out = torch.empty((m_shard, d_model), dtype=torch.bfloat16, device=dev)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """all_gather_into_tensor, two matmuls with SwiGLU between them, reduce_scatter_tensor."""
        dist.all_gather_into_tensor(self.gathered, x_shard, group=self.group)
        hc = self.gathered @ self.w_gate_up.t()
        h = torch.nn.functional.silu(hc[:, :self.ff]) * hc[:, self.ff:]
        partial = h @ self.w_down.t()
        dist.reduce_scatter_tensor(self.out, partial, group=self.group)
        return self.out

    __call__ = forward
