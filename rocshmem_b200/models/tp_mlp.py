"""Tensor-parallel SwiGLU MLP block with sequence-parallel activations.

Every rank holds ``x_shard [m_shard, d_model]`` (rows ``rank * m_shard ...`` of the token matrix), the
column shard ``w_gate_up [2 * ff_local, d_model]`` of the up projection (gate rows first, then up rows)
and the row shard ``w_down [d_model, ff_local]`` of the down projection. One forward is two kernels::

    all-gather(x) -> GEMM -> silu(gate) * up          one launch, transfer overlapped tile by tile
    GEMM -> reduce-scatter                            one launch, epilogue stores to the owners' staging

The reference ships no model code; the collectives it would be assembled from are fcollect and the
reductions (src/ipc/context_ipc_tmpl_device.hpp:166-531).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt
from ..ops import gemm
from ..utils.trace import traced
from ..ops.gemm import TensorParallelLinear


def mlp_weights(rank: int, n_ranks: int, d_model: int, d_ff: int, seed: int = 0, device="cpu"):
    """Deterministic shards of rank ``rank``: ``w_gate_up [2 * d_ff / n_ranks, d_model]`` and
    ``w_down [d_model, d_ff / n_ranks]``, bf16."""
    ff = d_ff // n_ranks
    g = torch.Generator().manual_seed(seed * 7919 + rank)
    w1 = (torch.randn(2 * ff, d_model, generator=g) * d_model ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(d_model, ff, generator=g) * d_ff ** -0.5).to(torch.bfloat16)
    return w1.to(device), w2.to(device)


class TensorParallelMLP:
    """SwiGLU MLP with weights sharded over the team: all-gather -> up projection, down projection -> reduce-scatter, two fused kernels."""

    def __init__(self, d_model: int, d_ff: int, m_shard: int, team: Optional[rt.Team] = None, seed: int = 0):
        self.tp = TensorParallelLinear(m_shard, team=team)
        P = self.tp.n_ranks
        if d_ff % P:
            raise ValueError("d_ff must be divisible by the team size")
        self.d_model, self.d_ff, self.ff_local, self.m_shard = d_model, d_ff, d_ff // P, m_shard
        dev = rt.device()
        self.w_gate_up, self.w_down = mlp_weights(self.tp.team.my_pe(), P, d_model, d_ff, seed, dev)
        self.h = torch.empty((P * m_shard, self.ff_local), dtype=torch.bfloat16, device=dev)

    def input_buffer(self) -> torch.Tensor:
        """Symmetric ``[m_shard, d_model]`` buffer: writing the activations here saves the copy in
        :meth:`forward`."""
        return self.tp.ag_input(self.d_model)

    def destroy(self) -> None:
        """Collective: free the symmetric gather / staging buffers (the weights are ordinary tensors)."""
        self.tp.destroy()

    @traced("rocshmem_b200.tp_mlp")
    def forward(self, x_shard: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                stream=None) -> torch.Tensor:
        """Returns this rank's ``[m_shard, d_model]`` rows of the MLP output. ``x_shard=None`` uses
        the current content of :meth:`input_buffer`."""
        if x_shard is not None:
            self.input_buffer().copy_(x_shard)
        self.tp.ag_gemm(self.w_gate_up, out=self.h, swiglu=True, stream=stream)
        return self.tp.gemm_rs(self.h, self.w_down, out=out, stream=stream)

    __call__ = forward

    @property
    def kernel_launches(self) -> int:
        """Kernels launched by this object so far."""
        return self.tp.kernel_launches


class TensorParallelMLPFp8:
    """The same block with block-scaled e4m3 GEMMs: activations are quantised 1 x 128 (the input shard before
    the all-gather, the hidden activation before the down projection), weights 128 x 128. Four kernels per
    forward: quantise, all-gather -> GEMM -> SwiGLU, quantise, GEMM -> reduce-scatter."""

    def __init__(self, d_model: int, d_ff: int, m_shard: int, team: Optional[rt.Team] = None, seed: int = 0):
        self.tp = gemm.TensorParallelLinearFp8(m_shard, team=team)
        P = self.tp.n_ranks
        if d_ff % P or (d_ff // P) % 512 or d_model % 512:
            raise ValueError("d_model and d_ff / n_ranks must be multiples of 512")
        self.d_model, self.d_ff, self.ff_local, self.m_shard = d_model, d_ff, d_ff // P, m_shard
        dev = rt.device()
        w1, w2 = mlp_weights(self.tp.team.my_pe(), P, d_model, d_ff, seed, dev)
        self.w1_q, self.w1_s = gemm.quantize_weight_128x128(w1)
        self.w2_q, self.w2_s = gemm.quantize_weight_128x128(w2)
        M = P * m_shard
        self.h = torch.empty((M, self.ff_local), dtype=torch.bfloat16, device=dev)
        self.h_q = torch.empty((M, self.ff_local), dtype=torch.uint8, device=dev)
        self.h_s = torch.empty((M, self.ff_local // 128), dtype=torch.float32, device=dev)

    def destroy(self) -> None:
        """Collective: free the symmetric gather / staging buffers (the weights are ordinary tensors)."""
        self.tp.destroy()

    @traced("rocshmem_b200.tp_mlp_fp8")
    def forward(self, x_shard: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """Quantise the shard, all-gather -> up projection with SwiGLU, quantise, down projection -> reduce-scatter."""
        self.tp.set_input(x_shard, stream)
        self.tp.ag_gemm(self.w1_q, self.w1_s, out=self.h, swiglu=True, stream=stream)
        gemm.quantize_1x128_into(self.h, self.h_q, self.h_s, stream)
        self.tp.kernel_launches += 1
        return self.tp.gemm_rs(self.h_q, self.h_s, self.w2_q, self.w2_s, out=out, stream=stream)

    __call__ = forward

    @property
    def kernel_launches(self) -> int:
        """Kernels launched by this object so far."""
        return self.tp.kernel_launches


def reference_forward_fp8(x_full: torch.Tensor, n_ranks: int, d_model: int, d_ff: int, seed: int = 0) -> torch.Tensor:
    """fp32 evaluation of :class:`TensorParallelMLPFp8` with the same quantisation points."""
    from ..ops import moe
    q, s = moe.ref_quantize_1x128(x_full.cpu())
    x = moe.ref_dequantize_1x128(q, s).float()
    out = torch.zeros(x.shape[0], d_model)
    ff = d_ff // n_ranks
    for r in range(n_ranks):
        w1, w2 = mlp_weights(r, n_ranks, d_model, d_ff, seed)
        w1d = gemm.dequantize_weight_128x128(*gemm.quantize_weight_128x128(w1))
        w2d = gemm.dequantize_weight_128x128(*gemm.quantize_weight_128x128(w2))
        hc = x @ w1d.t()
        h = (torch.nn.functional.silu(hc[:, :ff]) * hc[:, ff:]).to(torch.bfloat16)
        hq, hs = moe.ref_quantize_1x128(h)
        out += (moe.ref_dequantize_1x128(hq, hs).float() @ w2d.t()).to(torch.bfloat16).float()
    return out


def reference_forward(x_full: torch.Tensor, n_ranks: int, d_model: int, d_ff: int, seed: int = 0) -> torch.Tensor:
    """Plain PyTorch fp32 evaluation on the full token matrix (all shards rebuilt locally); the hidden
    activation and each rank's partial product are rounded to bf16 where the kernels store bf16."""
    x = x_full.float().cpu()
    out = torch.zeros(x.shape[0], d_model)
    ff = d_ff // n_ranks
    for r in range(n_ranks):
        w1, w2 = mlp_weights(r, n_ranks, d_model, d_ff, seed)
        hc = x @ w1.float().t()
        h = (torch.nn.functional.silu(hc[:, :ff]) * hc[:, ff:]).to(torch.bfloat16).float()
        out += (h @ w2.float().t()).to(torch.bfloat16).float()
    return out
