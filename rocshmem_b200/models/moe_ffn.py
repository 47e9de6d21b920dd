"""Expert-parallel MoE feed-forward layer (SwiGLU experts) built from this package's kernels.

One call runs, stream-ordered and without a host synchronisation, as four kernels (plus a memset-like one on a
side stream)::

    dispatch       fp8 1x128 rows over NVLink; its tail groups the received (row, k) pairs by local expert
    gate/up GEMM   grouped tcgen05 GEMM whose producer warps gather the received rows by index (de-quantising
                   e4m3 to bf16 on the way into shared memory), SwiGLU in the epilogue
    down GEMM      grouped tcgen05 GEMM whose epilogue multiplies every row by its gate weight and adds it into
                   the row's slot of the result buffer (the sum over a token's local experts)
    combine        pull over NVLink, sum over the ranks a token went to

With ``fp8_experts`` both GEMMs are block-scaled e4m3: the received e4m3 rows and their scales are gathered as they
are, and the first GEMM's epilogue quantises the hidden activation for the second. ``fused=False`` keeps the
separate gather, quantise and per-row reduction kernels.

Experts are sharded over the team: rank r owns global experts ``[r * E_local, (r + 1) * E_local)``.
The reference has no model code; its nearest building block is the fixed-size alltoall
(src/ipc/context_ipc_tmpl_device.hpp:474-501).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt
from ..ops import gemm, moe
from ..utils.trace import traced


def expert_weights(expert: int, hidden: int, inter: int, seed: int = 0, device="cpu"):
    """Deterministic random weights of one global expert: ``w13 [2 * inter, hidden]`` (gate rows first,
    then up rows) and ``w2 [hidden, inter]``, bf16. Any rank can rebuild any expert from its id."""
    g = torch.Generator().manual_seed(seed * 100003 + expert)
    w13 = (torch.randn(2 * inter, hidden, generator=g) * hidden ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(hidden, inter, generator=g) * inter ** -0.5).to(torch.bfloat16)
    return w13.to(device), w2.to(device)


class MoEFeedForward:
    """``num_experts`` SwiGLU experts of shape hidden -> inter -> hidden, top-k routing done by the caller.

    ``pair_capacity`` bounds the number of (row, expert) pairs this rank can process in one call; the
    default is the worst case ``n_ranks * max_tokens * top_k``. With balanced routing the expected number
    is ``max_tokens * top_k``, and a tighter bound saves memory; exceeding it is the caller's error.
    """

    def __init__(self, num_experts: int, top_k: int, hidden: int, inter: int, max_tokens: int,
                 team: Optional[rt.Team] = None, quantize: bool = True, layout: str = "compact", seed: int = 0,
                 pair_capacity: Optional[int] = None, fp8_experts: bool = False, fused: Optional[bool] = None,
                 low_latency: bool = False):
        if rt.n_local_pes() != 1:
            raise RuntimeError("MoEFeedForward needs one PE per process")
        self.fused = (hidden % 128 == 0) if fused is None else bool(fused)
        if self.fused and hidden % 128:
            raise ValueError("the fused path needs hidden % 128 == 0")
        self.d = moe.EpDispatcher(num_experts, top_k, hidden, max_tokens, team=team, quantize=quantize, layout=layout,
                                  expert_layout=self.fused, low_latency=low_latency)
        self.hidden, self.inter, self.top_k = hidden, inter, top_k
        self.n_ranks, self.e_local = self.d.n_ranks, self.d.experts_per_rank
        dev = rt.device()
        first = self.d.team.my_pe() * self.e_local
        ws = [expert_weights(first + e, hidden, inter, seed) for e in range(self.e_local)]
        self.w13 = torch.stack([w[0] for w in ws]).to(dev).contiguous()   # [E_local, 2 * inter, hidden]
        self.w2 = torch.stack([w[1] for w in ws]).to(dev).contiguous()    # [E_local, hidden, inter]
        cap = pair_capacity or self.n_ranks * max_tokens * top_k
        self.pair_capacity = cap
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.h = torch.zeros((cap, inter), **bf)        # silu(gate) * up
        if self.fused:
            self.side = torch.cuda.Stream()
            self.ev_dispatched, self.ev_zeroed = torch.cuda.Event(), torch.cuda.Event()
        else:
            self.xs = torch.zeros((cap, hidden), **bf)      # rows in expert order
            self.yp = torch.zeros((cap, hidden), **bf)      # expert outputs per pair
            self.inverse = torch.zeros(self.n_ranks * max_tokens * top_k, dtype=torch.int32, device=dev)
        self.kernel_launches = 0
        # Block-scaled e4m3 experts: the received e4m3 rows feed the first grouped GEMM as they are (no
        # de-quantisation), the hidden activation is re-quantised for the second one.
        self.fp8_experts = bool(fp8_experts)
        if self.fp8_experts:
            if not quantize or hidden % 1024 or inter % 512:
                raise ValueError("fp8 experts need an fp8 dispatch, hidden % 1024 == 0 and inter % 512 == 0")
            self.w13_q, self.w13_s = gemm.quantize_weight_128x128(self.w13)
            self.w2_q, self.w2_s = gemm.quantize_weight_128x128(self.w2)
            if not self.fused:
                self.xs_q = torch.zeros((cap, hidden), dtype=torch.uint8, device=dev)
                self.xs_s = torch.zeros((cap, hidden // 128), dtype=torch.float32, device=dev)
            self.h_q = torch.zeros((cap, inter), dtype=torch.uint8, device=dev)
            self.h_s = torch.zeros((cap, inter // 128), dtype=torch.float32, device=dev)

    def destroy(self) -> None:
        """Collective: free the dispatcher's symmetric buffers (the weights and work buffers are ordinary tensors)."""
        self.d.destroy()

    @traced("rocshmem_b200.moe_feed_forward")
    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                out: Optional[torch.Tensor] = None, stream=None, stage_us: Optional[dict] = None) -> torch.Tensor:
        """x [T, hidden] bf16, topk_idx [T, top_k] int32 global expert ids (-1 = unused), topk_weights
        [T, top_k] fp32. Returns [T, hidden] bf16: sum_k w_k * expert_k(x).

        With ``stage_us`` (a dict) the call synchronises and fills it with the device time of every stage in
        microseconds (for profiling; the stages then run back to back without overlap of their launches)."""
        C = rt._C()
        d = self.d
        s = moe._stream(stream)
        before = d.kernel_launches
        marks = []

        def mark(name):
            if stage_us is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        d.dispatch(x, topk_idx, topk_weights, stream=stream)
        mark("dispatch")
        if self.fused:
            cur = torch.cuda.ExternalStream(stream) if isinstance(stream, int) else (stream or torch.cuda.current_stream())
            offsets, lay_row, _, lay_w = d.expert_pairs()
            y = d.result_buffer()
            # The result rows start from zero; clearing them runs beside the first GEMM.
            self.ev_dispatched.record(cur)
            self.side.wait_event(self.ev_dispatched)
            C.moe_zero_rows(d.recv_info.data_ptr(), self.n_ranks, self.hidden, y.data_ptr(), self.side.cuda_stream)
            self.ev_zeroed.record(self.side)
            if self.fp8_experts:
                # Received e4m3 rows and their scales feed the first GEMM as they are; its epilogue quantises the
                # hidden activation for the second one.
                gemm.grouped_gemm_fp8_swiglu_quant(d.recv_x, d.recv_scales, self.w13_q, self.w13_s, offsets, self.h_q,
                                                   self.h_s, row_index=lay_row, stream=stream)
                mark("gemm_gate_up")
                cur.wait_event(self.ev_zeroed)
                gemm.grouped_gemm_fp8_scatter_add(self.h_q, self.h_s, self.w2_q, self.w2_s, offsets, lay_row, y,
                                                  weights=lay_w, stream=stream)
            else:
                gemm.grouped_gemm_bf16_gathered(d.recv_x, lay_row, self.w13, offsets,
                                                a_scales=d.recv_scales if d.quantize else None, swiglu=True,
                                                out=self.h, stream=stream)
                mark("gemm_gate_up")
                cur.wait_event(self.ev_zeroed)
                gemm.grouped_gemm_bf16_scatter_add(self.h, self.w2, offsets, lay_row, y, weights=lay_w, stream=stream)
            mark("gemm_down")
            out = d.combine(y, topk_idx, topk_weights, x.shape[0], weighted=False, out=out, stream=stream)
            mark("combine")
            self.kernel_launches += (d.kernel_launches - before) + 3
            if stage_us is not None:
                torch.cuda.synchronize()
                for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                    stage_us[name] = a.elapsed_time(b) * 1e3
            return out
        offsets, row_index, pair_k = d.expert_layout(stream=stream)
        C.moe_inverse_map(offsets.data_ptr(), self.e_local, row_index.data_ptr(), pair_k.data_ptr(), self.top_k,
                          self.inverse.data_ptr(), s)
        mark("layout")
        if self.fp8_experts:
            # Rows and their scales are copied as raw bytes (the gather kernel's 2-byte element view).
            C.moe_gather_rows(d.recv_x.data_ptr(), 0, 0, offsets.data_ptr(), self.e_local, row_index.data_ptr(),
                              self.hidden // 2, self.xs_q.data_ptr(), s)
            C.moe_gather_rows(d.recv_scales.data_ptr(), 0, 0, offsets.data_ptr(), self.e_local,
                              row_index.data_ptr(), self.hidden // 128 * 2, self.xs_s.data_ptr(), s)
            mark("gather")
            gemm.grouped_gemm_fp8_blockscaled(self.xs_q, self.xs_s, self.w13_q, self.w13_s, offsets, swiglu=True,
                                              out=self.h, stream=stream)
            mark("gemm_gate_up")
            gemm.quantize_1x128_into(self.h, self.h_q, self.h_s, stream)
            mark("quantize_hidden")
            gemm.grouped_gemm_fp8_blockscaled(self.h_q, self.h_s, self.w2_q, self.w2_s, offsets, out=self.yp,
                                              stream=stream)
            mark("gemm_down")
            self.kernel_launches += 2
        else:
            C.moe_gather_rows(d.recv_x.data_ptr(), d.recv_scales.data_ptr(), int(d.quantize), offsets.data_ptr(),
                              self.e_local, row_index.data_ptr(), self.hidden, self.xs.data_ptr(), s)
            mark("gather")
            gemm.grouped_gemm_bf16(self.xs, self.w13, offsets, swiglu=True, out=self.h, stream=stream)
            mark("gemm_gate_up")
            gemm.grouped_gemm_bf16(self.h, self.w2, offsets, out=self.yp, stream=stream)
            mark("gemm_down")
        y = d.result_buffer()
        C.moe_reduce_pairs(self.yp.data_ptr(), self.inverse.data_ptr(), d.recv_meta.data_ptr(),
                           d.recv_info.data_ptr(), self.n_ranks, self.top_k, self.hidden, 1, y.data_ptr(), s)
        mark("reduce_pairs")
        out = d.combine(y, topk_idx, topk_weights, x.shape[0], weighted=False, out=out, stream=stream)
        mark("combine")
        self.kernel_launches += (d.kernel_launches - before) + 5
        if stage_us is not None:
            torch.cuda.synchronize()
            for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                stage_us[name] = a.elapsed_time(b) * 1e3
        return out

    __call__ = forward


def reference_forward(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, hidden: int, inter: int,
                      seed: int = 0, quantize: bool = True, fp8_experts: bool = False) -> torch.Tensor:
    """Plain PyTorch fp32 evaluation of the same layer for the tokens of one rank (all experts rebuilt
    locally). With ``quantize`` the input passes through the same 1x128 e4m3 quantisation as dispatch.
    The intermediate activations are rounded to bf16 where the kernels store bf16."""
    xin = x.float().cpu()
    if quantize:
        q, sc = moe.ref_quantize_1x128(x.cpu())
        xin = moe.ref_dequantize_1x128(q, sc).float()
    if not fp8_experts:
        xin = xin.to(torch.bfloat16).float()
    idx, w = topk_idx.cpu(), topk_weights.cpu()
    out = torch.zeros(x.shape[0], hidden)
    for e in idx[idx >= 0].unique().tolist():
        w13, w2 = expert_weights(int(e), hidden, inter, seed)
        w13, w2 = w13.float(), w2.float()
        if fp8_experts:
            w13 = gemm.dequantize_weight_128x128(*gemm.quantize_weight_128x128(w13))
            w2 = gemm.dequantize_weight_128x128(*gemm.quantize_weight_128x128(w2))
        tok, k = (idx == e).nonzero(as_tuple=True)
        hcat = xin[tok] @ w13.t()
        h = (torch.nn.functional.silu(hcat[:, :inter]) * hcat[:, inter:]).to(torch.bfloat16)
        h = moe.ref_dequantize_1x128(*moe.ref_quantize_1x128(h)).float() if fp8_experts else h.float()
        y = (h @ w2.t()).to(torch.bfloat16).float()
        out.index_add_(0, tok, y * w[tok, k].unsqueeze(1))
    return out


class HostMoEFeedForward:
    """The same layer over :class:`rocshmem_b200.ops.moe_host.HostEpDispatcher` with the experts evaluated by
    ``torch.matmul``: host-API data movement, any backend (CPU shared memory included). The structure is that of
    :class:`MoEFeedForward` (dispatch, per-expert rows, per-row gate-weighted reduction, unweighted combine), so
    multi-process CPU tests cover the layer's logic; it is not a fast path."""

    def __init__(self, num_experts: int, top_k: int, hidden: int, inter: int, max_tokens: int, seed: int = 0):
        from ..ops import moe_host
        self.d = moe_host.HostEpDispatcher(num_experts, top_k, hidden, max_tokens)
        self.hidden, self.inter, self.top_k = hidden, inter, top_k
        self.e_local = self.d.experts_per_rank
        first = rt.my_pe() * self.e_local
        self.weights = [expert_weights(first + e, hidden, inter, seed) for e in range(self.e_local)]

    def destroy(self) -> None:
        """Collective: free the dispatcher's symmetric buffers."""
        self.d.destroy()

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """Dispatch, per-expert SwiGLU feed-forward in PyTorch, combine; collective."""
        res = self.d.dispatch(x, topk_idx, topk_weights)
        rows = res.num_rows()
        xin = moe.ref_dequantize_1x128(res.recv_x[:rows].cpu(), res.recv_scales[:rows].cpu()).to(torch.bfloat16).float()
        local = res.local_expert_idx()[:rows].cpu()
        gates = res.gate_weights()[:rows].cpu()
        y_rows = torch.zeros((rows, self.hidden))
        for e, (w13, w2) in enumerate(self.weights):
            r, k = (local == e).nonzero(as_tuple=True)
            if r.numel() == 0:
                continue
            hc = xin[r] @ w13.float().t()
            h = (torch.nn.functional.silu(hc[:, :self.inter]) * hc[:, self.inter:]).to(torch.bfloat16).float()
            y = (h @ w2.float().t()).to(torch.bfloat16).float()
            y_rows.index_add_(0, r, y * gates[r, k].unsqueeze(1))
        buf = self.d.result_buffer()
        buf[:rows].copy_(y_rows.to(torch.bfloat16).to(buf.device))
        return self.d.combine(buf, topk_idx, topk_weights, x.shape[0], weighted=False)

    __call__ = forward
