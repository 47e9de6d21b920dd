"""Expert-parallel MoE feed-forward layer (SwiGLU experts) built from this package's kernels.

One call runs, stream-ordered and without a host synchronisation, as four kernels (plus a memset-like one on a
side stream)::

    dispatch       fp8 1x128 rows over NVLink; its tail groups the received (row, k) pairs by local expert
    gate/up GEMM   grouped block-scaled e4m3 tcgen05 GEMM whose producer warps gather the received rows (and the
                   accumulate warps their scales) by index; the epilogue applies SwiGLU and quantises the hidden
                   activation to e4m3 1 x 128 for the next GEMM
    down GEMM      grouped block-scaled GEMM whose epilogue multiplies every row by its gate weight and adds it into
                   the row's slot of the result buffer (the sum over a token's local experts)
    combine        pull over NVLink, sum over the ranks a token went to

With bf16 experts the GEMMs are the bf16 kernels (bf16 rows gathered inside the GEMM; e4m3 rows de-quantised into
expert order by one extra kernel first).

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

    ``fp8_experts``: block-scaled e4m3 expert GEMMs (1 x 128 activation scales, 128 x 128 weight scales). ``None``
    chooses them whenever the dispatch is quantised and the shapes allow (hidden % 512 == 0, inter % 512 == 0): the
    received e4m3 rows then feed the tensor cores as they are. With bf16 experts behind a quantised dispatch one
    extra kernel de-quantises the rows into expert order (doing that inside the GEMM's producer warps was measured
    slower); with a bf16 dispatch the bf16 rows are gathered inside the GEMM.

    ``pair_capacity`` bounds the number of (row, expert) pairs this rank can process in one call; the
    default is the worst case ``n_ranks * max_tokens * top_k``. With balanced routing the expected number
    is ``max_tokens * top_k``, and a tighter bound saves memory; exceeding it is the caller's error.
    """

    def __init__(self, num_experts: int, top_k: int, hidden: int, inter: int, max_tokens: int,
                 team: Optional[rt.Team] = None, quantize: bool = True, layout: str = "compact", seed: int = 0,
                 pair_capacity: Optional[int] = None, fp8_experts: Optional[bool] = None, low_latency: bool = False):
        if rt.n_local_pes() != 1:
            raise RuntimeError("MoEFeedForward needs one PE per process")
        if hidden % 64 or inter % 64:
            raise ValueError("hidden and inter must be multiples of 64")
        fits_fp8 = quantize and hidden % 512 == 0 and inter % 512 == 0
        if fp8_experts and not fits_fp8:
            raise ValueError("fp8 experts need an fp8 dispatch, hidden % 512 == 0 and inter % 512 == 0")
        self.fp8_experts = fits_fp8 if fp8_experts is None else bool(fp8_experts)
        self.d = moe.EpDispatcher(num_experts, top_k, hidden, max_tokens, team=team, quantize=quantize, layout=layout,
                                  expert_layout=True, low_latency=low_latency)
        self.hidden, self.inter, self.top_k = hidden, inter, top_k
        self.n_ranks, self.e_local = self.d.n_ranks, self.d.experts_per_rank
        dev = rt.device()
        first = self.d.team.my_pe() * self.e_local
        ws = [expert_weights(first + e, hidden, inter, seed) for e in range(self.e_local)]
        w13 = torch.stack([w[0] for w in ws]).to(dev).contiguous()   # [E_local, 2 * inter, hidden]
        w2 = torch.stack([w[1] for w in ws]).to(dev).contiguous()    # [E_local, hidden, inter]
        cap = pair_capacity or self.n_ranks * max_tokens * top_k
        self.pair_capacity = cap
        self.side = torch.cuda.Stream()
        self.ev_dispatched, self.ev_zeroed = torch.cuda.Event(), torch.cuda.Event()
        self.kernel_launches = 0
        if self.fp8_experts:
            self.w13_q, self.w13_s = gemm.quantize_weight_128x128(w13)
            self.w2_q, self.w2_s = gemm.quantize_weight_128x128(w2)
            self.h_q = torch.zeros((cap, inter), dtype=torch.uint8, device=dev)
            self.h_s = torch.zeros((cap, inter // 128), dtype=torch.float32, device=dev)
        else:
            self.w13, self.w2 = w13, w2
            self.h = torch.zeros((cap, inter), dtype=torch.bfloat16, device=dev)        # silu(gate) * up
            if quantize:
                self.xs = torch.zeros((cap, hidden), dtype=torch.bfloat16, device=dev)  # de-quantised rows, expert order

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
        cur = torch.cuda.ExternalStream(stream) if isinstance(stream, int) else (stream or torch.cuda.current_stream())
        before = d.kernel_launches
        marks = []

        def mark(name):
            if stage_us is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(cur)
                marks.append((name, ev))

        mark("start")
        d.dispatch(x, topk_idx, topk_weights, stream=stream)
        mark("dispatch")
        offsets, lay_row, _, lay_w = d.expert_pairs()
        y = d.result_buffer()
        # The down projection adds into the result rows, which therefore start from zero; clearing them runs on a
        # side stream beside the first GEMM.
        self.ev_dispatched.record(cur)
        self.side.wait_event(self.ev_dispatched)
        C.moe_zero_rows(d.recv_info.data_ptr(), self.n_ranks, self.hidden, y.data_ptr(), self.side.cuda_stream)
        self.ev_zeroed.record(self.side)
        launches = 3
        if self.fp8_experts:
            # Received e4m3 rows and their scales feed the first GEMM as they are (gathered by its producer warps);
            # its epilogue quantises the hidden activation for the second one.
            gemm.grouped_gemm_fp8_swiglu_quant(d.recv_x, d.recv_scales, self.w13_q, self.w13_s, offsets, self.h_q,
                                               self.h_s, row_index=lay_row, stream=stream)
            mark("gemm_gate_up")
            cur.wait_event(self.ev_zeroed)
            gemm.grouped_gemm_fp8_scatter_add(self.h_q, self.h_s, self.w2_q, self.w2_s, offsets, lay_row, y,
                                              weights=lay_w, stream=stream)
        else:
            if d.quantize:
                C.moe_gather_rows(d.recv_x.data_ptr(), d.recv_scales.data_ptr(), 1, offsets.data_ptr(), self.e_local,
                                  lay_row.data_ptr(), self.hidden, self.xs.data_ptr(), s)
                mark("gather")
                gemm.grouped_gemm_bf16(self.xs, self.w13, offsets, swiglu=True, out=self.h, stream=stream)
                launches += 1
            else:
                gemm.grouped_gemm_bf16_gathered(d.recv_x, lay_row, self.w13, offsets, swiglu=True, out=self.h,
                                                stream=stream)
            mark("gemm_gate_up")
            cur.wait_event(self.ev_zeroed)
            gemm.grouped_gemm_bf16_scatter_add(self.h, self.w2, offsets, lay_row, y, weights=lay_w, stream=stream)
        mark("gemm_down")
        out = d.combine(y, topk_idx, topk_weights, x.shape[0], weighted=False, out=out, stream=stream)
        mark("combine")
        self.kernel_launches += (d.kernel_launches - before) + launches
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
