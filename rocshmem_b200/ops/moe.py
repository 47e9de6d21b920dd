"""Expert-parallel MoE dispatch / combine (DeepEP-style) on the symmetric heap, plus the 1x128
block-scaled e4m3 helpers and their fp32 reference implementations.

``EpDispatcher`` owns the symmetric receive buffers of one (team, shape) combination:

* :meth:`EpDispatcher.dispatch` sends every token once to each rank that hosts one of its top-k experts,
  quantised to e4m3 with one fp32 scale per 128 elements (or as bf16), directly into its final row of
  the destination's buffer, with a metadata record per row (local expert ids, gate weights, source);
* :meth:`EpDispatcher.combine` pulls the processed rows back and sums them per token in fp32, weighted
  by the gate weights of the experts that live on each rank.

``layout='compact'`` packs received rows by source rank (normal mode); ``layout='slotted'`` gives
every source a fixed window of ``max_tokens`` rows so that sending needs no count round-trip
(low-latency mode). There is no equivalent in the reference; the nearest primitive is its fixed-size
``alltoall`` (``src/ipc/context_ipc_tmpl_device.hpp:474-501``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import runtime as rt
from ..utils.trace import trace_range

E4M3_MAX = 448.0


def _stream(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


@dataclass
class DispatchResult:
    """Views into the dispatcher's receive buffers (valid until the next dispatch)."""
    recv_x: torch.Tensor        # [P * max_tokens, hidden] float8_e4m3fn (or bf16 without quantisation)
    recv_scales: torch.Tensor   # [P * max_tokens, hidden / 128] fp32
    recv_meta: torch.Tensor     # [P * max_tokens, 32] int32 records
    recv_info: torch.Tensor     # int32: [0] rows, [1+s] first row of source s, [1+P+s] rows of source s,
                                #        [1+2P+e] (row, k) pairs of local expert e
    n_ranks: int
    top_k: int

    def num_rows(self) -> int:
        """Total received rows (synchronises: reads one int from the device)."""
        return int(self.recv_info[0].item())

    def local_expert_idx(self) -> torch.Tensor:
        """[rows, top_k] local expert index of every choice that lives on this rank, -1 otherwise."""
        return self.recv_meta[:, 0:self.top_k]

    def gate_weights(self) -> torch.Tensor:
        """[rows, top_k] fp32 gate weights as sent by the source."""
        return self.recv_meta[:, 8:8 + self.top_k].view(torch.float32)

    def src_token(self) -> torch.Tensor:
        """Token index on the source rank, per row."""
        return self.recv_meta[:, 16]

    def src_rank(self) -> torch.Tensor:
        """Source rank, per row."""
        return self.recv_meta[:, 17]

    def row_ranges(self):
        """[(first_row, n_rows)] per source rank (synchronises)."""
        info = self.recv_info.cpu().tolist()
        P = self.n_ranks
        return [(info[1 + s], info[1 + P + s]) for s in range(P)]

    def rows_per_expert(self) -> torch.Tensor:
        """Number of (row, choice) pairs per local expert."""
        P = self.n_ranks
        return self.recv_info[1 + 2 * P:]


class EpDispatcher:
    """Symmetric receive buffers and launch state of dispatch / combine for one (team, shape) combination."""

    def __init__(self, num_experts: int, top_k: int, hidden: int, max_tokens: int,
                 team: Optional[rt.Team] = None, quantize: bool = True, layout: str = "compact",
                 blocks: Optional[int] = None, dynamic: Optional[bool] = None, expert_layout: bool = False,
                 low_latency: bool = False):
        """``dynamic``: dispatch hands (token, destination) pairs to warps through per-destination counters and
        combine hands tokens out through a counter (levels the tail when fixed shares carry unequal numbers of
        bytes; dispatch pays a second grid barrier for it). ``None`` takes ``ROCSHMEM_EP_DYNAMIC`` (default on).

        ``expert_layout``: the dispatch kernel also groups the received (row, k) pairs by local expert
        (:meth:`expert_pairs`), which a grouped GEMM consumes directly.

        ``low_latency``: for small batches (decode): one ordinary launch with a block per token, the slotted
        layout (implied), one signal word per source instead of a count round-trip, and a combine without the
        closing barrier: the result buffer may be rewritten only after the next dispatch on this object has
        completed. Every member must choose the same options."""
        C = rt._C()
        if not C.is_cuda():
            raise RuntimeError("EpDispatcher needs the CUDA backend")
        self.team = team or rt.team_world()
        P = self.team.n_pes()
        if P > C.EP_MAX_RANKS:
            raise ValueError(f"EpDispatcher supports teams of at most {C.EP_MAX_RANKS} ranks")
        if num_experts % P:
            raise ValueError("num_experts must be divisible by the team size")
        if hidden % 512 or not (512 <= hidden <= 8192):
            raise ValueError("hidden must be a multiple of 512 in [512, 8192]")
        if not (1 <= top_k <= 8):
            raise ValueError("top_k must be in [1, 8]")
        self.num_experts, self.top_k, self.hidden, self.max_tokens = num_experts, top_k, hidden, max_tokens
        self.n_ranks, self.experts_per_rank = P, num_experts // P
        self.quantize = bool(quantize)
        self.low_latency = bool(low_latency)
        if self.low_latency:
            layout = "slotted"
        self.layout = {"compact": 0, "slotted": 1}[layout]
        self.blocks = int(blocks or C.ep_default_blocks())
        # tokens handled per block must fit the kernel's shared-memory tables
        while (max_tokens + self.blocks - 1) // self.blocks * ((P + top_k) * 4 + 8) > 40 * 1024:
            self.blocks *= 2
        if dynamic is None:
            dynamic = os.environ.get("ROCSHMEM_EP_DYNAMIC", "1") not in ("", "0")
        self.dynamic = bool(dynamic) and not self.low_latency
        self.with_expert_layout = bool(expert_layout)
        rows = P * max_tokens
        z = rt.zeros
        self.recv_x = z((rows, hidden), torch.uint8 if quantize else torch.bfloat16)
        self.recv_scales = z((rows, hidden // 128), torch.float32)
        self.recv_meta = z((rows, C.EP_META_WORDS), torch.int32)
        self.cnt_in = z(2 * P * P, torch.int64)
        self.exp_in = z(2 * P * self.experts_per_rank, torch.int64)
        self.sent_slot = z((max_tokens, P), torch.int32)
        self.tok_mask = z(max_tokens, torch.int64)
        self.blk_cnt = z(self.blocks * P, torch.int32)
        self.exp_cnt = z(2 * num_experts, torch.int32)
        self.grid_counter = z(1, torch.int64)
        self.phase_ns = z(16, torch.int64)
        self.recv_info = z(1 + 2 * P + self.experts_per_rank, torch.int32)
        self.work_counter = z(C.EP_WORK_WORDS, torch.int64)
        self._buffers = ["recv_x", "recv_scales", "recv_meta", "cnt_in", "exp_in", "sent_slot", "tok_mask", "blk_cnt",
                         "exp_cnt", "grid_counter", "phase_ns", "recv_info", "work_counter"]
        if self.dynamic:
            self.stage_meta = z((max_tokens, C.EP_META_WORDS), torch.int32)
            self.item_tok = z((P, max_tokens), torch.int32)
            self._buffers += ["stage_meta", "item_tok"]
        if self.with_expert_layout:
            cap = rows * top_k
            self.lay_offsets = z(self.experts_per_rank + 1, torch.int32)
            self.lay_row = z(cap, torch.int32)
            self.lay_k = z(cap, torch.int32)
            self.lay_w = z(cap, torch.float32)
            self._buffers += ["lay_offsets", "lay_row", "lay_k", "lay_w"]
        self._y = None
        ptrs = {name: getattr(self, name).data_ptr() for name in self._buffers}
        self._h = C.EpHandle(self.team.handle, num_experts, top_k, hidden, max_tokens, int(quantize),
                             self.layout, self.blocks, int(self.dynamic), int(self.with_expert_layout),
                             int(self.low_latency), ptrs)
        self.kernel_launches = 0

    def destroy(self) -> None:
        """Collective: give the symmetric buffers back to the heap. The object must not be used afterwards and no
        kernel that uses the buffers may be in flight on any member."""
        if self._h is None:
            return
        if rt.is_cuda():
            torch.cuda.synchronize()
        lay = list(getattr(self, "_lay", ()))
        rt.free_all([getattr(self, name) for name in self._buffers] + [self._y] + lay)
        self._h = None
        self._y = None
        if lay:
            del self._lay

    # -- buffers -------------------------------------------------------------------------------------------
    def result_buffer(self) -> torch.Tensor:
        """Symmetric [P * max_tokens, hidden] bf16 buffer for the experts' output rows (input of
        :meth:`combine`), in the row layout of the receive buffers."""
        if self._y is None:
            self._y = rt.zeros((self.n_ranks * self.max_tokens, self.hidden), torch.bfloat16)
        return self._y

    def _result(self) -> DispatchResult:
        x = self.recv_x.view(torch.float8_e4m3fn) if self.quantize else self.recv_x
        return DispatchResult(x, self.recv_scales, self.recv_meta, self.recv_info, self.n_ranks, self.top_k)

    # -- operations -------------------------------------------------------------------------------------------
    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                 stream=None) -> DispatchResult:
        """x [T, hidden] bf16, topk_idx [T, top_k] int32 (global expert ids, -1 unused), topk_weights
        [T, top_k] fp32; all contiguous on this PE's GPU. Stream-ordered."""
        T = x.shape[0]
        if T > self.max_tokens or x.shape[1] != self.hidden or x.dtype != torch.bfloat16:
            raise ValueError("dispatch: x must be [T <= max_tokens, hidden] bf16")
        if topk_idx.dtype != torch.int32 or topk_weights.dtype != torch.float32:
            raise TypeError("dispatch: topk_idx must be int32 and topk_weights fp32")
        if tuple(topk_idx.shape) != (T, self.top_k) or tuple(topk_weights.shape) != (T, self.top_k):
            raise ValueError("dispatch: topk tensors must be [T, top_k]")
        for t in (x, topk_idx, topk_weights):
            if not t.is_contiguous():
                raise ValueError("dispatch: tensors must be contiguous")
        with trace_range("rocshmem_b200.ep_dispatch"):
            self._h.dispatch(x.data_ptr(), topk_idx.data_ptr(), topk_weights.data_ptr(), T, _stream(stream))
        self.kernel_launches += 1
        return self._result()

    def combine(self, y: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                num_tokens: int, weighted: bool = True, out: Optional[torch.Tensor] = None,
                stream=None) -> torch.Tensor:
        """y: the symmetric :meth:`result_buffer`. Returns out [num_tokens, hidden] bf16 with, for every
        token, the (weighted) sum of its rows over the ranks it was dispatched to."""
        if y.data_ptr() != self.result_buffer().data_ptr():
            raise ValueError("combine: y must be this dispatcher's result_buffer()")
        if not 0 <= num_tokens <= self.max_tokens:
            raise ValueError("combine: num_tokens must be in [0, max_tokens]")
        if topk_idx.dtype != torch.int32 or topk_weights.dtype != torch.float32:
            raise TypeError("combine: topk_idx must be int32 and topk_weights fp32")
        for t in (topk_idx, topk_weights):
            if not t.is_contiguous() or t.shape[0] < num_tokens or t.shape[1] != self.top_k:
                raise ValueError("combine: topk tensors must be contiguous [>= num_tokens, top_k]")
        if out is None:
            out = torch.empty((num_tokens, self.hidden), dtype=torch.bfloat16, device=y.device)
        elif (out.dtype != torch.bfloat16 or not out.is_contiguous() or out.shape[0] < num_tokens
              or out.shape[1] != self.hidden):
            raise ValueError("combine: out must be a contiguous [>= num_tokens, hidden] bf16 tensor")
        with trace_range("rocshmem_b200.ep_combine"):
            self._h.combine(y.data_ptr(), out.data_ptr(), topk_idx.data_ptr(), topk_weights.data_ptr(), num_tokens,
                            int(weighted), _stream(stream))
        self.kernel_launches += 1
        return out

    def phase_times_us(self) -> dict:
        """Device timestamps of the last dispatch and combine (block 0), as microseconds since the
        kernel's first timestamp. Synchronises."""
        ns = self.phase_ns.cpu().tolist()
        if self.low_latency:
            names_d = {0: "start", 4: "sent", 5: "peers_done", 6: "outputs"}
        else:
            names_d = dict(enumerate(["start", "scan", "grid_barrier", "offsets_counts", "sent", "peers_done",
                                      "outputs"]))
        names_c = ["start", "peers_ready", "summed", "peers_done"]
        return {"dispatch": {n: (ns[i] - ns[0]) / 1e3 for i, n in names_d.items()},
                "combine": {n: (ns[8 + i] - ns[8]) / 1e3 for i, n in enumerate(names_c)}}

    def expert_pairs(self):
        """Expert-grouped pair lists written by the last dispatch (``expert_layout=True``): ``offsets``
        [E_local + 1], and per position the received row, the top-k position and the gate weight. Only the first
        ``offsets[-1]`` entries are meaningful; the order inside one expert's range is unspecified."""
        if not self.with_expert_layout:
            raise RuntimeError("the dispatcher was created without expert_layout=True")
        return self.lay_offsets, self.lay_row, self.lay_k, self.lay_w

    def expert_layout(self, stream=None):
        """Row lists grouped by local expert for a grouped GEMM: ``offsets`` [E_local + 1], ``row_index``
        and ``pair_k`` [P * max_tokens * top_k] (only the first ``offsets[-1]`` entries are meaningful)."""
        if not hasattr(self, "_lay"):
            cap = self.n_ranks * self.max_tokens * self.top_k
            self._lay = (rt.zeros(self.experts_per_rank + 1, torch.int32), rt.zeros(cap, torch.int32),
                         rt.zeros(cap, torch.int32), rt.zeros(self.experts_per_rank, torch.int32))
        offsets, row_index, pair_k, cursor = self._lay
        self._h.expert_layout(self.n_ranks, offsets.data_ptr(), row_index.data_ptr(), pair_k.data_ptr(),
                              cursor.data_ptr(), _stream(stream))
        self.kernel_launches += 2
        return offsets, row_index, pair_k


# ---- block-scaled fp8 ---------------------------------------------------------------------------------------------

def fp8_quantize_1x128(x: torch.Tensor, stream=None):
    """[rows, hidden] bf16 -> (e4m3 [rows, hidden], fp32 scales [rows, hidden / 128]); x ~ q * scale."""
    rows, hidden = x.shape
    q = torch.empty((rows, hidden), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, hidden // 128), dtype=torch.float32, device=x.device)
    rt._C().fp8_quantize_1x128(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, hidden, _stream(stream))
    return q.view(torch.float8_e4m3fn), s


def fp8_dequantize_1x128(q: torch.Tensor, scales: torch.Tensor, stream=None) -> torch.Tensor:
    """CUDA kernel: e4m3 rows with one fp32 scale per 128 elements back to bf16."""
    rows, hidden = q.shape
    out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=q.device)
    rt._C().fp8_dequantize_1x128(q.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, hidden, _stream(stream))
    return out


# ---- fp32 references (plain PyTorch, any device) -------------------------------------------------------------------------

def ref_quantize_1x128(x: torch.Tensor):
    """PyTorch reference of the 1 x 128 e4m3 quantisation; returns (float8_e4m3fn rows, fp32 scales)."""
    rows, hidden = x.shape
    xf = x.float().view(rows, hidden // 128, 128)
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax * (1.0 / E4M3_MAX), torch.ones_like(amax))
    inv = torch.where(amax > 0, E4M3_MAX / amax, torch.ones_like(amax))
    q = (xf * inv).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(rows, hidden), scale.view(rows, hidden // 128)


def ref_dequantize_1x128(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """PyTorch reference of the de-quantisation, in fp32."""
    rows, hidden = q.shape
    return (q.float().view(rows, hidden // 128, 128) * scales.view(rows, hidden // 128, 1)).view(rows, hidden)


def ref_dispatch(idxs, n_ranks: int, num_experts: int):
    """Reference routing: for every destination rank the list of (source rank, token) pairs in the
    order the compact layout uses (by source rank, then by token)."""
    epr = num_experts // n_ranks
    out = [[] for _ in range(n_ranks)]
    for s, idx in enumerate(idxs):
        ranks = torch.where(idx >= 0, idx // epr, torch.full_like(idx, -1))
        for t in range(idx.shape[0]):
            for d in sorted(set(int(r) for r in ranks[t].tolist() if r >= 0)):
                out[d].append((s, t))
    return out


def make_routing(num_tokens: int, num_experts: int, top_k: int, seed: int, device="cpu"):
    """Top-k gating from N(0,1) logits with softmax weights over the selected experts."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(num_tokens, num_experts, generator=g)
    vals, idx = logits.topk(top_k, dim=-1)
    w = torch.softmax(vals, dim=-1)
    return idx.to(torch.int32).to(device), w.to(torch.float32).to(device)


def smoke() -> None:
    """One tiny dispatch + combine on whatever runtime is initialised (used by the driver's smoke test)."""
    P = rt.n_pes()
    if rt.n_local_pes() != P:
        return
    T, H, E, K = 64, 1024, 8 * P, 4
    d = EpDispatcher(E, K, H, T)
    dev = rt.device()
    x = rt.zeros((T, H), torch.bfloat16)
    idx = rt.zeros((T, K), torch.int32)
    w = rt.zeros((T, K), torch.float32)
    out = rt.zeros((T, H), torch.bfloat16)
    for l in range(P):
        g = torch.Generator().manual_seed(l)
        rt.local_view(x, l).copy_(torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev))
        i, ww = make_routing(T, E, K, 100 + l, dev)
        rt.local_view(idx, l).copy_(i)
        rt.local_view(w, l).copy_(ww)
    torch.cuda.synchronize()
    res = d.dispatch(x, idx, w)
    y = d.result_buffer()
    for l in range(P):
        q = rt.local_view(res.recv_x.view(torch.uint8), l).view(torch.float8_e4m3fn)
        rt.local_view(y, l).copy_(ref_dequantize_1x128(q, rt.local_view(res.recv_scales, l)).to(torch.bfloat16))
    d.combine(y, idx, w, T, weighted=True, out=out)
    torch.cuda.synchronize()
    for l in range(P):
        got = rt.local_view(out, l).float()
        want = rt.local_view(x, l).float()
        err = (got - want).abs().max().item()
        assert err < 0.35, f"moe smoke: combine error {err}"
