"""Expert-parallel dispatch / combine written against the host API only (put, get, barrier).

It produces exactly the buffers of :class:`rocshmem_b200.ops.moe.EpDispatcher` (compact layout: e4m3 rows with
1 x 128 scales, 128-byte metadata records, ``recv_info``) but moves the data with ``putmem`` / ``getmem`` from the
host, so it runs on the CPU shared-memory backend as well as on GPUs. It serves as an executable description of
the protocol the fused kernels implement, as the oracle of multi-process CPU tests, and as a fallback where the
fused kernels cannot be used. Not a fast path: every step synchronises with ``barrier_all``.

Protocol of one dispatch on rank ``me``:

1. every token gets the set of ranks that own one of its experts (a token is sent to a rank once, however many
   of its experts live there);
2. the per-destination counts are put into row ``me`` of every rank's count matrix; after a barrier every rank
   knows the whole matrix, and therefore where each source's rows start in every receive buffer;
3. the rows for destination ``d`` (quantised) are put as one block at that offset, with their scales and records;
4. after a second barrier every rank derives ``recv_info`` from the matrix and its own records.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt
from . import moe

META_WORDS = 32


class HostEpDispatcher:
    """Dispatch / combine with the buffers of ``EpDispatcher`` (compact layout), moved by host-API puts and gets."""

    def __init__(self, num_experts: int, top_k: int, hidden: int, max_tokens: int, quantize: bool = True):
        P = rt.n_pes()
        if num_experts % P or hidden % 128 or not (1 <= top_k <= 8):
            raise ValueError("num_experts must divide by the PE count, hidden by 128, top_k in [1, 8]")
        self.num_experts, self.top_k, self.hidden, self.max_tokens = num_experts, top_k, hidden, max_tokens
        self.n_ranks, self.experts_per_rank = P, num_experts // P
        self.quantize = bool(quantize)
        rows = P * max_tokens
        z = rt.zeros
        self.recv_x = z((rows, hidden), torch.uint8 if quantize else torch.bfloat16)
        self.recv_scales = z((rows, hidden // 128), torch.float32)
        self.recv_meta = z((rows, META_WORDS), torch.int32)
        self.recv_info = z(1 + 2 * P + self.experts_per_rank, torch.int32)
        self.counts = z((P, P), torch.int32)          # counts[s, d]: rows source s sends to destination d
        self._y: Optional[torch.Tensor] = None
        self._sent_slot: Optional[torch.Tensor] = None

    def destroy(self) -> None:
        """Collective: give the symmetric buffers back to the heap."""
        rt.free_all([self.recv_x, self.recv_scales, self.recv_meta, self.recv_info, self.counts, self._y])
        self.recv_x = self.recv_scales = self.recv_meta = self.recv_info = self.counts = self._y = None

    def result_buffer(self) -> torch.Tensor:
        """Symmetric bf16 buffer the experts write their result rows to (row ``i`` answers received row ``i``)."""
        if self._y is None:
            self._y = rt.zeros((self.n_ranks * self.max_tokens, self.hidden), torch.bfloat16)
        return self._y

    def _dev(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.recv_x.device)

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> moe.DispatchResult:
        """Send every token once to each rank that owns one of its experts; collective."""
        P, me, K, epr = self.n_ranks, rt.my_pe(), self.top_k, self.experts_per_rank
        T = x.shape[0]
        if T > self.max_tokens:
            raise ValueError("too many tokens")
        idx, w = topk_idx.cpu(), topk_weights.cpu()
        rank_of = torch.where(idx >= 0, idx // epr, torch.full_like(idx, -1))
        goes = torch.zeros((T, P), dtype=torch.bool)
        for d in range(P):
            goes[:, d] = (rank_of == d).any(dim=1)
        counts = goes.sum(dim=0).to(torch.int32)
        # 2. my row of the count matrix, everywhere
        row = self._dev(counts.contiguous())
        for d in range(P):
            rt.putmem(self.counts[me], row, d)
        rt.barrier_all()
        matrix = self.counts.cpu()
        # 3. payload: rows in token order, one block per destination
        xq = x.cpu()
        if self.quantize:
            q, sc = moe.ref_quantize_1x128(xq)
            payload = q.view(torch.uint8)
        else:
            payload, sc = xq, torch.zeros((T, self.hidden // 128))
        self._sent_slot = torch.full((T, P), -1, dtype=torch.int64)
        for dd in range(P):
            d = (me + dd) % P                      # rotate the order like the kernels do
            toks = goes[:, d].nonzero(as_tuple=True)[0]
            n = toks.numel()
            if n == 0:
                continue
            base = int(matrix[:me, d].sum())
            self._sent_slot[toks, d] = base + torch.arange(n)
            meta = torch.zeros((n, META_WORDS), dtype=torch.int32)
            local = torch.where((rank_of[toks] == d), idx[toks] % epr, torch.full_like(idx[toks], -1))
            meta[:, 0:K] = local.to(torch.int32)
            meta[:, 8:8 + K] = w[toks].contiguous().view(torch.int32)
            meta[:, 16] = toks.to(torch.int32)
            meta[:, 17] = me
            rt.putmem(self.recv_x[base:base + n], self._dev(payload[toks].contiguous()), d)
            rt.putmem(self.recv_scales[base:base + n], self._dev(sc[toks].contiguous().float()), d)
            rt.putmem(self.recv_meta[base:base + n], self._dev(meta), d)
        rt.barrier_all()
        # 4. receive-side bookkeeping
        info = torch.zeros(1 + 2 * P + epr, dtype=torch.int32)
        col = matrix[:, me]
        info[0] = int(col.sum())
        info[1:1 + P] = torch.cumsum(col, 0) - col
        info[1 + P:1 + 2 * P] = col
        rows = int(col.sum())
        local_idx = self.recv_meta[:rows, 0:K].cpu()
        for e in range(epr):
            info[1 + 2 * P + e] = int((local_idx == e).sum())
        self.recv_info.copy_(self._dev(info))
        x_view = self.recv_x.view(torch.float8_e4m3fn) if self.quantize else self.recv_x
        return moe.DispatchResult(x_view, self.recv_scales, self.recv_meta, self.recv_info, P, K)

    def combine(self, y: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, num_tokens: int,
                weighted: bool = True) -> torch.Tensor:
        """For every token the (weighted) sum over the ranks it was sent to of that rank's result row."""
        if self._sent_slot is None:
            raise RuntimeError("combine before dispatch")
        P, me, epr = self.n_ranks, rt.my_pe(), self.experts_per_rank
        rt.barrier_all()                                  # every rank's result rows are complete
        idx, w = topk_idx.cpu(), topk_weights.cpu()
        rank_of = torch.where(idx >= 0, idx // epr, torch.full_like(idx, -1))
        matrix = self.counts.cpu()
        out = torch.zeros((num_tokens, self.hidden), dtype=torch.float32)
        for d in range(P):
            slots = self._sent_slot[:num_tokens, d]
            toks = (slots >= 0).nonzero(as_tuple=True)[0]
            n = toks.numel()
            if n == 0:
                continue
            base = int(matrix[:me, d].sum())
            block = torch.empty((n, self.hidden), dtype=torch.bfloat16, device=y.device)
            rt.getmem(block, y[base:base + n], d)         # my rows on rank d are one contiguous block
            gate = ((rank_of[toks] == d).float() * w[toks]).sum(dim=1) if weighted else torch.ones(n)
            out[toks] += block.cpu().float() * gate.unsqueeze(1)
        rt.barrier_all()                                  # nobody reuses its rows while a peer still reads them
        return out.to(torch.bfloat16)
