"""Alternative alltoall / fcollect schedules built from host-API puts, gets and barriers.

The reference carries several schedules for these two collectives besides the linear one: Bruck's log-step
exchange (``alltoall_brucks`` / ``fcollect_brucks``, ``src/gpu_ib/context_ib_tmpl_device.hpp:516-1045``) and the
two-phase "GPU-centric" clustered exchange (``_gcen`` / ``_gcen2``: gather inside a cluster of about sqrt(n)
PEs, then one larger message between matching PEs of different clusters; host form in
``src/reverse_offload/mpi_transport.cpp:490-1031``), chosen by heuristics. They trade message count against
bytes moved: the linear schedule sends n - 1 messages of one block, Bruck's ceil(log2 n) messages of n / 2 blocks,
the clustered one about 2 sqrt(n) messages.

On one NVSwitch box every peer is one hop away at full bandwidth, so the library kernels
(``ops.collectives.alltoall_async`` / ``fcollect_async``) use the linear schedule from all SMs and that is the fast
path. The schedules here exist for the case the reference built them for - per-message cost dominating, e.g. tiny
blocks through the host proxy - and as executable descriptions with tests. They run on any backend (CPU included),
for the world team.

All functions are collective over all PEs, take symmetric ``dest`` / ``source`` tensors laid out like the library
collectives (block j of ``source`` goes to PE j; block i of ``dest`` comes from PE i) and synchronise with
``barrier_all``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import runtime as rt


def _blocks(t: torch.Tensor, n: int) -> torch.Tensor:
    b = t.view(torch.uint8).view(-1)
    if b.numel() % n:
        raise ValueError("tensor size must divide by the number of PEs")
    return b.view(n, b.numel() // n)


class HostCollectivePlan:
    """Staging buffers (symmetric, allocated collectively once) for blocks of up to ``max_block_bytes`` bytes."""

    def __init__(self, max_block_bytes: int):
        self.n = rt.n_pes()
        self.me = rt.my_pe()
        self.max_block_bytes = int(max_block_bytes)
        n = self.n
        self.tmp = rt.zeros((n, self.max_block_bytes), torch.uint8)     # rotated working copy
        self.stage = rt.zeros((n, self.max_block_bytes), torch.uint8)   # landing area of one step
        self.cluster = cluster_size(n)

    def destroy(self) -> None:
        """Free the staging buffers (collective)."""
        rt.free(self.stage)
        rt.free(self.tmp)

    def _check(self, nbytes: int) -> None:
        if nbytes > self.max_block_bytes:
            raise ValueError(f"block of {nbytes} bytes exceeds the plan's {self.max_block_bytes}")

    # ---- alltoall ---------------------------------------------------------------------------------------

    def alltoall_linear(self, dest: torch.Tensor, source: torch.Tensor) -> None:
        """n - 1 puts of one block each."""
        n, me = self.n, self.me
        d, s = _blocks(dest, n), _blocks(source, n)
        rt.barrier_all()
        for j in range(n):
            pe = (me + j) % n
            rt.putmem(d[me], s[pe], pe, nbi=True)
        rt.barrier_all()

    def alltoall_bruck(self, dest: torch.Tensor, source: torch.Tensor) -> None:
        """ceil(log2 n) rounds; in round k every PE sends the blocks whose index has bit k set, packed into one
        message, to the PE 2^k above it."""
        n, me = self.n, self.me
        d, s = _blocks(dest, n), _blocks(source, n)
        nb = s.shape[1]
        self._check(nb)
        tmp = self.tmp[:, :nb]
        for i in range(n):                       # tmp[i]: my block for PE me + i
            self.tmp[i, :nb] = s[(me + i) % n]
        k = 1
        while k < n:
            idx = [i for i in range(n) if i & k]
            packed = torch.stack([tmp[i] for i in idx]).contiguous()
            rt.barrier_all()                     # the receiver has unpacked the previous round
            # a packed message lands at the start of the peer's staging area
            rt.putmem(self.stage.view(-1)[:packed.numel()], packed.view(-1), (me + k) % n)
            rt.barrier_all()
            got = self.stage.view(-1)[:packed.numel()].view(len(idx), nb)
            for r, i in enumerate(idx):
                self.tmp[i, :nb] = got[r]
            k <<= 1
        for i in range(n):                       # tmp[i] now comes from PE me - i
            d[(me - i) % n] = tmp[i]
        rt.barrier_all()

    def alltoall_clustered(self, dest: torch.Tensor, source: torch.Tensor, cluster: Optional[int] = None) -> None:
        """Two phases over clusters of ``c`` consecutive PEs (c divides n). Phase 1: PE (g, l) fetches from every
        mate m of its cluster the blocks that m has for the PEs with local index l of every cluster. Phase 2: it
        sends each cluster g' one message of c blocks, straight into PE (g', l)'s ``dest``."""
        n, me = self.n, self.me
        c = cluster or self.cluster
        if n % c:
            raise ValueError("cluster size must divide the number of PEs")
        d, s = _blocks(dest, n), _blocks(source, n)
        nb = s.shape[1]
        self._check(nb)
        g, l = divmod(me, c)
        ncl = n // c
        rt.barrier_all()                         # every source is ready
        # stage[g' * c + m]: block of mate m (of my cluster) for PE (g', l)
        for m in range(c):
            mate = g * c + (l + m) % c
            for gp in range(ncl):
                rt.getmem(self.stage[gp * c + (mate % c), :nb], s[gp * c + l], mate, nbi=True)
        rt.quiet()
        keep = []                                # sources of non-blocking puts stay alive until the barrier
        for gp in range(ncl):
            tgt = ((g + gp) % ncl)
            block = self.stage[tgt * c:(tgt + 1) * c, :nb].contiguous()
            keep.append(block)
            rt.putmem(d[g * c:(g + 1) * c].view(-1), block.view(-1), tgt * c + l, nbi=True)
        rt.barrier_all()
        del keep

    # ---- fcollect ---------------------------------------------------------------------------------------

    def fcollect_linear(self, dest: torch.Tensor, source: torch.Tensor) -> None:
        """My block to every PE with one put each."""
        n, me = self.n, self.me
        d = _blocks(dest, n)
        src = source.view(torch.uint8).view(-1)
        rt.barrier_all()
        for j in range(n):
            rt.putmem(d[me], src, (me + j) % n, nbi=True)
        rt.barrier_all()

    def fcollect_bruck(self, dest: torch.Tensor, source: torch.Tensor) -> None:
        """Doubling: after round k every PE holds the blocks of the 2^(k+1) PEs starting at itself."""
        n, me = self.n, self.me
        d = _blocks(dest, n)
        src = source.view(torch.uint8).view(-1)
        nb = src.numel()
        self._check(nb)
        self.tmp[0, :nb] = src                   # tmp[i]: block of PE me + i
        have = 1
        rt.barrier_all()
        while have < n:
            cnt = min(have, n - have)
            # my first `cnt` blocks are blocks [have, have + cnt) of the PE `have` below me
            if nb == self.max_block_bytes:
                rt.putmem(self.tmp[have:have + cnt].view(-1), self.tmp[:cnt].view(-1), (me - have) % n)
            else:
                for i in range(cnt):
                    rt.putmem(self.tmp[have + i, :nb], self.tmp[i, :nb].contiguous(), (me - have) % n, nbi=True)
            rt.barrier_all()
            have += cnt
        for i in range(n):
            d[(me + i) % n] = self.tmp[i, :nb]
        rt.barrier_all()

    def fcollect_clustered(self, dest: torch.Tensor, source: torch.Tensor, cluster: Optional[int] = None) -> None:
        """Gather inside the cluster, then every PE sends its cluster's c blocks as one message to the PEs with
        its local index in the other clusters, and finally cluster mates exchange what they received."""
        n, me = self.n, self.me
        c = cluster or self.cluster
        if n % c:
            raise ValueError("cluster size must divide the number of PEs")
        d = _blocks(dest, n)
        src = source.view(torch.uint8).view(-1)
        g, l = divmod(me, c)
        ncl = n // c
        rt.barrier_all()
        for m in range(c):                       # phase 1: my block to every mate
            rt.putmem(d[me], src, g * c + (l + m) % c, nbi=True)
        rt.barrier_all()
        mine = d[g * c:(g + 1) * c].contiguous()
        for gp in range(1, ncl):                 # phase 2: my cluster's blocks to PE (g', l)
            tgt = (g + gp) % ncl
            rt.putmem(d[g * c:(g + 1) * c].view(-1), mine.view(-1), tgt * c + l, nbi=True)
        rt.barrier_all()
        # Phase 2 already delivered every cluster's blocks to every PE: PE (g', l) received cluster g from PE
        # (g, l) for every g. Nothing is left to exchange.

    # ---- selection ----------------------------------------------------------------------------------------

    def alltoall(self, dest: torch.Tensor, source: torch.Tensor, algorithm: str = "auto") -> str:
        """Run the named schedule (``linear``, ``bruck``, ``clustered`` or ``auto``); returns the one used."""
        nb = _blocks(source, self.n).shape[1]
        if algorithm == "auto":
            algorithm = choose_algorithm(self.n, nb)
        getattr(self, "alltoall_" + algorithm)(dest, source)
        return algorithm

    def fcollect(self, dest: torch.Tensor, source: torch.Tensor, algorithm: str = "auto") -> str:
        """Run the named schedule (``linear``, ``bruck``, ``clustered`` or ``auto``); returns the one used."""
        nb = source.numel() * source.element_size()
        if algorithm == "auto":
            algorithm = choose_algorithm(self.n, nb)
        getattr(self, "fcollect_" + algorithm)(dest, source)
        return algorithm


def cluster_size(n: int) -> int:
    """The divisor of n closest to sqrt(n) (1 for primes: the clustered schedule then equals the linear one)."""
    best, root = 1, math.sqrt(n)
    for c in range(1, n + 1):
        if n % c == 0 and abs(c - root) < abs(best - root):
            best = c
    return best


def choose_algorithm(n: int, block_bytes: int, per_message_us: float = 6.0, gbytes_per_s: float = 700.0) -> str:
    """Pick the schedule with the lowest modelled time: messages x per-message cost + bytes sent / bandwidth.

    The defaults describe host-issued copies between B200s (a stream copy costs a few microseconds to issue,
    a peer copy moves about 700 GB/s): there the linear schedule wins above a few KiB per block, Bruck's or the
    clustered one only for very small blocks on many PEs.
    """
    if n <= 2:
        return "linear"
    per_byte_us = 1e-3 / gbytes_per_s
    c = cluster_size(n)
    rounds = math.ceil(math.log2(n))
    cost = {
        "linear": (n - 1) * per_message_us + (n - 1) * block_bytes * per_byte_us,
        "bruck": rounds * 3 * per_message_us + rounds * (n // 2) * block_bytes * per_byte_us,
    }
    if c > 1:
        cost["clustered"] = (n + n // c) * per_message_us + 2 * n * block_bytes * per_byte_us
    return min(cost, key=cost.get)


class HostAllToAllV:
    """Variable-count all-to-all over the host API (the reference's ``alltoall`` is fixed-size only).

    Every PE sends ``send_counts[j]`` rows of ``source`` to PE ``j`` (rows for PE 0 first, then PE 1, ...); the rows a
    PE receives land in ``dest`` ordered by source PE. Counts travel first (one row of a symmetric count matrix per
    PE), then every PE knows where each source's rows start in every destination and puts its rows there directly -
    the protocol of the MoE dispatch without the routing. Collective over all PEs; ``dest`` and ``source`` are
    symmetric tensors whose first dimension is the row index.
    """

    def __init__(self):
        self.n, self.me = rt.n_pes(), rt.my_pe()
        self.counts = rt.zeros((self.n, self.n), torch.int64)       # counts[s, d]: rows PE s sends to PE d

    def destroy(self) -> None:
        """Collective: free the count matrix."""
        rt.free(self.counts)
        self.counts = None

    def __call__(self, dest: torch.Tensor, source: torch.Tensor, send_counts) -> torch.Tensor:
        """Returns the int64 tensor of rows received from every PE (``recv_counts``); the rows are in
        ``dest[:recv_counts.sum()]``. Raises ``ValueError`` on every PE alike when ``dest`` is too small for some PE."""
        n, me = self.n, self.me
        send = torch.as_tensor(list(send_counts), dtype=torch.int64)
        if send.numel() != n or int(send.min()) < 0 or int(send.sum()) > source.shape[0]:
            raise ValueError("send_counts needs one non-negative entry per PE and may not exceed the rows of source")
        row = send.to(self.counts.device)
        for d in range(n):
            rt.putmem(self.counts[me], row, d, nbi=True)
        rt.barrier_all()                       # completes the puts: the whole matrix is everywhere
        matrix = self.counts.cpu()
        recv = matrix[:, me].clone()
        # dest is symmetric, so it has the same number of rows everywhere: every PE can check every destination
        # and all of them agree on whether the exchange takes place.
        need = matrix.sum(dim=0)
        if int(need.max()) > dest.shape[0]:
            raise ValueError(f"dest holds {dest.shape[0]} rows, up to {int(need.max())} arrive")
        for dd in range(n):
            d = (me + dd) % n
            cnt = int(send[d])
            start = int(send[:d].sum())
            if cnt:
                base = int(matrix[:me, d].sum())       # rows that PEs before me send to d
                rt.putmem(dest[base:base + cnt], source[start:start + cnt], d, nbi=True)
        rt.barrier_all()
        return recv
