#!/usr/bin/env python
"""Context-parallel causal attention: the sequence is sharded over the ranks, keys and values travel around a ring
(put, counter, wait_until on the host API) while every rank accumulates its queries' output online; the result is
checked against attention over the whole sequence. Runs on GPUs and, without them, on the CPU backend.

    python -m rocshmem_b200.launch -n 4 python examples/python/ring_attention.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.parallel.ring import RingExchange, ring_attention  # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local % torch.cuda.device_count())
    shm.init(heap_size="256M", device=local)
    me, n = shm.my_pe(), shm.n_pes()
    dev = shm.device()
    S, H, D = 64 * n, 4, 32
    sl = S // n
    g = torch.Generator().manual_seed(7)                    # everybody can rebuild the whole problem for the check
    q, k, v = (torch.randn(S, H, D, generator=g) for _ in range(3))
    mine = slice(me * sl, (me + 1) * sl)
    rk, rv = RingExchange((sl, H, D), torch.float32), RingExchange((sl, H, D), torch.float32)
    out = ring_attention(q[mine].to(dev), k[mine].to(dev), v[mine].to(dev), rk, rv, causal=True)
    scores = torch.einsum("shd,thd->hst", q, k) / D ** 0.5
    scores = scores.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
    want = torch.einsum("hst,thd->shd", torch.softmax(scores, dim=-1), v)[mine]
    err = (out.cpu() - want).abs().max().item()
    ok = err < 1e-4
    print(f"pe {me}/{n}: {sl} of {S} positions, max error {err:.2e}: {'PASS' if ok else 'FAIL'}")
    shm.barrier_all()
    rk.destroy()
    rv.destroy()
    shm.finalize()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
