#!/usr/bin/env python
"""Data-parallel training of a small MLP: every rank computes gradients on its own batches, GradientBuckets
averages them over all ranks (symmetric buckets, allreduce), every rank takes the same optimiser step. Runs on GPUs
and, without them, on the CPU shared-memory backend.

    python -m rocshmem_b200.launch -n 4 python examples/python/data_parallel.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402
from rocshmem_b200.parallel.data_parallel import GradientBuckets  # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local % torch.cuda.device_count())
    shm.init(heap_size="256M", device=local)
    me, n = shm.my_pe(), shm.n_pes()
    dev = shm.device()
    torch.manual_seed(0)                                   # the same initial weights everywhere
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 1)).to(dev)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    dp = GradientBuckets(model.parameters(), bucket_bytes=4 << 10)
    teacher = torch.randn(32, 1, generator=torch.Generator().manual_seed(1)).to(dev)
    g = torch.Generator().manual_seed(100 + me)            # different data on every rank
    first = last = None
    for step in range(60):
        x = torch.randn(64, 32, generator=g).to(dev)
        loss = ((model(x) - x @ teacher) ** 2).mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        dp.finish()
        opt.step()
        first = loss.item() if first is None else first
        last = loss.item()
    # the replicas have stayed identical: the maximum over ranks of a checksum equals the minimum
    check = shm.zeros(2, torch.float64)
    s = sum(p.double().sum().item() for p in model.parameters())
    check.copy_(torch.tensor([s, -s], dtype=torch.float64))
    both = shm.zeros(2, torch.float64)
    coll.reduce(both, check, shm.OP_MAX)
    hi, neg_lo = both.cpu().tolist()
    ok = last < 0.5 * first and abs(hi + neg_lo) < 1e-9
    print(f"pe {me}/{n}: loss {first:.4f} -> {last:.4f}, replicas {'in sync' if abs(hi + neg_lo) < 1e-9 else 'DIVERGED'}: "
          f"{'PASS' if ok else 'FAIL'}")
    shm.free(both)
    shm.free(check)
    dp.destroy()
    shm.finalize()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
