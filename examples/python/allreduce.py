#!/usr/bin/env python
"""Symmetric tensors and a stream-ordered allreduce from Python.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/allreduce.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    shm.init(heap_size="1G", device=local)       # rendezvous through the torchrun store (or alone)
    me, n = shm.my_pe(), shm.n_pes()
    src = shm.zeros(1 << 20, torch.bfloat16)      # same offset in every PE's heap
    dst = shm.zeros(1 << 20, torch.bfloat16)
    src.fill_(me + 1)
    torch.cuda.synchronize()
    shm.barrier_all()
    coll.allreduce_async(dst, src, shm.OP_SUM)    # one kernel on the current stream
    torch.cuda.synchronize()
    ok = bool(torch.all(dst.float() == n * (n + 1) / 2))
    print(f"[PE {me}] allreduce: {'PASS' if ok else 'FAIL'}")
    shm.barrier_all()
    shm.finalize()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
