#!/usr/bin/env python
"""A tensor-parallel SwiGLU MLP block: all-gather -> GEMM -> SwiGLU and GEMM -> reduce-scatter, each one kernel.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/tp_mlp.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.models import tp_mlp  # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    shm.init(heap_size="2G", device=local)
    me, n = shm.my_pe(), shm.n_pes()
    d_model, d_ff, m_shard = 2048, 1024 * n, 256          # every rank holds 256 tokens and d_ff / n of the hidden units
    mlp = tp_mlp.TensorParallelMLP(d_model, d_ff, m_shard, seed=3)
    shards = [(torch.randn(m_shard, d_model, generator=torch.Generator().manual_seed(p)) * 0.5).to(torch.bfloat16)
              for p in range(n)]
    out = mlp(shards[me].cuda())                            # this rank's 256 rows of the block's output
    torch.cuda.synchronize()
    want = tp_mlp.reference_forward(torch.cat(shards), n, d_model, d_ff, seed=3)[me * m_shard:(me + 1) * m_shard]
    err = (out.float().cpu() - want).abs().max().item()
    ok = err <= 2e-2 * want.abs().max().item() + 0.05 and shm.get_error()["count"] == 0
    print(f"[PE {me}] tensor-parallel MLP: max abs error {err:.4f}: {'PASS' if ok else 'FAIL'}")
    shm.barrier_all()
    shm.finalize()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
