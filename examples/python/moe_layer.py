#!/usr/bin/env python
"""An expert-parallel MoE feed-forward layer: dispatch -> grouped GEMMs -> combine, checked against fp32.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/moe_layer.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.models import moe_ffn  # noqa: E402
from rocshmem_b200.ops import moe  # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    shm.init(heap_size="2G", device=local)
    me, n = shm.my_pe(), shm.n_pes()
    experts, top_k, hidden, inter, tokens = 8 * n, 4, 2048, 1024, 512
    layer = moe_ffn.MoEFeedForward(experts, top_k, hidden, inter, max_tokens=tokens, seed=1)
    x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(me)).to(torch.bfloat16)
    idx, w = moe.make_routing(tokens, experts, top_k, seed=10 + me)
    out = layer(x.cuda(), idx.cuda(), w.cuda())
    torch.cuda.synchronize()
    want = moe_ffn.reference_forward(x, idx, w, hidden, inter, seed=1, fp8_experts=layer.fp8_experts)
    err = (out.float().cpu() - want).abs().max().item()
    ok = err <= 5e-2 * want.abs().max().item() + 0.03 and shm.get_error()["count"] == 0
    print(f"[PE {me}] moe layer: max abs error {err:.4f}: {'PASS' if ok else 'FAIL'}")
    shm.barrier_all()
    shm.finalize()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
