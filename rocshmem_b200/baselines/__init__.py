"""Library baselines the package's kernels are measured against: NCCL collectives, NCCL + cuBLAS
tensor-parallel MLP, and an NCCL all-to-all MoE layer. Everything here calls library kernels only
(``torch.distributed`` / ``torch.matmul``); nothing here is used by the package's own operations."""
from .nccl_collectives import allreduce, allgather, alltoall, broadcast  # noqa: F401
from .tp_mlp import NcclTensorParallelMLP  # noqa: F401
from .moe import NcclMoEFeedForward  # noqa: F401
