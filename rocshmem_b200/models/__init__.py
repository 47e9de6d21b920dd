"""Model blocks assembled from the package's kernels: a tensor-parallel SwiGLU MLP (all-gather -> GEMM,
GEMM -> reduce-scatter) and an expert-parallel MoE feed-forward layer (dispatch -> grouped GEMMs -> combine)."""
from .moe_ffn import MoEFeedForward  # noqa: F401
from .tp_mlp import TensorParallelMLP, TensorParallelMLPFp8  # noqa: F401
