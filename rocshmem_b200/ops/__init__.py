"""Operations on symmetric tensors: collectives, MoE dispatch/combine, GEMMs and fused paths."""
from . import collectives  # noqa: F401
