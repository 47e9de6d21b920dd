"""rocshmem_b200: a Blackwell-native GPU-initiated OpenSHMEM runtime with a PyTorch layer.

The C++/CUDA API (``csrc/include/rocshmem/rocshmem.h``) follows the public surface of ROCm/rocSHMEM;
this package adds symmetric tensors, teams, host-side OpenSHMEM calls and stream-ordered collective,
MoE and tensor-parallel operations on top of the same runtime.
"""
from .runtime import (  # noqa: F401
    ALLREDUCE_AUTO, ALLREDUCE_LL, ALLREDUCE_NVLS, ALLREDUCE_ONE_SHOT, ALLREDUCE_TWO_SHOT, AMO_ADD, AMO_AND, AMO_CAS,
    AMO_FETCH, AMO_OR, AMO_SWAP, AMO_XOR, CMP_EQ, CMP_GE, CMP_GT, CMP_LE, CMP_LT, CMP_NE, CTX_NOSTORE,
    ERROR, OP_AND, OP_MAX, OP_MIN, OP_OR, OP_PROD, OP_SUM, OP_XOR, SIGNAL_ADD, SIGNAL_SET, SUCCESS,
    Context, Team, atomic, atomic_compare_swap, atomic_fetch, atomic_fetch_add, atomic_swap,
    barrier_all, clear_error, debug_print_ring, describe_error, device, empty, fence, finalize, free, free_all, get_error, getmem, heap_info, init,
    is_cuda, is_initialized, is_symmetric, require_symmetric, local_view, my_pe, n_local_pes, n_pes, nvls_available, peer_address,
    putmem, quiet, set_local_pe, set_wait_timeout_ms, sync_all, team_world, tensor_from_address, test,
    wait_until, wait_until_all, wait_until_any, wait_until_some, zeros,
)

__version__ = "0.1.0"
