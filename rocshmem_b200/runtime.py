"""Python face of the runtime: initialisation over a ``torch.distributed`` store, the symmetric heap
as torch tensors, teams, contexts and the host-side OpenSHMEM calls.

Reference counterparts: ``rocshmem_init`` / ``rocshmem_malloc`` / teams / contexts and the host API of
``include/rocshmem/rocshmem.hpp``; MPI is replaced by a key-value store (``TCPStore`` or the store of the
default process group) that the native runtime uses for every bootstrap exchange.

The symmetric heap is GPU memory, so this layer is also what replaces the reference examples' habit
of dereferencing ``rocshmem_malloc`` pointers on the CPU: tensors returned by :func:`empty` /
:func:`zeros` live on the heap, at the same offset on every PE.
"""
from __future__ import annotations

import ctypes
import datetime
import os
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch

from . import _native

# ---- constants mirrored from rocshmem_common.h -------------------------------------------------------
CMP_EQ, CMP_NE, CMP_GT, CMP_GE, CMP_LT, CMP_LE = range(6)
OP_SUM, OP_MAX, OP_MIN, OP_PROD, OP_AND, OP_OR, OP_XOR = range(7)
SIGNAL_SET, SIGNAL_ADD = 0, 1
AMO_FETCH, AMO_SWAP, AMO_CAS, AMO_ADD, AMO_AND, AMO_OR, AMO_XOR = range(7)
CTX_NOSTORE, CTX_SERIALIZED, CTX_WG_PRIVATE, CTX_SHARED = 1, 2, 4, 8
ALLREDUCE_AUTO, ALLREDUCE_ONE_SHOT, ALLREDUCE_TWO_SHOT, ALLREDUCE_NVLS, ALLREDUCE_LL = range(5)
COLL_PRE_SYNC = 1
SUCCESS, ERROR = 0, 1

_DTYPE_CODE = {
    torch.int8: 0, torch.uint8: 1, torch.int16: 2, torch.int32: 4, torch.int64: 6,
    torch.float32: 8, torch.float64: 9, torch.float16: 10, torch.bfloat16: 11,
}
for _name, _code in (("uint16", 3), ("uint32", 5), ("uint64", 7)):
    if hasattr(torch, _name):
        _DTYPE_CODE[getattr(torch, _name)] = _code


def dtype_code(dtype: torch.dtype) -> int:
    """Element type code of the untyped host engine (``rocshmem_dtype``) for a torch dtype."""
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"rocshmem_b200: unsupported dtype {dtype}") from None


@dataclass
class _State:
    initialised: bool = False
    device: Optional[torch.device] = None
    store: object = None
    prefix: str = ""
    allocations: Dict[int, int] = None  # data_ptr -> bytes
    heap_lo: int = 0                    # address range of the heaps of this process's PEs
    init_args: Dict[str, object] = None # keyword arguments of the last init (for a re-initialisation)
    heap_hi: int = 0


_state = _State(allocations={})
_init_count = 0


def _C():
    return _native.load()


# ---- lifecycle ---------------------------------------------------------------------------------------------

def init(store=None, rank: Optional[int] = None, world_size: Optional[int] = None, *,
         n_local: int = 1, device: Optional[int] = None, heap_size=None, backend: Optional[str] = None,
         timeout_s: float = 120.0, generation: Optional[int] = None, **overrides) -> None:
    """Collective initialisation.

    ``store`` is any ``torch.distributed`` store; when omitted, the store of the default process group
    is used if there is one, else a ``TCPStore`` is created from ``MASTER_ADDR`` / ``MASTER_PORT``
    (``RANK`` / ``WORLD_SIZE`` as set by torchrun), else the process runs alone. ``n_local > 1`` hosts
    several PEs in this process on one GPU. Keyword overrides use the names of the environment
    variables (``ROCSHMEM_HEAP_SIZE='64M'`` ...); ``heap_size`` and ``backend`` are shorthands. ``generation``
    names the key space inside the store; by default it counts the initialisations of this process, which agrees
    between processes that have lived through the same ones (a process that joins a running job passes the value it
    was told, see ``parallel.elastic``).
    """
    global _init_count
    C = _C()
    if C.is_initialized():
        raise RuntimeError("rocshmem_b200.init: already initialised")
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
    ov = {str(k): str(v) for k, v in overrides.items()}
    if heap_size is not None:
        ov["ROCSHMEM_HEAP_SIZE"] = str(heap_size)
    if backend is not None:
        ov["ROCSHMEM_BACKEND"] = backend
    want_cuda = ov.get("ROCSHMEM_BACKEND", os.environ.get("ROCSHMEM_BACKEND", "auto")) != "host"
    if device is None:
        device = int(os.environ.get("LOCAL_RANK", "0"))
    if want_cuda and torch.cuda.is_available():
        device = device % torch.cuda.device_count()
        torch.cuda.set_device(device)
        _state.device = torch.device("cuda", device)
    else:
        _state.device = torch.device("cpu")
    timeout_ms = int(timeout_s * 1000)
    if world_size > 1:
        if store is None:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                store = dist.distributed_c10d._get_default_store()
            else:
                # Under torchrun the agent already serves a store on MASTER_PORT; workers only connect.
                agent_store = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "") == "True"
                store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"),
                                      int(os.environ.get("MASTER_PORT", "29500")), world_size,
                                      rank == 0 and not agent_store,
                                      timeout=datetime.timedelta(seconds=timeout_s))
        _init_count = _init_count + 1 if generation is None else int(generation)
        prefix = f"rocshmem_b200/{_init_count}/"
        wait = datetime.timedelta(milliseconds=timeout_ms)

        def put(key: str, value: bytes) -> None:
            store.set(prefix + key, value)

        def get(key: str, ms: int) -> bytes:
            store.wait([prefix + key], datetime.timedelta(milliseconds=ms) if ms > 0 else wait)
            return bytes(store.get(prefix + key))

        _state.store = store
        _state.prefix = prefix
        C.init_with_store(rank, world_size, put, get, ov, n_local, device, timeout_ms)
    else:
        C.init_file(0, 1, "", ov, n_local, device, timeout_ms)
    _state.initialised = True
    _state.allocations = {}
    _state.init_args = dict(n_local=n_local, device=device if _state.device.type == "cuda" else None,
                            timeout_s=timeout_s, **ov)
    first = C.my_pe()                   # local PE 0 is current right after init
    _state.heap_lo = C.heap_base(first)
    _state.heap_hi = C.heap_base(first + n_local - 1) + C.heap_size()


def bootstrap_store():
    """The ``torch.distributed`` store the last multi-process ``init`` exchanged its descriptors through (``None``
    for a single process). It outlives ``finalize``, so a smaller or larger world can be initialised over it."""
    return _state.store


def generation() -> int:
    """The key-space number of the last multi-process ``init`` (see its ``generation`` argument)."""
    return _init_count


def last_init_arguments() -> dict:
    """Keyword arguments of the last ``init`` (PEs per process, device, time-out, configuration overrides)."""
    return dict(_state.init_args or {})


def finalize() -> None:
    """Collective tear-down: frees the heap mappings, stops the proxy, checks the guard regions."""
    C = _C()
    if C.is_initialized():
        if C.is_cuda():
            torch.cuda.synchronize()
        C.finalize()
    _state.initialised = False
    _state.allocations = {}
    _state.heap_lo = _state.heap_hi = 0


def is_initialized() -> bool:
    """True between ``init`` and ``finalize``."""
    return _C().is_initialized()


def my_pe() -> int:
    """This process's PE number (the current local PE when several are hosted)."""
    return _C().my_pe()


def n_pes() -> int:
    """Total number of PEs."""
    return _C().n_pes()


def n_local_pes() -> int:
    """PEs hosted by this process (1 unless ``init(n_local=...)``)."""
    return _C().n_local()


def set_local_pe(index: int) -> None:
    """With several PEs per process: choose the PE that later host calls of this thread act for."""
    _C().set_local_pe(index)


def is_cuda() -> bool:
    """True when the heap is GPU memory (CUDA backend), False on the CPU shared-memory backend."""
    return _C().is_cuda()


def device() -> torch.device:
    """The torch device that holds this PE's heap."""
    return _state.device


def nvls_available() -> bool:
    """True when the heap is also mapped through an NVLink multicast object (``multimem`` collectives)."""
    return _C().nvls_available()


# ---- heap as tensors ------------------------------------------------------------------------------------------

class _CudaBlob:
    """Exposes a raw device address through ``__cuda_array_interface__`` so torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_address(ptr: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
    """A tensor view of heap memory at ``ptr`` (no ownership)."""
    numel = 1
    for s in shape:
        numel *= int(s)
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    if nbytes == 0:
        return torch.empty(tuple(shape), dtype=dtype, device=_state.device)
    if _C().is_cuda():
        raw = torch.as_tensor(_CudaBlob(ptr, nbytes), device=_state.device)
    else:
        buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
        raw = torch.frombuffer(buf, dtype=torch.uint8)
    return raw.view(dtype).view(tuple(shape))


def empty(shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Collective ``rocshmem_malloc``: a tensor at the same heap offset on every PE."""
    if isinstance(shape, int):
        shape = (shape,)
    numel = 1
    for s in shape:
        numel *= int(s)
    nbytes = max(1, numel * torch.empty((), dtype=dtype).element_size())
    ptr = _C().malloc(nbytes)
    if ptr == 0:
        raise MemoryError(f"rocshmem_b200: symmetric heap exhausted ({nbytes} bytes requested, "
                          f"{_C().heap_avail()} available)")
    _state.allocations[ptr] = nbytes
    return tensor_from_address(ptr, shape, dtype)


def zeros(shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Collective: a zero-filled symmetric tensor (same heap offset on every PE)."""
    t = empty(shape, dtype)
    for l in range(n_local_pes()):
        local_view(t, l).zero_()
    if is_cuda():
        torch.cuda.current_stream().synchronize()
    barrier_all()
    return t


def free(t: torch.Tensor) -> None:
    """Collective ``rocshmem_free`` of a tensor obtained from :func:`empty` / :func:`zeros`."""
    ptr = t.data_ptr()
    if ptr not in _state.allocations:
        raise ValueError("rocshmem_b200.free: tensor does not start a symmetric allocation")
    del _state.allocations[ptr]
    _C().free(ptr)


def free_all(tensors) -> None:
    """Collective: :func:`free` every tensor of an iterable (``None`` entries are skipped), last allocated first."""
    for t in reversed([t for t in tensors if t is not None]):
        free(t)


def local_view(t: torch.Tensor, local_index: int) -> torch.Tensor:
    """The copy of symmetric tensor ``t`` that belongs to local PE ``local_index`` of this process."""
    if local_index == 0:
        return t
    C = _C()
    ptr = C.ptr(t.data_ptr(), C.first_pe() + local_index)
    return tensor_from_address(ptr, t.shape, t.dtype)


def peer_address(t: torch.Tensor, pe: int) -> int:
    """Address of ``t`` on ``pe`` inside this process's mapping of the window (``rocshmem_ptr``)."""
    return _C().ptr(t.data_ptr(), pe)


def heap_info() -> dict:
    """Heap size, stride between PEs, bytes used and available, backend name, NVLS availability."""
    C = _C()
    return {"size": C.heap_size(), "stride": C.heap_stride(), "used": C.heap_used(),
            "avail": C.heap_avail(), "backend": C.backend_name(), "nvls": C.nvls_available()}


# ---- teams and contexts -------------------------------------------------------------------------------------------

class Team:
    """A strided set of PEs (``rocshmem_team_t``)."""

    def __init__(self, handle: int):
        self.handle = handle

    @property
    def valid(self) -> bool:
        """False for the invalid team (returned by a split to PEs that are not members)."""
        return self.handle != 0

    def n_pes(self) -> int:
        """Number of members."""
        return _C().team_n_pes(self.handle)

    def my_pe(self) -> int:
        """My index in the team, -1 when I am not a member."""
        return _C().team_my_pe(self.handle)

    def translate_pe(self, pe: int, dst: "Team") -> int:
        """Index in ``dst`` of the PE that has index ``pe`` in this team, -1 when it is not a member of ``dst``."""
        return _C().team_translate_pe(self.handle, pe, dst.handle)

    def split_strided(self, start: int, stride: int, size: int) -> "Team":
        """Collective over this team. Returns an invalid team on PEs that are not members; raises
        ``ValueError`` for an impossible request and ``RuntimeError`` when no team slot is free."""
        rc, h = _C().team_split_strided(self.handle, start, stride, size)
        if rc != 0:
            if _C().num_user_teams() >= team_capacity() - 1:
                raise RuntimeError("rocshmem_b200: no free team slot")
            raise ValueError(f"rocshmem_b200: invalid team split ({start}, {stride}, {size})")
        return Team(h)

    def has_nvls(self) -> bool:
        """True when the team has an NVLink multicast mapping of the heap that spans exactly its members (the
        switch-side allreduce, all-gather and broadcast kernels are then used for it). Split teams get one when
        every member is a process of its own and ``ROCSHMEM_TEAM_NVLS`` is not 0."""
        return bool(self.handle) and _C().team_has_nvls(self.handle)

    def sync(self) -> int:
        """Host-side team barrier without the completion of outstanding operations; 0 on success."""
        return _C().team_sync(self.handle)

    def destroy(self) -> None:
        """Release the team's slot. Collective over the members when the team has a multicast object of its own
        (:meth:`has_nvls` on a split team): the call waits for the GPU's queued work and for the other members,
        so every member destroys its teams in the same order; local otherwise."""
        if self.handle:
            _C().team_destroy(self.handle)
            self.handle = 0

    def __repr__(self) -> str:
        return f"Team(handle=0x{self.handle:x})"


def team_world() -> Team:
    """The team of all PEs."""
    return Team(_C().team_world())


def team_capacity() -> int:
    """Number of team slots (``ROCSHMEM_MAX_NUM_TEAMS``), the world team included."""
    return _C().config_from_env({})["max_teams"]


class Context:
    """A host context: an ordering and completion domain backed by its own stream."""

    def __init__(self, options: int = 0, team: Optional[Team] = None):
        if team is None:
            rc, c, t = _C().ctx_create(options)
        else:
            rc, c, t = _C().team_create_ctx(team.handle, options)
        if rc != 0:
            raise RuntimeError("rocshmem_b200: host context pool exhausted")
        self.handle, self.team_handle = c, t

    def quiet(self) -> None:
        """Wait until every operation issued on this context has completed."""
        _C().quiet(self.handle, self.team_handle)

    def destroy(self) -> None:
        """Complete outstanding operations and release the context."""
        if self.handle:
            _C().ctx_destroy(self.handle, self.team_handle)
            self.handle = 0


def _ctx_args(ctx: Optional[Context]):
    return (ctx.handle, ctx.team_handle) if ctx is not None else (0, 0)


# ---- host-side OpenSHMEM calls -----------------------------------------------------------------------------------------

def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _check_contig(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_contiguous():
            raise ValueError("rocshmem_b200: tensors must be contiguous")


def is_symmetric(t: torch.Tensor) -> bool:
    """True when the tensor's memory lies inside the symmetric heap of one of this process's PEs."""
    ptr = t.data_ptr()
    return _state.heap_lo <= ptr and ptr + t.numel() * t.element_size() <= _state.heap_hi and _state.heap_hi > 0


def require_symmetric(**tensors: torch.Tensor) -> None:
    """Raise ``ValueError`` naming the first argument that is not a contiguous tensor on the symmetric heap.
    Kernels derive peer addresses from these pointers, so anything else would make them touch foreign memory."""
    for name, t in tensors.items():
        if t.numel() == 0:
            continue                    # nothing is read or written; the collectives treat it as a no-op
        if not t.is_contiguous():
            raise ValueError(f"rocshmem_b200: `{name}` must be contiguous")
        if not is_symmetric(t):
            raise ValueError(f"rocshmem_b200: `{name}` must live on the symmetric heap (rocshmem_b200.empty / zeros)")


def putmem(dest: torch.Tensor, source: torch.Tensor, pe: int, ctx: Optional[Context] = None,
           nbi: bool = False) -> None:
    """Copy ``source`` (any local tensor) into symmetric ``dest`` on ``pe``."""
    _check_contig(dest, source)
    n = min(_nbytes(dest), _nbytes(source))
    fn = _C().putmem_nbi if nbi else _C().putmem
    fn(dest.data_ptr(), source.data_ptr(), n, pe, *_ctx_args(ctx))


def getmem(dest: torch.Tensor, source: torch.Tensor, pe: int, ctx: Optional[Context] = None,
           nbi: bool = False) -> None:
    """Copy symmetric ``source`` on ``pe`` into local ``dest``."""
    _check_contig(dest, source)
    n = min(_nbytes(dest), _nbytes(source))
    fn = _C().getmem_nbi if nbi else _C().getmem
    fn(dest.data_ptr(), source.data_ptr(), n, pe, *_ctx_args(ctx))


def _bits(value, dtype: torch.dtype) -> int:
    t = torch.tensor([value], dtype=dtype)
    width = t.element_size()
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[width]
    return int(t.view(view).item()) & ((1 << (8 * width)) - 1)


def _from_bits(bits: int, dtype: torch.dtype):
    width = torch.empty((), dtype=dtype).element_size()
    bits &= (1 << (8 * width)) - 1
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[width]
    signed = bits - (1 << (8 * width)) if (view != torch.uint8 and bits >> (8 * width - 1)) else bits
    return torch.tensor([signed], dtype=view).view(dtype).item()


def _element_ptr(t: torch.Tensor, index: int) -> int:
    return t.data_ptr() + index * t.element_size()


def atomic(op: int, target: torch.Tensor, value=0, pe: int = 0, cond=0, index: int = 0,
           ctx: Optional[Context] = None):
    """Atomic ``op`` (``AMO_*``) on element ``index`` of symmetric ``target`` at ``pe``; returns the
    previous value."""
    code = dtype_code(target.dtype)
    old = _C().amo(op, code, _element_ptr(target, index), _bits(value, target.dtype),
                   _bits(cond, target.dtype), pe, *_ctx_args(ctx))
    return _from_bits(old, target.dtype)


def atomic_fetch_add(target, value, pe, index=0, ctx=None):
    """Add ``value`` to element ``index`` of ``target`` on ``pe``; returns the previous value."""
    return atomic(AMO_ADD, target, value, pe, index=index, ctx=ctx)


def atomic_compare_swap(target, cond, value, pe, index=0, ctx=None):
    """Store ``value`` if the element equals ``cond``; returns the previous value."""
    return atomic(AMO_CAS, target, value, pe, cond=cond, index=index, ctx=ctx)


def atomic_swap(target, value, pe, index=0, ctx=None):
    """Store ``value``; returns the previous value."""
    return atomic(AMO_SWAP, target, value, pe, index=index, ctx=ctx)


def atomic_fetch(target, pe, index=0, ctx=None):
    """Atomic read of element ``index`` of ``target`` on ``pe``."""
    return atomic(AMO_FETCH, target, 0, pe, index=index, ctx=ctx)


def wait_until(ivar: torch.Tensor, cmp: int, value, index: int = 0) -> int:
    """Bounded wait on a local symmetric variable; ``SUCCESS`` or ``ERROR`` (time-out)."""
    return _C().wait_until(_element_ptr(ivar, index), dtype_code(ivar.dtype), cmp, _bits(value, ivar.dtype))


def test(ivar: torch.Tensor, cmp: int, value, index: int = 0) -> bool:
    """One non-blocking evaluation of the comparison ``wait_until`` would wait for."""
    return bool(_C().test(_element_ptr(ivar, index), dtype_code(ivar.dtype), cmp, _bits(value, ivar.dtype)))


def wait_until_all(ivars: torch.Tensor, cmp: int, values, status: Sequence[int] = ()) -> None:
    """Wait until every element (whose ``status`` entry is 0) satisfies the comparison."""
    vec = isinstance(values, (list, tuple))
    vals = [_bits(v, ivars.dtype) for v in (values if vec else [values])]
    _C().wait_until_all(ivars.data_ptr(), ivars.numel(), list(status), dtype_code(ivars.dtype), cmp, vals, vec)


def wait_until_any(ivars: torch.Tensor, cmp: int, values, status: Sequence[int] = ()) -> int:
    """Wait until one element satisfies the comparison; returns its index (``SIZE_MAX`` for an empty set)."""
    vec = isinstance(values, (list, tuple))
    vals = [_bits(v, ivars.dtype) for v in (values if vec else [values])]
    r = _C().wait_until_any(ivars.data_ptr(), ivars.numel(), list(status), dtype_code(ivars.dtype), cmp, vals, vec)
    return -1 if r >= (1 << 63) else r


def wait_until_some(ivars: torch.Tensor, cmp: int, values, status: Sequence[int] = ()):
    """Wait until at least one element satisfies the comparison; returns the indices of all that do."""
    vec = isinstance(values, (list, tuple))
    vals = [_bits(v, ivars.dtype) for v in (values if vec else [values])]
    return _C().wait_until_some(ivars.data_ptr(), ivars.numel(), list(status), dtype_code(ivars.dtype), cmp, vals, vec)


def fence() -> None:
    """Order this PE's earlier puts before its later ones, per destination."""
    _C().fence()


def quiet(ctx: Optional[Context] = None) -> None:
    """Wait until every operation issued on the context (default context if none) has completed."""
    _C().quiet(*_ctx_args(ctx))


def barrier_all() -> None:
    """Complete outstanding operations, then synchronise all PEs."""
    _C().barrier_all()


def sync_all() -> None:
    """Synchronise all PEs without completing outstanding operations."""
    _C().sync_all()


def get_error(local: int = -1) -> dict:
    """First error recorded by a bounded wait or debug check on this PE (``kind == 0``: none)."""
    return _C().get_error(local)


ERROR_KINDS = {0: "none", 1: "wait_until timed out", 2: "barrier / collective flag wait timed out", 3: "PE out of range",
               4: "address outside the symmetric heap", 5: "device context pool exhausted",
               6: "reverse-offload ring timed out", 7: "grid barrier timed out", 8: "library kernel gave up on an internal wait"}

# The `where` field of an error record: which operation recorded it.
ERROR_SITES = {
    0: "a host API call", 1: "reverse-offload ring: no free slot", 2: "reverse-offload ring: no completion",
    10: "putmem", 11: "getmem", 12: "p", 13: "g", 20: "atomic add / fetch_add", 21: "atomic swap / set",
    22: "atomic compare_swap", 23: "atomic fetch", 24: "atomic and", 25: "atomic or", 26: "atomic xor",
    30: "put with signal", 40: "wait_until", 41: "wait_until_any", 42: "wait_until_some",
    50: "team barrier / sync", 60: "library collective: peer block did not arrive", 61: "library kernel: grid barrier",
    70: "MoE dispatch: count exchange", 80: "all-gather -> GEMM: rows of a peer did not arrive",
    81: "all-gather -> GEMM (two CTAs per tile): rows of a peer did not arrive",
    90: "ticket lock", 91: "spin lock", 92: "rocshmemx_grid_sync",
}


def debug_print_ring(first: int = 0, count: int = 8) -> None:
    """Print ``count`` command slots of the reverse-offload ring, starting at ``first``, to standard error: state,
    operation, PE, addresses, size. Says so in one line when the process runs no proxy thread
    (``ROCSHMEM_USE_PROXY`` off). Counterpart of ``debug_print_sq`` (include/rocshmem/rocshmem_debug.hpp:28-30)."""
    _C().debug_print_ring(int(first), int(count))


def describe_error(err: Optional[dict] = None) -> str:
    """One line of plain words for an error record (the current one of this PE by default)."""
    err = get_error() if err is None else err
    if not err.get("count"):
        return "no error recorded"
    kind = ERROR_KINDS.get(err.get("kind"), f"kind {err.get('kind')}")
    site = ERROR_SITES.get(err.get("where"), f"site {err.get('where')}")
    peer = f", peer PE {err['pe']}" if err.get("pe", -1) >= 0 else ""
    return (f"{kind} in {site}{peer}: expected {err.get('expected')}, observed {err.get('observed')} at address "
            f"0x{err.get('addr', 0):x} ({err['count']} error(s) since the record was cleared)")


def clear_error() -> None:
    """Reset the first-error record of this PE."""
    _C().clear_error()


def set_wait_timeout_ms(ms: int) -> None:
    """Change the budget of host- and device-side waits (must be positive)."""
    _C().set_wait_timeout_ms(ms)
