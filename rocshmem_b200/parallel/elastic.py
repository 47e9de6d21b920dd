"""Shrinking and growing a running job: ranks leave or join between steps, the others re-initialise a world of the new
size and carry on.

The reference has no recovery of any kind (an error aborts the job, ``src/ipc/backend_ipc.cpp:28-34``). Teams
cannot express an arbitrary set of survivors either: OpenSHMEM teams are strided, and the survivors of a job that
lost rank 2 of 4 are not. So the world itself is rebuilt: every rank of the old world calls :func:`shrink` at the same
point between two steps, with nothing in flight; those that leave say so; everybody finalises the runtime (the last
collective the old world performs); the survivors initialise a new runtime over the same store with dense PE
numbers in the old order. Heap contents do not survive a re-initialisation: take a
``rocshmem_b200.utils.checkpoint.snapshot`` before and ``restore`` it into the tensors allocated afterwards.
:func:`grow` and :func:`join` are the opposite direction: the members re-initialise with a larger world and new
processes take the additional PE numbers.

This is the host-side half of failure handling: a rank that decides to go (draining a node, a failed health check
seen between steps), or one that vanished between steps and whose heartbeat went stale (``dead=``). A rank that dies
in the middle of a step is a different matter: its peers' waits
run out, their error records say which PE did not answer (``describe_error``), and the job decides on the host what
to do next; no kernel waits for ever in either case.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

from .. import runtime as rt
from .membership import Membership


def shrink(membership: Membership, leaving: bool = False, dead: Sequence[int] = ()) -> Optional[Tuple[int, int]]:
    """Collective over the current world. Returns ``(new_pe, new_n_pes)`` on survivors, ``None`` on ranks that left
    (their runtime is finalised; they may exit). Requires a multi-process runtime initialised over a store that
    survives the departure (under torchrun the agent serves it; otherwise the rank that hosts it must stay).

    ``dead``: ranks that went away without saying so (every survivor passes the same list, e.g. from
    ``membership.stale(age)`` with an age that all agree on). They are recorded as gone on their behalf; the old
    world's last synchronisation then runs into its time-out (the bootstrap time-out given to ``init``) instead of
    completing, which is reported on stderr and otherwise harmless."""
    store = rt.bootstrap_store()
    if store is None or not rt.is_initialized():
        raise RuntimeError("shrink needs a runtime that was initialised over a store")
    args = rt.last_init_arguments()
    old_pe = membership.rank
    if leaving:
        membership.announce_leave()
    for r in dead:
        membership.declare_left(int(r))
    # finalize synchronises the old world: every leave record is in the store before anybody goes on
    rt.finalize()
    if leaving:
        return None
    alive = membership.alive()
    if old_pe not in alive:
        raise RuntimeError("this rank was declared gone by its own record")
    new_pe, new_n = alive.index(old_pe), len(alive)
    timeout_s = args.pop("timeout_s", 120.0)
    n_local = args.pop("n_local", 1)
    device = args.pop("device", None)
    rt.init(store, new_pe, new_n, n_local=n_local, device=device, timeout_s=timeout_s, **args)
    return new_pe, new_n


_GROW_KEY = "rocshmem_b200/grow"


def grow(new_world_size: int) -> Tuple[int, int]:
    """Collective over the current world (one PE per process): finalise and re-initialise with ``new_world_size``
    PEs. The current members keep their PE numbers; the additional ones are processes that call :func:`join` with
    PE numbers from the old size upwards. Returns ``(pe, new_world_size)``. Heap contents do not survive (snapshot
    and restore, as for :func:`shrink`)."""
    store = rt.bootstrap_store()
    if store is None or not rt.is_initialized():
        raise RuntimeError("grow needs a runtime that was initialised over a store")
    if rt.n_local_pes() != 1 or new_world_size <= rt.n_pes():
        raise ValueError("grow needs one PE per process and a larger world")
    args = rt.last_init_arguments()
    pe, gen = rt.my_pe(), rt.generation() + 1
    if pe == 0:
        store.set(_GROW_KEY, f"{gen}:{new_world_size}")
    rt.finalize()
    rt.init(store, pe, new_world_size, n_local=args.pop("n_local", 1), device=args.pop("device", None),
            timeout_s=args.pop("timeout_s", 120.0), generation=gen, **args)
    return pe, new_world_size


def join(store, pe: int, timeout_s: float = 120.0, **init_arguments) -> Tuple[int, int]:
    """Called by a new process: wait until the running job announces that it grows, then initialise as PE ``pe`` of
    the new world over ``store`` (a client connection to the job's store). ``init_arguments`` are those of
    ``rocshmem_b200.init`` (heap size, backend, device ...) and must match the running job's."""
    import datetime
    store.wait([_GROW_KEY], datetime.timedelta(seconds=timeout_s))
    gen, n = (int(v) for v in bytes(store.get(_GROW_KEY)).decode().split(":"))
    if not gen > 0 or not 0 <= pe < n:
        raise ValueError(f"cannot join as PE {pe} of {n}")
    rt.init(store, pe, n, timeout_s=timeout_s, generation=gen, **init_arguments)
    return pe, n
