"""Host-side membership and failure detection over a ``torch.distributed`` store.

The reference has no failure handling: an MPI or HIP error aborts the process and every device wait
spins for ever (``src/ipc/backend_ipc.cpp:28-34``, ``src/context_tmpl_device.hpp:204``). Here the
device side is covered by bounded waits that return a status; this module covers the host side:

* every rank publishes a heartbeat and, when it leaves on purpose, a leave record;
* before launching the next step a rank asks :meth:`Membership.alive` / :meth:`Membership.stale` and
  learns about a departed or silent peer on the CPU, with no kernel or collective in flight;
* survivors then continue on a team that excludes the missing rank (team splits and active-set
  collectives involve only the members of the new set).

A rank may leave only between steps, after ``quiet``; it must keep its process (and so its heap
mapping) alive until the survivors have stopped addressing it, which :meth:`post` / :meth:`wait_for`
coordinate.
"""
from __future__ import annotations

import datetime
import os
import time
from typing import List, Optional

import torch.distributed as dist


class Membership:
    """Heartbeats and departure notes of the ranks of a job in a key-value store, for failure detection between steps."""

    def __init__(self, store, rank: int, world_size: int, prefix: str = "membership"):
        self.store = store
        self.rank = rank
        self.world_size = world_size
        self.prefix = prefix
        self.heartbeat()

    @classmethod
    def from_env(cls, prefix: str = "membership", path: Optional[str] = None) -> "Membership":
        """A file-backed store shared by the ranks of one node (``ROCSHMEM_TEST_TMP`` or ``path``)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        base = path or os.environ.get("ROCSHMEM_TEST_TMP") or "/tmp"
        store = dist.FileStore(os.path.join(base, f"rocshmem_b200_{prefix}.store"), world)
        return cls(store, rank, world, prefix)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    # ---- liveness ----------------------------------------------------------------------------------
    def heartbeat(self) -> None:
        """Record that this rank is alive now."""
        self.store.set(self._key("hb", self.rank), repr(time.time()))

    def announce_leave(self) -> None:
        """Record that this rank leaves the job (call between steps, with nothing in flight)."""
        self.store.set(self._key("left", self.rank), "1")

    def declare_left(self, rank: int) -> None:
        """Record on behalf of ``rank`` that it is gone (a peer that stopped sending heartbeats). Idempotent."""
        self.store.set(self._key("left", rank), "1")

    def has_left(self, rank: int) -> bool:
        """True once ``rank`` has announced its departure."""
        return bool(self.store.check([self._key("left", rank)]))

    def alive(self) -> List[int]:
        """Ranks that have not announced their departure."""
        return [r for r in range(self.world_size) if not self.has_left(r)]

    def stale(self, older_than_s: float) -> List[int]:
        """Ranks whose last heartbeat is older than ``older_than_s`` seconds (or missing)."""
        now = time.time()
        out = []
        for r in range(self.world_size):
            key = self._key("hb", r)
            if not self.store.check([key]):
                out.append(r)
                continue
            try:
                last = float(bytes(self.store.get(key)).decode())
            except ValueError:
                last = 0.0
            if now - last > older_than_s:
                out.append(r)
        return out

    def wait_for_change(self, expected_alive: int, timeout_s: float = 30.0) -> List[int]:
        """Poll until exactly ``expected_alive`` ranks remain; raises ``TimeoutError`` otherwise."""
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            a = self.alive()
            if len(a) == expected_alive:
                return a
            time.sleep(0.02)
        raise TimeoutError(f"membership did not reach {expected_alive} live ranks: {self.alive()}")

    # ---- simple rendezvous -----------------------------------------------------------------------------
    def post(self, name: str) -> None:
        """Set a named one-shot flag."""
        self.store.set(f"{self.prefix}/post/{name}", "1")

    def wait_for(self, name: str, timeout_s: float = 60.0) -> None:
        """Block until the named flag has been posted (raises on time-out)."""
        self.store.wait([f"{self.prefix}/post/{name}"], datetime.timedelta(seconds=timeout_s))
