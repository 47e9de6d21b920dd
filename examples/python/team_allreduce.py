#!/usr/bin/env python
"""Teams: the PEs split into a lower and an upper half and into even and odd PEs, every PE reduces over each of
its two teams, and the teams are destroyed again. On GPUs a split team whose members are processes of their own
gets an NVLink multicast object (``Team.has_nvls()``), and teams of four or more then reduce inside the switch.
Runs on GPUs and, without them, on the CPU shared-memory backend.

    python -m rocshmem_b200.launch -n 4 python examples/python/team_allreduce.py
    python -m rocshmem_b200.launch -n 4 --backend host python examples/python/team_allreduce.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import rocshmem_b200 as shm  # noqa: E402
from rocshmem_b200.ops import collectives as coll  # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local % torch.cuda.device_count())
    shm.init(heap_size="64M", device=local)
    me, n = shm.my_pe(), shm.n_pes()
    world = shm.team_world()
    half = max(1, n // 2)
    # Splits are collective over the parent team: every PE takes part in each of them and keeps the teams it is in.
    splits = {"lower": (0, 1, half), "upper": (half, 1, n - half), "even": (0, 2, (n + 1) // 2), "odd": (1, 2, n // 2)}
    teams = {name: world.split_strided(*triple) for name, triple in splits.items() if triple[2] > 0}
    src = shm.zeros(1024, torch.float32)
    dst = shm.zeros(1024, torch.float32)
    src.fill_(float(me + 1))
    if shm.is_cuda():
        torch.cuda.synchronize()
    shm.barrier_all()
    ok = True
    mine = []
    for name, team in teams.items():
        if not team.valid:                      # not a member: the split returned the invalid team
            continue
        start, stride, size = splits[name]
        members = [start + i * stride for i in range(size)]
        assert team.my_pe() == members.index(me) and team.n_pes() == size
        if shm.is_cuda():
            coll.allreduce_async(dst, src, shm.OP_SUM, team=team)      # one kernel on the current stream
            torch.cuda.synchronize()
        else:
            coll.reduce(dst, src, shm.OP_SUM, team)                    # the host API's blocking form
        want = float(sum(p + 1 for p in members))
        ok = ok and bool(torch.all(dst.cpu() == want))
        mine.append(f"{name}{' (switch)' if team.has_nvls() else ''}")
    shm.barrier_all()
    for team in teams.values():
        if team.valid:
            team.destroy()                      # collective over the team's members
    ok = ok and shm.get_error()["count"] == 0
    print(f"pe {me}/{n}: member of {', '.join(mine)}: {'PASS' if ok else 'FAIL'}")
    shm.free(dst)
    shm.free(src)
    shm.finalize()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
