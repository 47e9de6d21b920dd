"""Process launcher for programs of this runtime, the counterpart of ``mpirun -np N ./prog`` for the reference:

    python -m rocshmem_b200.launch -n 4 ./examples/build/allreduce
    python -m rocshmem_b200.launch -n 2 --backend host ./my_host_program arg1 arg2
    python -m rocshmem_b200.launch -n 8 python train.py

Starts ``N`` copies of the command on this node with ``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK``, ``MASTER_ADDR``
(127.0.0.1), ``MASTER_PORT`` and a fresh ``ROCSHMEM_BOOTSTRAP_DIR`` in their environment, which is all that
``rocshmem_init()`` (C++) and ``rocshmem_b200.init()`` (Python) need. Output lines are prefixed with the rank. If a
process fails, the others are terminated and the launcher exits with that process's code. ``torch.distributed.run``
does the same job for Python programs and for C++ programs with ``--no-python``; this launcher has no dependency
on torch and also takes care of the rendezvous directory.
"""
from __future__ import annotations

import argparse
import os
import shutil
import signal
import socket
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _pump(rank: int, stream, out, tag: bool) -> None:
    for line in iter(stream.readline, ""):
        out.write(f"[{rank}] {line}" if tag else line)
        out.flush()
    stream.close()


def launch(command: List[str], nprocs: int, backend: Optional[str] = None, local_pes: int = 1,
           timeout_s: Optional[float] = None, tag_output: bool = True, extra_env: Optional[dict] = None,
           out=None) -> int:
    """Run ``command`` as ``nprocs`` ranks; returns 0 when all exit with 0, else the first non-zero exit code
    (124 on time-out)."""
    out = out or sys.stdout
    port = _free_port()
    kv = tempfile.mkdtemp(prefix="rocshmem_b200_launch_")
    procs, pumps = [], []
    try:
        for r in range(nprocs):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(nprocs), LOCAL_RANK=str(r), LOCAL_WORLD_SIZE=str(nprocs),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), ROCSHMEM_BOOTSTRAP_DIR=kv)
            if backend:
                env["ROCSHMEM_BACKEND"] = backend
            if local_pes > 1:
                env["ROCSHMEM_LOCAL_PES"] = str(local_pes)
            env.update(extra_env or {})
            p = subprocess.Popen(command, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                 start_new_session=True)
            procs.append(p)
            t = threading.Thread(target=_pump, args=(r, p.stdout, out, tag_output), daemon=True)
            t.start()
            pumps.append(t)
        deadline = time.time() + timeout_s if timeout_s else None
        rc = 0
        running = set(range(nprocs))
        while running:
            for r in list(running):
                code = procs[r].poll()
                if code is None:
                    continue
                running.discard(r)
                if code != 0 and rc == 0:
                    rc = code
            if rc != 0 or (deadline and time.time() > deadline):
                if rc == 0:
                    rc = 124
                break
            time.sleep(0.02)
        return rc
    finally:
        # Each rank runs in its own session: end exactly the process groups started here.
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        for p in procs:
            try:
                p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
        for t in pumps:
            t.join(timeout=2)
        shutil.rmtree(kv, ignore_errors=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m rocshmem_b200.launch", description=__doc__.split("\n")[0])
    ap.add_argument("-n", "--nprocs", type=int, required=True, help="number of processes (one per GPU)")
    ap.add_argument("--backend", choices=["auto", "cuda", "host"], default=None, help="sets ROCSHMEM_BACKEND")
    ap.add_argument("--local-pes", type=int, default=1, help="PEs per process (sets ROCSHMEM_LOCAL_PES)")
    ap.add_argument("--timeout", type=float, default=None, help="seconds after which all ranks are terminated")
    ap.add_argument("--no-tag", action="store_true", help="do not prefix output lines with the rank")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="program and its arguments")
    args = ap.parse_args(argv)
    cmd = args.command[1:] if args.command[:1] == ["--"] else args.command
    if not cmd:
        ap.error("no command given")
    return launch(cmd, args.nprocs, args.backend, args.local_pes, args.timeout, not args.no_tag)


if __name__ == "__main__":
    sys.exit(main())
