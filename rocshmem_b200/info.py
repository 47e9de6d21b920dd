"""Prints what this installation is and how it is configured: ``python -m rocshmem_b200.info``.

Package version and build state, the CUDA devices visible to the process, the configuration that ``init`` would
use (environment variables applied and validated), and - with ``--init`` - a single-PE start-up that reports the
backend chosen, the heap and whether the NVLink multicast mapping could be set up.
"""
from __future__ import annotations

import argparse
import json
import sys


def collect(do_init: bool = False) -> dict:
    import torch

    import rocshmem_b200 as shm
    from rocshmem_b200 import _build, runtime as rt
    info = {"version": shm.__version__, "built": _build.is_built(), "test_kernels_built": _build.is_built(with_tests=True),
            "torch": torch.__version__, "cuda_available": torch.cuda.is_available(), "devices": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                    "memory_gib": round(p.total_memory / 2 ** 30, 1)})
    try:
        info["config"] = rt._C().config_from_env({})
    except Exception as e:  # noqa: BLE001 - a bad environment variable is part of the report
        info["config_error"] = str(e)
    if do_init:
        was = shm.is_initialized()
        if not was:
            shm.init()
        info["runtime"] = dict(shm.heap_info(), n_pes=shm.n_pes(), my_pe=shm.my_pe(), team_slots=shm.runtime.team_capacity())
        if not was:
            shm.finalize()
    return info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m rocshmem_b200.info", description=__doc__.split("\n")[0])
    ap.add_argument("--init", action="store_true", help="also start a single-PE runtime and report on it")
    ap.add_argument("--json", action="store_true", help="machine-readable output")
    args = ap.parse_args(argv)
    info = collect(args.init)
    if args.json:
        print(json.dumps(info, indent=2, default=str))
        return 0
    print(f"rocshmem_b200 {info['version']}  (native parts built: {info['built']}, test kernels: {info['test_kernels_built']})")
    print(f"torch {info['torch']}, CUDA available: {info['cuda_available']}")
    for d in info["devices"]:
        print(f"  device {d['index']}: {d['name']}, sm_{d['sm'].replace('.', '')}, {d['sms']} SMs, {d['memory_gib']} GiB")
    if "config_error" in info:
        print("configuration error:", info["config_error"])
    else:
        print("configuration (environment applied):")
        for k, v in info["config"].items():
            print(f"  {k:20s} {v}")
    if "runtime" in info:
        print("runtime (single PE):")
        for k, v in info["runtime"].items():
            print(f"  {k:20s} {v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
