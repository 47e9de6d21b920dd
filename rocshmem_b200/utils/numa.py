"""Keep a process and its pinned host buffers on the NUMA node of its GPU.

On a two-socket host every GPU hangs off one socket. Pinned memory that lives on the other socket reaches the
GPU through the inter-socket link, and when eight ranks all allocate from the node their launcher happened to
start on, their host-to-device copies share that link. :func:`bind_to_device_node` reads the GPU's node from
sysfs, restricts the calling process to that node's CPUs and asks the kernel to prefer that node for new pages;
call it before allocating pinned memory. Everything is best effort: on a host without NUMA information (a single
node, a container that hides sysfs) it changes nothing and reports why.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

MPOL_PREFERRED = 1
MPOL_INTERLEAVE = 3
_SYS_set_mempolicy = 238  # x86_64


def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def device_numa_node(device_index: int, sysfs: str = "/sys") -> Optional[int]:
    """NUMA node of a CUDA device, or None when the host does not tell."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(os.path.join(sysfs, "bus/pci/devices", bdf, "numa_node")) as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, ValueError, AttributeError, RuntimeError, AssertionError):
        return None


def node_cpus(node: int, sysfs: str = "/sys") -> set:
    """CPUs of a NUMA node (empty when unknown)."""
    try:
        with open(os.path.join(sysfs, f"devices/system/node/node{node}/cpulist")) as f:
            return _parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()


def online_nodes(sysfs: str = "/sys") -> list:
    """NUMA nodes of the host (empty when unknown)."""
    try:
        with open(os.path.join(sysfs, "devices/system/node/online")) as f:
            return sorted(_parse_cpulist(f.read()))
    except (OSError, ValueError):
        return []


def _set_mempolicy(mode: int, nodes) -> bool:
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        nbits = max(64, max(nodes) + 1)
        mask = (ctypes.c_ulong * ((nbits + 63) // 64))()
        for n in nodes:
            mask[n // 64] |= 1 << (n % 64)
        return libc.syscall(_SYS_set_mempolicy, mode, mask, nbits + 1) == 0
    except (OSError, AttributeError, ValueError):
        return False


def bind_to_device_node(device_index: int, sysfs: str = "/sys") -> dict:
    """Restrict this process to the CPUs of the GPU's NUMA node and prefer that node for new pages.

    Returns ``{"node": n or None, "cpus": count, "mempolicy": bool, "note": str}``."""
    out = {"node": None, "cpus": 0, "mempolicy": False, "note": ""}
    node = device_numa_node(device_index, sysfs)
    if node is None:
        # The host does not say where the GPU sits (common in containers). Spreading new pages over all nodes at
        # least keeps eight ranks from filling, and copying out of, one socket's memory.
        nodes = online_nodes(sysfs)
        out["note"] = "no NUMA node reported for the device"
        if len(nodes) > 1:
            out["mempolicy"] = _set_mempolicy(MPOL_INTERLEAVE, nodes)
            out["note"] += f"; pages interleaved over nodes {nodes}" if out["mempolicy"] else ""
        return out
    out["node"] = node
    cpus = node_cpus(node, sysfs)
    try:
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if use:
            os.sched_setaffinity(0, use)
            out["cpus"] = len(use)
        else:
            out["note"] = "none of the node's CPUs is available to this process"
    except (OSError, AttributeError) as e:
        out["note"] = f"affinity not changed: {e}"
    out["mempolicy"] = _set_mempolicy(MPOL_PREFERRED, [node])
    return out
