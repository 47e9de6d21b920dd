"""Generator of the typed OpenSHMEM API name tables.

The public header builds its typed functions with X-macros; this module builds the same set of names
independently, from type lists and name patterns, the way the reference's generator emits its expanded
headers (utils/header_files_gen/RMA.py:27-41, AMO.py:27-48, COLL.py:164-209, SIG_OP.py, P2P_SYNC.py).
It is used to

* write the API listing (``python -m rocshmem_b200.utils.gen_api --markdown docs/API.md``),
* emit a translation unit that takes the address of nothing but *names* every function inside an
  unevaluated context (``--surface-cu``), so a compiler run proves the header declares all of them,
* and cross-check the header in the CPU test-suite (every generated name must appear in the
  pre-processed header).
"""
from __future__ import annotations

import argparse
import sys
from typing import Dict, List

STANDARD_RMA = ["float", "double", "char", "schar", "short", "int", "long", "longlong", "uchar", "ushort", "uint",
                "ulong", "ulonglong"]
FIXED_RMA = ["int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64", "size", "ptrdiff"]
AMO_STANDARD = ["int", "long", "longlong", "uint", "ulong", "ulonglong", "int32", "int64", "uint32", "uint64", "size",
                "ptrdiff"]
AMO_EXTENDED_ONLY = ["float", "double"]
AMO_BITWISE = ["uint", "ulong", "ulonglong", "int32", "int64", "uint32", "uint64"]
SYNC = STANDARD_RMA + ["int32", "int64", "uint32", "uint64", "size", "ptrdiff"]
REDUCE_INT = ["short", "int", "long", "longlong"]
REDUCE_FLOAT = ["float", "double"]
REDUCE_EXTRA = ["half", "bfloat16"]         # additions of this library (sum / min / max / prod)
INT_OPS = ["sum", "min", "max", "prod", "or", "and", "xor"]
FLOAT_OPS = ["sum", "min", "max", "prod"]
SCOPES = ["", "_wave", "_wg", "_warp", "_block"]   # wave / wg are the reference's names, warp / block aliases


def _both(name: str) -> List[str]:
    """A function and its explicit-context form."""
    return [f"rocshmem_{name}", f"rocshmem_ctx_{name}"]


def rma_names() -> List[str]:
    out: List[str] = []
    for op in ("put", "get", "put_nbi", "get_nbi"):
        for scope in SCOPES:
            for t in STANDARD_RMA + FIXED_RMA:
                out += _both(f"{t}_{op}{scope}")
            out += _both(f"{op.replace('put', 'putmem').replace('get', 'getmem')}{scope}")
    for t in STANDARD_RMA + FIXED_RMA:
        out += _both(f"{t}_p") + _both(f"{t}_g")
    return out


def signal_names() -> List[str]:
    out: List[str] = []
    for nbi in ("", "_nbi"):
        for scope in SCOPES:
            out += _both(f"putmem_signal{nbi}{scope}")
            for t in STANDARD_RMA:
                out += _both(f"{t}_put_signal{nbi}{scope}")
    out += [f"rocshmem_signal_fetch{s}" for s in SCOPES]
    return out


def amo_names() -> List[str]:
    out: List[str] = []
    for t in AMO_STANDARD + AMO_EXTENDED_ONLY:
        for op in ("fetch", "set", "swap"):
            out += _both(f"{t}_atomic_{op}")
    for t in AMO_STANDARD:
        for op in ("compare_swap", "fetch_inc", "inc", "fetch_add", "add"):
            out += _both(f"{t}_atomic_{op}")
    for t in AMO_BITWISE:
        for op in ("fetch_and", "and", "fetch_or", "or", "fetch_xor", "xor"):
            out += _both(f"{t}_atomic_{op}")
    return out


def sync_names() -> List[str]:
    out: List[str] = []
    for t in SYNC:
        for op in ("wait_until", "wait_until_all", "wait_until_any", "wait_until_some", "wait_until_all_vector",
                   "wait_until_any_vector", "wait_until_some_vector", "test"):
            out.append(f"rocshmem_{t}_{op}")
    return out


def collective_names() -> List[str]:
    out: List[str] = []
    for t in STANDARD_RMA:
        for op in ("broadcast", "fcollect", "alltoall"):
            out.append(f"rocshmem_ctx_{t}_wg_{op}")
    for t in REDUCE_INT:
        out += [f"rocshmem_ctx_{t}_{op}_wg_reduce" for op in INT_OPS]
    for t in REDUCE_FLOAT + REDUCE_EXTRA:
        out += [f"rocshmem_ctx_{t}_{op}_wg_reduce" for op in FLOAT_OPS]
    return out


def untyped_names() -> List[str]:
    return [
        "rocshmem_init", "rocshmem_init_thread", "rocshmem_query_thread", "rocshmem_finalize", "rocshmem_global_exit",
        "rocshmem_dump_stats", "rocshmem_reset_stats", "rocshmem_my_pe", "rocshmem_n_pes", "rocshmem_malloc",
        "rocshmem_free", "rocshmem_ptr", "rocshmem_ctx_create", "rocshmem_ctx_destroy", "rocshmem_wg_init",
        "rocshmem_wg_init_thread", "rocshmem_wg_finalize", "rocshmem_wg_ctx_create", "rocshmem_wg_team_create_ctx",
        "rocshmem_wg_ctx_destroy", "rocshmem_ctx_my_pe", "rocshmem_ctx_n_pes", "rocshmem_team_split_strided",
        "rocshmem_team_destroy", "rocshmem_team_n_pes", "rocshmem_team_my_pe", "rocshmem_team_translate_pe",
        "rocshmem_fence", "rocshmem_ctx_fence", "rocshmem_quiet", "rocshmem_ctx_quiet",
        "rocshmem_threadfence_system", "rocshmem_ctx_threadfence_system", "rocshmem_barrier_all", "rocshmem_sync_all",
        "rocshmem_wg_barrier_all", "rocshmem_ctx_wg_barrier_all", "rocshmem_wg_sync_all", "rocshmem_ctx_wg_sync_all",
        "rocshmem_wg_team_sync", "rocshmem_ctx_wg_team_sync",
    ]


def extension_names() -> List[str]:
    """``rocshmemx_*``: additions of this library (host side unless noted)."""
    return [
        "rocshmemx_set_local_pe", "rocshmemx_n_local_pes", "rocshmemx_get_error", "rocshmemx_clear_error",
        "rocshmemx_set_wait_timeout_ms", "rocshmemx_heap_write", "rocshmemx_heap_read", "rocshmemx_default_stream",
        "rocshmemx_slab_create", "rocshmemx_slab_destroy", "rocshmemx_slab_reset", "rocshmemx_slab_used",
        "rocshmemx_slab_alloc_host",
        # device side
        "rocshmemx_slab_alloc", "rocshmemx_slab_alloc_wave", "rocshmemx_slab_alloc_wg", "rocshmemx_team_my_pe",
        "rocshmemx_team_n_pes", "rocshmemx_local", "rocshmemx_block_team_sync_status", "rocshmemx_grid_sync",
        "rocshmemx_ticket_lock_block", "rocshmemx_ticket_unlock_block", "rocshmemx_spin_lock", "rocshmemx_spin_unlock",
    ]


def families() -> Dict[str, List[str]]:
    return {"lifecycle, identity, heap, teams, contexts, ordering, barriers": untyped_names(), "RMA": rma_names(),
            "signalling": signal_names(), "atomics": amo_names(), "point-to-point synchronisation": sync_names(),
            "collectives": collective_names()}


def all_names() -> List[str]:
    seen, out = set(), []
    for names in families().values():
        for n in names:
            if n not in seen:
                seen.add(n)
                out.append(n)
    return out


# Host-callable launchers of the library kernels with the limits their validators enforce.
LIBRARY_LAUNCHERS = [
    ("kernels.hpp", ["coll_barrier", "coll_allreduce", "coll_broadcast", "coll_fcollect", "coll_alltoall", "coll_preload",
                     "coll_blocks_for", "nvls_available", "host_amo"],
     "symmetric buffers; allreduce: `ALLREDUCE_LL` up to 2 KiB of 2- or 4-byte elements, `ALLREDUCE_NVLS` sum of fp32 / "
     "fp16 / bf16 on teams with a multicast mapping, 16-byte aligned"),
    ("ep_kernels.hpp", ["ep_dispatch", "ep_combine", "ep_combine_fetches", "ep_expert_layout", "ep_default_blocks",
                        "fp8_quantize_1x128", "fp8_dequantize_1x128"],
     "teams of at most 32 ranks (`EP_MAX_RANKS`; a destination rank is a lane of a warp), hidden a multiple of 512, at "
     "most 1024 experts and divisible by the team size, top-k at most `EP_MAX_TOPK`, low-latency mode needs the "
     "slotted layout"),
    ("gemm_kernels.hpp", ["gemm_bf16", "gemm_bf16_one_cta", "gemm_bf16_pair", "grouped_gemm_bf16",
                          "grouped_gemm_bf16_gathered", "grouped_gemm_bf16_scatter_add", "gemm_fp8_blockscaled",
                          "grouped_gemm_fp8_blockscaled", "grouped_gemm_fp8_swiglu_quant", "grouped_gemm_fp8_scatter_add",
                          "ag_gemm_bf16", "gemm_rs_bf16", "ag_gemm_fp8", "gemm_rs_fp8", "gemm_error_count"],
     "row-major operands, 16-byte aligned; bf16: K a multiple of 8 (64 with gathered rows); e4m3: K a multiple of 512, "
     "N of 128 (256 with SwiGLU); fused kernels: shard rows a multiple of 128"),
    ("moe_kernels.hpp", ["moe_gather_rows", "moe_zero_rows"], "hidden a multiple of 8 (512 for e4m3 rows)"),
    ("no_alloc.h", ["rocshmem_b200_expert_layout_noalloc"], "at most 1024 experts per rank; calls must not overlap on a GPU"),
]


def markdown() -> str:
    lines = ["# API listing", "",
             "Generated by `python -m rocshmem_b200.utils.gen_api --markdown`; every name is declared by",
             "`rocshmem_b200/csrc/include/rocshmem/rocshmem.h` (device and host) or `rocshmem_host.h`.", ""]
    for fam, names in families().items():
        lines += [f"## {fam} ({len(names)} functions)", "", "```"]
        lines += sorted(names)
        lines += ["```", ""]
    ext = extension_names()
    lines += [f"## extensions ({len(ext)} functions, not part of the count above; described in `GUIDE.md`)", "", "```"]
    lines += sorted(ext)
    lines += ["```", ""]
    lines += ["## library kernels (host-callable launchers, `rocshmem::kernels`, not part of the count above)", "",
              "Stream-ordered launchers of `rocshmem_b200/csrc/kernels/*.hpp`; the Python layer (`docs/PYTHON_API.md`) wraps",
              "every one of them. All return 0 or a CUDA error code.", "",
              "| Header | Launchers | Limits |", "|---|---|---|"]
    lines += [f"| `{h}` | {', '.join(f'`{n}`' for n in names)} | {limits} |" for h, names, limits in LIBRARY_LAUNCHERS]
    lines += [""]
    return "\n".join(lines)


def surface_cu() -> str:
    """A translation unit that names every function in an unevaluated operand."""
    body = "\n".join(f"  (void)sizeof(&{n});" if not _overloaded(n) else f"  // {n}: overloaded, covered by name lookup below"
                     for n in all_names())
    return ("#include <rocshmem/rocshmem.h>\n\nusing namespace rocshmem;\n"
            "__global__ void rocshmem_api_names() {\n" + body + "\n}\n")


def _overloaded(name: str) -> bool:
    return name in ("rocshmem_fence", "rocshmem_ctx_fence", "rocshmem_init", "rocshmem_wg_init_thread")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--markdown", metavar="FILE", help="write the API listing")
    ap.add_argument("--surface-cu", metavar="FILE", help="write the name-coverage translation unit")
    ap.add_argument("--count", action="store_true", help="print the number of names per family")
    args = ap.parse_args(argv)
    if args.markdown:
        with open(args.markdown, "w") as f:
            f.write(markdown())
    if args.surface_cu:
        with open(args.surface_cu, "w") as f:
            f.write(surface_cu())
    if args.count or not (args.markdown or args.surface_cu):
        for fam, names in families().items():
            print(f"{len(names):5d}  {fam}")
        print(f"{len(all_names()):5d}  total")
    return 0


if __name__ == "__main__":
    sys.exit(main())
