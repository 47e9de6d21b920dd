"""In-tree build of the native code for sm_100a.

Three artefacts, all inside the package directory so that they travel with a source snapshot:

* ``lib/librocshmem_b200.so`` - host runtime (C++) plus every CUDA kernel of the library;
* ``_C.<abi>.so``             - pybind11 bindings, linked against the library;
* ``_testk.<abi>.so``         - kernels of the functional test-suite that exercise the device API
                                from user code, linked against the same library (built on demand).

The build is described by a generated ``build.ninja`` with paths relative to the package, so an
unchanged tree is not rebuilt after it has been copied elsewhere. ``nvcc`` cross-compiles without a
GPU. Run ``python -m rocshmem_b200._build`` or call :func:`build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIBDIR = PKG / "lib"
EXT = sysconfig.get_config_var("EXT_SUFFIX") or ".so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

RUNTIME_CPP = [
    "runtime/config.cpp", "runtime/allocator.cpp", "runtime/team.cpp", "runtime/bootstrap.cpp",
    "runtime/host_shm_provider.cpp", "runtime/cuda_vmm_provider.cpp", "runtime/runtime.cpp",
    "runtime/host_ops_cpu.cpp", "runtime/host_api.cpp", "runtime/proxy.cpp",
]
LIB_CU = [
    "runtime/host_ops_cuda.cu", "kernels/coll_kernels.cu", "kernels/ep_kernels.cu",
    "kernels/gemm_kernels.cu", "kernels/fused_kernels.cu", "kernels/no_alloc.cu", "kernels/moe_kernels.cu", "kernels/gemm_fp8.cu",
]
BIND_CPP = ["bindings.cpp", "kernels/bindings_ep.cpp", "kernels/bindings_gemm.cpp"]


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return cand
    nvcc = shutil.which("nvcc")
    if nvcc:
        return str(Path(nvcc).resolve().parent.parent)
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def _pybind_include() -> str:
    import pybind11
    return pybind11.get_include()


def _rel(p: Path) -> str:
    return os.path.relpath(p, PKG)


def _ninja_text(with_tests: bool) -> str:
    cuda = _cuda_home()
    py_inc = sysconfig.get_paths()["include"]
    incs = f"-I{_rel(CSRC / 'include')} -I{_rel(CSRC)} -I{cuda}/include"
    cxxflags = f"-O2 -g1 -std=c++17 -fPIC -Wall -Wno-unused-function {incs}"
    nvflags = (f"-O3 -std=c++17 {' '.join(ARCH_FLAGS)} -lineinfo --expt-relaxed-constexpr "
               f"-Xcompiler -fPIC -Xcompiler -Wno-unused-function -diag-suppress 177,550 {incs}")
    pyflags = f"-I{py_inc} -I{_pybind_include()} -fvisibility=hidden"
    lines = [
        "ninja_required_version = 1.5",
        f"nvcc = {cuda}/bin/nvcc",
        "cxx = g++",
        f"cxxflags = {cxxflags}",
        f"nvflags = {nvflags}",
        f"pyflags = {pyflags}",
        "rule cxx",
        "  command = $cxx $cxxflags $extra -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule nvcc",
        "  command = $nvcc $nvflags $extra -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule linklib",
        "  command = $nvcc -shared -o $out $in -lpthread -ldl -lrt",
        "rule linkext",
        f"  command = $nvcc -shared -o $out $in -L{_rel(LIBDIR)} -lrocshmem_b200 "
        "-Xlinker -rpath -Xlinker '$$ORIGIN/lib' -lpthread -ldl -lrt",
    ]
    lib_objs = []
    for src in RUNTIME_CPP:
        if not (CSRC / src).exists():
            continue
        obj = _rel(OBJ / (src.replace("/", "_") + ".o"))
        lines.append(f"build {obj}: cxx {_rel(CSRC / src)}")
        lib_objs.append(obj)
    for src in LIB_CU:
        if not (CSRC / src).exists():
            continue
        obj = _rel(OBJ / (src.replace("/", "_") + ".o"))
        lines.append(f"build {obj}: nvcc {_rel(CSRC / src)}")
        lib_objs.append(obj)
    lib = _rel(LIBDIR / "librocshmem_b200.so")
    lines.append(f"build {lib}: linklib {' '.join(lib_objs)}")
    bind_objs = []
    for src in BIND_CPP:
        if not (CSRC / src).exists():
            continue
        obj = _rel(OBJ / (src.replace("/", "_") + ".o"))
        lines.append(f"build {obj}: cxx {_rel(CSRC / src)}")
        lines.append("  extra = $pyflags")
        bind_objs.append(obj)
    ext = _rel(PKG / f"_C{EXT}")
    lines.append(f"build {ext}: linkext {' '.join(bind_objs)} | {lib}")
    targets = [ext]
    tests_src = PKG.parent / "tests" / "csrc" / "test_kernels.cu"
    if with_tests and tests_src.exists():
        obj = _rel(OBJ / "tests_test_kernels.cu.o")
        lines.append(f"build {obj}: nvcc {_rel(tests_src)}")
        # The test kernels count their API calls (device statistics are compiled in per translation unit).
        lines.append("  extra = -DROCSHMEM_PROFILE -Xcompiler -fvisibility=hidden "
                     f"-I{py_inc} -I{_pybind_include()}")
        text = _rel(PKG / f"_testk{EXT}")
        lines.append(f"build {text}: linkext {obj} | {lib}")
        targets.append(text)
    lines.append(f"default {' '.join(targets)}")
    return "\n".join(lines) + "\n"


def build(with_tests: bool = True, verbose: bool = False, jobs: int | None = None) -> None:
    """Compile everything that is out of date. Raises ``RuntimeError`` with the compiler output."""
    OBJ.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    ninja_file = PKG / "build.ninja"
    text = _ninja_text(with_tests)
    if not ninja_file.exists() or ninja_file.read_text() != text:
        ninja_file.write_text(text)
    cmd = [sys.executable, "-m", "ninja", "-C", str(PKG)]
    if jobs:
        cmd += ["-j", str(jobs)]
    if verbose:
        cmd.append("-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        # Compiler diagnostics quote whole macro expansions; keep the message readable.
        lines = [ln[:400] for ln in (proc.stdout + proc.stderr).splitlines()]
        keep = [ln for ln in lines if "error" in ln.lower() or "FAILED" in ln][:60]
        raise RuntimeError("native build failed:\n" + "\n".join(keep or lines[-60:]))
    if verbose:
        print(proc.stdout)


def is_built(with_tests: bool = False) -> bool:
    ok = (LIBDIR / "librocshmem_b200.so").exists() and (PKG / f"_C{EXT}").exists()
    if with_tests:
        ok = ok and (PKG / f"_testk{EXT}").exists()
    return ok


if __name__ == "__main__":
    build(with_tests=True, verbose="-v" in sys.argv)
    print("built:", PKG / f"_C{EXT}")
