"""The CMake package as a C++ user sees it: build and install the library with CMake, then configure a separate
project with ``find_package(rocshmem_b200)``, link ``roc::rocshmem`` (the reference's target name) and run the
resulting program on the CPU backend."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CONSUMER = """cmake_minimum_required(VERSION 3.24)
project(consumer LANGUAGES CXX CUDA)
set(CMAKE_CUDA_ARCHITECTURES "100a")
set(CMAKE_CUDA_STANDARD 17)
find_package(rocshmem_b200 REQUIRED)
find_package(CUDAToolkit REQUIRED)
add_executable(sos {src})
target_link_libraries(sos PRIVATE roc::rocshmem)
# a program that uses the device API from its own kernels (compiled and linked here, run by the GPU tests)
add_executable(allreduce {cu})
target_link_libraries(allreduce PRIVATE roc::rocshmem CUDA::cudart CUDA::cuda_driver)
"""


def _run(cmd, **kw):
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, **kw)
    assert out.returncode == 0, " ".join(cmd) + "\n" + out.stdout[-2000:] + out.stderr[-3000:]


@pytest.mark.skipif(shutil.which("cmake") is None or shutil.which("nvcc") is None, reason="needs cmake and nvcc")
def test_installed_package_is_usable_from_another_cmake_project(tmp_path):
    build, prefix = tmp_path / "build", tmp_path / "prefix"
    _run(["cmake", "-S", ROOT, "-B", str(build), "-DCMAKE_BUILD_TYPE=Release", "-DROCSHMEM_BUILD_EXAMPLES=OFF"])
    _run(["cmake", "--build", str(build), "-j", str(min(16, os.cpu_count() or 4))])
    _run(["cmake", "--install", str(build), "--prefix", str(prefix)])
    assert (prefix / "include" / "rocshmem" / "rocshmem.h").exists()
    consumer = tmp_path / "consumer"
    consumer.mkdir()
    (consumer / "CMakeLists.txt").write_text(CONSUMER.format(src=os.path.join(ROOT, "tests", "cpp", "host_api_sos.cpp"),
                                                              cu=os.path.join(ROOT, "examples", "allreduce.cu")))
    cbuild = tmp_path / "cbuild"
    _run(["cmake", "-S", str(consumer), "-B", str(cbuild), f"-DCMAKE_PREFIX_PATH={prefix}"])
    _run(["cmake", "--build", str(cbuild), "-j", "4"])
    assert (cbuild / "allreduce").exists()
    kv = tmp_path / "kv"
    kv.mkdir()
    procs = [subprocess.Popen([str(cbuild / "sos")],
                              env=dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), ROCSHMEM_BACKEND="host",
                                       ROCSHMEM_HEAP_SIZE="16M", ROCSHMEM_BOOTSTRAP_DIR=str(kv)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    try:
        for r, p in enumerate(procs):
            out, _ = p.communicate(timeout=180)
            assert p.returncode == 0 and f"[pe {r}] PASS" in out, out[-2000:]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
