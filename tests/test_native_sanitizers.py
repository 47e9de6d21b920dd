"""Builds the native unit-test program of the host-side runtime (allocator, teams, configuration, bootstrap)
with sanitizers and runs it: AddressSanitizer + UBSan for memory errors and undefined behaviour, ThreadSanitizer
for data races between the threads that play the ranks of the bootstrap test. A second test instruments the whole
host side of the runtime library and runs multi-threaded programs (host API, reverse-offload ring) against it."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RT = os.path.join(ROOT, "rocshmem_b200", "csrc", "runtime")
SRCS = [os.path.join(ROOT, "tests", "cpp", "runtime_unit.cpp")] + [
    os.path.join(RT, f) for f in ("allocator.cpp", "team.cpp", "config.cpp", "bootstrap.cpp")]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
@pytest.mark.parametrize("flags", [["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"],
                                   ["-fsanitize=thread"]], ids=["asan-ubsan", "tsan"])
def test_runtime_unit_program_under_sanitizers(flags, tmp_path):
    exe = str(tmp_path / "runtime_unit")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, f"-I{RT}",
                            f"-I{os.path.join(ROOT, 'rocshmem_b200', 'csrc', 'include')}", *SRCS, "-o", exe, "-lpthread"],
                           capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime libraries are not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    scratch = tmp_path / "kv"
    scratch.mkdir()
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([exe, str(scratch)], capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "all passed" in run.stdout


SAN_MODES = {
    "tsan": (["-fsanitize=thread", "-Wno-tsan"], ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1 exitcode=66"},
             "ThreadSanitizer"),
    "asan-ubsan": (["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"],
                   ["-fsanitize=address", "-fsanitize=undefined"],
                   {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0"}, "Sanitizer"),
}


@pytest.mark.skipif(shutil.which("g++") is None or shutil.which("nvcc") is None, reason="needs g++ and nvcc")
@pytest.mark.parametrize("mode", sorted(SAN_MODES))
def test_whole_runtime_with_threads_and_proxy_under_sanitizers(mode, tmp_path):
    """The host side of the runtime library (all .cpp files, instrumented) linked with the device objects of the
    regular build, then three programs on the CPU backend: the typed host API (three processes), several host
    threads per process on it (two processes), and several producer threads on the reverse-offload ring with command
    merging on. A data race between user threads, the runtime and the proxy's consumer thread (ThreadSanitizer), or
    a memory error, a leak or undefined behaviour anywhere in the host runtime (AddressSanitizer + UBSan) fails it."""
    cflags, ldflags, san_env, marker = SAN_MODES[mode]
    from rocshmem_b200 import _build
    if not _build.is_built():
        _build.build(with_tests=False)
    objdir = os.path.join(ROOT, "rocshmem_b200", "build")
    cu_objs = sorted(os.path.join(objdir, f) for f in os.listdir(objdir)
                     if f.endswith(".cu.o") and (f.startswith("kernels_") or f == "runtime_host_ops_cuda.cu.o"))
    assert cu_objs, "device objects of the regular build are missing"
    inc = [f"-I{os.path.join(ROOT, 'rocshmem_b200', 'csrc', 'include')}", f"-I{os.path.join(ROOT, 'rocshmem_b200', 'csrc')}"]
    cuda_home = os.path.dirname(os.path.dirname(os.path.realpath(shutil.which("nvcc"))))
    inc.append(f"-I{os.path.join(cuda_home, 'include')}")
    objs = []
    for name in ("config", "allocator", "team", "bootstrap", "host_shm_provider", "runtime", "host_ops_cpu", "host_api",
                 "proxy", "cuda_vmm_provider"):
        obj = str(tmp_path / f"{name}.o")
        cc = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fPIC", *cflags, *inc, "-c",
                             os.path.join(RT, name + ".cpp"), "-o", obj], capture_output=True, text=True, timeout=600)
        if cc.returncode != 0 and "sanitize" in cc.stderr and "cannot find" in cc.stderr:
            pytest.skip("sanitizer runtime libraries are not installed")
        assert cc.returncode == 0, cc.stderr[-3000:]
        objs.append(obj)
    lib = str(tmp_path / "librocshmem_b200_san.so")
    xflags = [x for f in ldflags for x in ("-Xcompiler", f)]      # one flag per -Xcompiler: nvcc splits at commas
    link = subprocess.run(["nvcc", "-shared", "-o", lib, *objs, *cu_objs, *xflags, "-lpthread", "-ldl", "-lrt"],
                          capture_output=True, text=True, timeout=600)
    if link.returncode != 0 and "san" in link.stderr and "cannot find" in link.stderr:
        pytest.skip("sanitizer runtime libraries are not installed")
    assert link.returncode == 0, link.stderr[-3000:]
    exes = {}
    for prog in ("host_api_sos", "host_threads_sos", "proxy_threads"):
        exe = str(tmp_path / prog)
        cc = subprocess.run(["g++", "-std=c++17", "-O1", "-g", *cflags, *inc,
                             os.path.join(ROOT, "tests", "cpp", prog + ".cpp"), "-o", exe, f"-L{tmp_path}",
                             "-lrocshmem_b200_san", f"-Wl,-rpath,{tmp_path}", "-lpthread"],
                            capture_output=True, text=True, timeout=600)
        assert cc.returncode == 0, cc.stderr[-3000:]
        exes[prog] = exe
    base = dict(os.environ, ROCSHMEM_BACKEND="host", ROCSHMEM_HEAP_SIZE="16M", ROCSHMEM_WAIT_TIMEOUT_MS="60000", **san_env)
    # the ring, one process with two PEs
    run = subprocess.run([exes["proxy_threads"]], env=dict(base, RANK="0", WORLD_SIZE="1", ROCSHMEM_LOCAL_PES="2"),
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and "PASS" in run.stdout, run.stdout[-2000:] + run.stderr[-4000:]
    assert marker not in run.stderr, run.stderr[-4000:]
    # the host API from one thread (three processes) and from several threads (two processes)
    # (the first with the stand-in for the NVLink multicast object: set-up and release of the world's and of split
    # teams' objects run under the sanitizers too)
    for prog, world, extra in (("host_api_sos", 3, {"ROCSHMEM_HOST_FAKE_MULTICAST": "1"}), ("host_threads_sos", 2, {})):
        kv = tmp_path / ("kv_" + prog)
        kv.mkdir()
        procs = [subprocess.Popen([exes[prog]], env=dict(base, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                                                         ROCSHMEM_BOOTSTRAP_DIR=str(kv), **extra),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(world)]
        try:
            for r, p in enumerate(procs):
                out, err = p.communicate(timeout=600)
                assert p.returncode == 0 and f"[pe {r}] PASS" in out, (prog, out[-2000:] + err[-4000:])
                assert marker not in err, err[-4000:]
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
