"""Builds the native unit-test program of the host-side runtime (allocator, teams, configuration, bootstrap)
with sanitizers and runs it: AddressSanitizer + UBSan for memory errors and undefined behaviour, ThreadSanitizer
for data races between the threads that play the ranks of the bootstrap test."""
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
