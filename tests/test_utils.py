"""Utility modules on the CPU backend: heap snapshots, roofline arithmetic, tracing switches."""
import json
import os

import pytest
import torch


@pytest.fixture()
def shm_cpu(tmp_path):
    import rocshmem_b200 as shm
    if shm.is_initialized():
        shm.finalize()
    shm.init(backend="host", n_local=2, heap_size="8M", ROCSHMEM_BOOTSTRAP_DIR=str(tmp_path))
    yield shm
    shm.finalize()


def test_snapshot_and_restore_round_trip(shm_cpu, tmp_path):
    from rocshmem_b200.utils import checkpoint
    shm = shm_cpu
    a = shm.zeros(1000, torch.float32)
    b = shm.zeros((16, 8), torch.int64)
    a.copy_(torch.arange(1000, dtype=torch.float32))
    b.fill_(7)
    saved = checkpoint.snapshot({"a": a, "b": b})
    a.zero_()
    b.zero_()
    checkpoint.restore({"a": a, "b": b}, saved)
    assert torch.equal(a.cpu(), torch.arange(1000, dtype=torch.float32)) and torch.all(b.cpu() == 7)
    path = str(tmp_path / "pe0.pt")
    checkpoint.save(path, {"a": a})
    a.fill_(-1)
    checkpoint.load(path, {"a": a})
    assert float(a[999]) == 999.0
    with pytest.raises(ValueError):
        checkpoint.restore({"a": b}, {"a": saved["a"]})
    with pytest.raises(KeyError):
        checkpoint.restore({"c": a}, saved)


def test_roofline_uses_measured_peaks_or_fallback(tmp_path):
    from rocshmem_b200.utils import roofline
    p = roofline.measured_peaks(str(tmp_path))
    assert p["source"] == "fallback" and p["hbm_gbs"] == 6650.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6000, "bf16_tflops": 1500, "bf16_tflops_sustained": 1300}))
    p = roofline.measured_peaks(str(tmp_path))
    assert p["source"] == "measured"
    assert roofline.memory_fraction(6e9, 1e-3, p) == pytest.approx(1.0)
    assert roofline.compute_fraction(1.5e12, 1e-3, peaks=p) == pytest.approx(1.0)
    # compute-bound and link-bound cases
    assert roofline.fused_roofline_seconds(1.3e12, 1e6, peaks=p) == pytest.approx(1e-3)
    assert roofline.fused_roofline_seconds(1e9, 770e6, peaks=p) == pytest.approx(1e-3)


def test_trace_range_is_a_no_op_without_nvtx(monkeypatch):
    from rocshmem_b200.utils import trace
    monkeypatch.delenv("ROCSHMEM_NVTX", raising=False)
    assert not trace.nvtx_enabled()
    calls = []

    @trace.traced("unit")
    def f(x):
        calls.append(x)
        return x + 1

    assert f(1) == 2 and calls == [1]
    monkeypatch.setenv("ROCSHMEM_NVTX", "1")
    assert trace.nvtx_enabled()
    with trace.trace_range("still fine without a GPU"):
        pass


def test_guard_regions_detect_an_overrun(shm_cpu):
    """Every internal sub-region (flags, descriptors, ...) is followed by a guard pattern; a write past the end
    of a region is reported by check_canaries() and at finalize."""
    from rocshmem_b200 import runtime as rt
    shm = shm_cpu
    C = rt._C()
    assert C.check_canaries() == 0
    guards = C.internal_guard_offsets()
    assert len(guards) >= 10 and all(g % 256 == 0 for g in guards)
    a = shm.zeros(1024, torch.int32)       # ordinary use leaves the guards alone
    shm.barrier_all()
    assert C.check_canaries() == 0
    internal = C.heap_base(1) + shm.heap_info()["size"]          # PE 1's internal area
    word = rt.tensor_from_address(internal + guards[3] + 8, (1,), torch.int64)
    saved = int(word[0])
    word[0] = 12345
    assert C.check_canaries() == 1
    word[0] = saved
    assert C.check_canaries() == 0
    shm.free(a)


def test_functional_driver_accepts_the_reference_test_numbers():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "functional_driver.py")
    spec = importlib.util.spec_from_file_location("functional_driver", path)
    fd = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fd)
    assert len(fd.REFERENCE_NAMES) == 59 and fd.REFERENCE_NAMES[58] == "WAVESignalFetch"
    assert fd.resolve_test("put") == "put" and fd.resolve_test("2") == "put_thread" and fd.resolve_test("34") == "allreduce"
    assert fd.resolve_test("13") == "pingpong" and fd.resolve_test("0") == "get_thread" and fd.resolve_test("31") == "put_wave"
    # names of the per-scope forms: operation, scope and "context created in the kernel"
    assert fd.rma_form("put_nbi_wave") == (1, 1, 0) and fd.rma_form("ctx_get_thread") == (2, 0, 1)
    assert fd.rma_form("g") == (5, 0, 0) and fd.rma_form("put") is None and fd.rma_form("allreduce") is None
    assert all(name in fd.AMO or name in fd.SIGNAL_SCOPES or fd.rma_form(name) is not None or
               name in ("pingpong", "pingall", "barrier", "allreduce", "broadcast", "fcollect", "alltoall", "shmem_ptr",
                        "ctx_infra")
               for name in fd.REFERENCE_NUMBERS.values())
    assert len(fd.REFERENCE_NUMBERS) >= 50
    with pytest.raises(SystemExit, match="RandomAccessTestType"):
        fd.resolve_test("14")
    with pytest.raises(SystemExit, match="0 to 58"):
        fd.resolve_test("59")


def test_info_command_reports_configuration_and_runtime(capsys, monkeypatch):
    import json

    import rocshmem_b200 as shm
    from rocshmem_b200 import info
    if shm.is_initialized():
        shm.finalize()
    monkeypatch.setenv("ROCSHMEM_HEAP_SIZE", "8M")
    monkeypatch.setenv("ROCSHMEM_BACKEND", "host")
    assert info.main(["--init", "--json"]) == 0
    data = json.loads(capsys.readouterr().out)
    assert data["built"] and data["config"]["heap_size"] == 8 << 20
    assert data["runtime"]["n_pes"] == 1 and data["runtime"]["backend"] == "host-shm" and data["runtime"]["size"] == 8 << 20
    assert not shm.is_initialized()
    monkeypatch.setenv("ROCSHMEM_MAX_NUM_TEAMS", "0")
    assert info.main([]) == 0
    assert "ROCSHMEM_MAX_NUM_TEAMS" in capsys.readouterr().out


def test_matrix_runner_lists_its_cases_and_parses_driver_tables(capsys):
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "run_matrix.py")
    spec = importlib.util.spec_from_file_location("run_matrix", path)
    rm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rm)
    assert rm.main(["--dry-run", "--only", "put,allreduce"]) == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l]
    assert len(lines) == 7 and all("functional_driver.py -a " in l and "--local-pes 2" in l for l in lines)
    assert rm.main(["--dry-run", "--gpus", "4"]) == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l]
    assert len(lines) == len(rm.MATRIX) and all("launch -n 4" in l and "--local-pes" not in l for l in lines)
    table = "\n".join(["# test put, 2 PEs", "    Size (B)     # msgs   Latency (us)   Bandwidth (GB/s)   Msg rate (msg/s)",
                       "[0]            8         10          0.310              0.026            3225806",
                       "        1048576         10          2.005            523.000             498753", "noise 1 2 3 4"])
    rows = list(rm.parse_rows(table))
    assert rows == [(8, 10, 0.31, 0.026, 3225806.0), (1048576, 10, 2.005, 523.0, 498753.0)]


def test_debug_level_two_traces_management_calls():
    import os
    import subprocess
    import sys
    code = ("import rocshmem_b200 as shm, torch\n"
            "shm.init(n_local=2, heap_size='4M', backend='host')\n"
            "x = shm.zeros(100, torch.float32)\n"
            "t = shm.team_world().split_strided(0, 1, 1)\n"
            "t.destroy(); shm.free(x); shm.finalize()\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for level, expect in (("2", True), ("0", False)):
        out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, ROCSHMEM_DEBUG=level, PYTHONPATH=root),
                             capture_output=True, text=True, timeout=120)
        assert out.returncode == 0, out.stderr[-2000:]
        traced = "malloc(400)" in out.stderr and "team_split_strided(start 0, stride 1, size 1) = 0" in out.stderr
        assert traced == expect, out.stderr[-2000:]


def test_configuration_header_carries_the_package_version():
    import os
    import re
    import rocshmem_b200
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "rocshmem_b200", "csrc", "include", "rocshmem", "rocshmem_config.h")).read()
    parts = [re.search(rf"#define ROCSHMEM_B200_VERSION_{k} (\d+)", text).group(1) for k in ("MAJOR", "MINOR", "PATCH")]
    assert ".".join(parts) == rocshmem_b200.__version__
    assert f'"{rocshmem_b200.__version__}"' in text


def test_ring_dump_without_a_proxy_says_so(fresh_runtime, capfd):
    shm = fresh_runtime
    shm.init(n_local=1, heap_size="1M", backend="host")
    try:
        shm.debug_print_ring(0, 2)
    finally:
        shm.finalize()
    assert "no reverse-offload ring in this process" in capfd.readouterr().err
