"""Configuration parsing: ROCSHMEM_* variables, size suffixes, validation."""
import pytest

from rocshmem_b200 import _native

C = _native.load()


@pytest.mark.parametrize("text,value", [("1024", 1024), ("64K", 64 << 10), ("64k", 64 << 10), ("3M", 3 << 20),
                                         ("2G", 2 << 30), ("1T", 1 << 40), ("0x100", 256), (" 16 M ", 16 << 20),
                                         ("8MB", 8 << 20), ("8MiB", 8 << 20)])
def test_parse_size(text, value):
    assert C.parse_size(text) == value


@pytest.mark.parametrize("text", ["", "abc", "-5", "12X", "1.5G", "99999999999999999999", "M"])
def test_parse_size_rejects(text):
    with pytest.raises(Exception):
        C.parse_size(text)


def test_defaults_match_reference(monkeypatch):
    for k in ("ROCSHMEM_HEAP_SIZE", "ROCSHMEM_MAX_NUM_CONTEXTS", "ROCSHMEM_MAX_NUM_TEAMS",
              "ROCSHMEM_MAX_NUM_HOST_CONTEXTS", "ROCSHMEM_WAIT_TIMEOUT_MS"):
        monkeypatch.delenv(k, raising=False)
    c = C.config_from_env({})
    assert c["heap_size"] == 1 << 30 and c["max_contexts"] == 1024 and c["max_teams"] == 40
    assert c["max_host_contexts"] == 40 and c["wait_timeout_ms"] == 10000 and c["backend"] == "auto"


def test_env_and_overrides(monkeypatch):
    monkeypatch.setenv("ROCSHMEM_HEAP_SIZE", "256M")
    monkeypatch.setenv("ROCSHMEM_MAX_NUM_TEAMS", "12")
    c = C.config_from_env({})
    assert c["heap_size"] == 256 << 20 and c["max_teams"] == 12
    c = C.config_from_env({"ROCSHMEM_HEAP_SIZE": "1G", "ROCSHMEM_USE_PROXY": "1"})
    assert c["heap_size"] == 1 << 30 and c["use_proxy"] == 1


@pytest.mark.parametrize("ov", [{"ROCSHMEM_HEAP_SIZE": "64"}, {"ROCSHMEM_MAX_NUM_TEAMS": "0"},
                                {"ROCSHMEM_MAX_NUM_TEAMS": "65"}, {"ROCSHMEM_MAX_NUM_CONTEXTS": "100000"},
                                {"ROCSHMEM_WAIT_TIMEOUT_MS": "0"}, {"RO_NET_QUEUE_SIZE": "100"},
                                {"ROCSHMEM_BACKEND": "rocm"}, {"ROCSHMEM_HEAP_SIZE": "lots"}])
def test_validation(ov):
    with pytest.raises(Exception):
        C.config_from_env(ov)
