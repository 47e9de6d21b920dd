"""The typed API name tables generated from type lists against what the public header really declares."""
import os
import re
import shutil
import subprocess

import pytest

from rocshmem_b200.utils import gen_api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "rocshmem_b200", "csrc", "include")


def test_family_sizes():
    # 23 RMA types x 4 ops x 5 scopes x 2 (ctx) + mem forms + p/g
    assert len(gen_api.rma_names()) == 23 * 4 * 5 * 2 + 4 * 5 * 2 + 23 * 2 * 2
    assert len(gen_api.amo_names()) == (14 * 3 + 12 * 5 + 7 * 6) * 2
    assert len(gen_api.sync_names()) == 19 * 8
    assert len(gen_api.collective_names()) == 13 * 3 + 4 * 7 + 4 * 4
    names = gen_api.all_names()
    assert len(names) == len(set(names))


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc to pre-process the header")
def test_every_generated_name_is_declared(tmp_path):
    src = tmp_path / "surface.cu"
    src.write_text("#include <rocshmem/rocshmem.h>\n")
    out = subprocess.run(["nvcc", "-E", "-std=c++17", "-I", INC, "-gencode", "arch=compute_100a,code=sm_100a", str(src)],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    declared = set(re.findall(r"\brocshmemx?_[a-z0-9_]+\b", out.stdout))
    missing = [n for n in gen_api.all_names() + gen_api.extension_names() if n not in declared]
    assert not missing, f"{len(missing)} names are not declared, e.g. {missing[:10]}"


def test_markdown_lists_every_family(tmp_path):
    path = tmp_path / "API.md"
    assert gen_api.main(["--markdown", str(path)]) == 0
    text = path.read_text()
    for fam in gen_api.families():
        assert fam in text
    assert "rocshmem_ctx_float_sum_wg_reduce" in text and "rocshmem_uint64_atomic_fetch_xor" in text


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc")
def test_name_coverage_translation_unit_compiles(tmp_path):
    """Every generated name resolves to a function when compiled for sm_100a."""
    src = tmp_path / "names.cu"
    assert gen_api.main(["--surface-cu", str(src)]) == 0
    out = subprocess.run(["nvcc", "-std=c++17", "-I", INC, "-gencode", "arch=compute_100a,code=sm_100a", "-c", str(src),
                          "-o", str(tmp_path / "names.o")], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:]


def test_every_public_python_name_has_a_docstring():
    """The Python listing (rocshmem_b200.utils.gen_pydoc) has a description for every public function, class and
    method of the package's modules."""
    from rocshmem_b200.utils import gen_pydoc
    text = gen_pydoc.markdown()
    missing = [line for line in text.splitlines() if line.rstrip().endswith("—")]
    assert not missing, missing
    assert "## `rocshmem_b200.ops.moe`" in text and "EpDispatcher" in text
