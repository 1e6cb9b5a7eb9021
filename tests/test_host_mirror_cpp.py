"""The C++ owner types above the C ABI (include/augur_nvfp4_sm100.hpp).

Without a GPU: the header and its test program compile and link against the in-tree library.
With a GPU: the program runs an FFN program, a projection and a prefill linear through the
C++ types and compares with the CPU oracle (it exits non-zero on any mismatch).
"""
import importlib.util
import pathlib
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _builder():
    spec = importlib.util.spec_from_file_location("build_host_mirror_test", ROOT / "tests/cpp/build_host_mirror_test.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_host_mirror_compiles_and_links():
    binary = _builder().build()
    assert binary.exists() and binary.stat().st_size > 0


@pytest.mark.gpu
def test_host_mirror_runs_against_oracle():
    binary = _builder().build()
    done = subprocess.run([str(binary)], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    assert done.stdout.strip().splitlines()[-1] == "ok", done.stdout
