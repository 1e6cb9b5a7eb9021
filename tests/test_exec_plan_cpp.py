"""The execution-plan layer above the C ABI (include/augur_nvfp4_sm100_exec.hpp), after the reference's
crates/augur-compiler/tests/m47_mxfp4_execution_plan.rs.

Without a GPU: the lowering stage (entry selected by address, weight requirements, unsupported nodes) runs here.
With a GPU: bind, eight executions against the oracle with a stable weight owner, per-kind profiling.
"""
import importlib.util
import pathlib
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _binary():
    spec = importlib.util.spec_from_file_location("build_host_mirror_test", ROOT / "tests/cpp/build_host_mirror_test.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.build("exec_plan_test")


def test_lowering_selects_entries_and_rejects_unsupported_nodes():
    done = subprocess.run([str(_binary()), "--cpu"], capture_output=True, text=True, timeout=120)
    assert done.returncode == 0, done.stdout + done.stderr
    assert done.stdout.strip().splitlines()[-1] == "ok", done.stdout


@pytest.mark.gpu
def test_bound_plan_executes_against_the_oracle():
    done = subprocess.run([str(_binary())], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    assert done.stdout.strip().splitlines()[-1] == "ok", done.stdout
