"""C++ host layer (gern_b200/host): Gern-shaped programs lowered onto the C ABI.  The checks live
in tests/cpp/test_host.cpp; these wrappers build and run it."""
import subprocess

import pytest

from gern_b200.host import build_test


def run(mode):
    exe = build_test.build()
    res = subprocess.run([exe, mode], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all host-layer checks passed" in res.stdout


def test_composition_and_lowering_cpu():
    run("cpu")


@pytest.mark.gpu
def test_programs_evaluate_on_gpu():
    run("gpu")
