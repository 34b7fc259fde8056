import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def pytest_sessionstart(session):
    """A fresh checkout holds sources only: compile the library (nvcc cross-compiles without a GPU)
    before any test imports it.  Where nvcc is absent too (a GPU box that received the built
    library with the tree) this is a no-op; a missing library then fails the tests loudly."""
    lib = os.path.join(ROOT, "gern_b200", "libgern_b200.so")
    if os.path.exists(lib):
        return
    try:
        from gern_b200 import build
        build.build()
    except Exception as e:  # noqa: BLE001 - reported by the tests that need the library
        sys.stderr.write(f"could not build libgern_b200.so: {e}\n")


@pytest.fixture(scope="session")
def oracle():
    from oracle import pyoracle
    return pyoracle.Oracle()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def golden_maker():
    """tests/golden/make_golden.py as a module: the tests regenerate the operands of the bf16
    fixtures with its bf16_inputs() instead of storing them."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def ctx():
    """The library context on cuda:0.  The shared library must already be built in-tree; there is
    no fallback."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test run without a GPU"
    from gern_b200 import api
    c = api.Context(0)
    yield c
    c.sync()
    c.close()
