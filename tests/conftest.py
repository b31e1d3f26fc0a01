"""pytest configuration: the ``gpu`` marker and import paths for the package and the oracle."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def mlxq():
    """The product package (loads libmlxq.so; builds it first if it is missing and nvcc is here)."""
    lib = os.path.join(ROOT, "mlx-runner_b200", "lib", "libmlxq.so")
    if not os.path.exists(lib):
        spec = importlib.util.spec_from_file_location("mlxq_build", os.path.join(ROOT, "mlx-runner_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return importlib.import_module("mlx-runner_b200")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure)."""
    from oracle import oracle as o
    o.lib()
    return o
