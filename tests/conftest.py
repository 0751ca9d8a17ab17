import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def lib_built():
    """Build the shared library if it is stale (nvcc cross-compiles without a GPU)."""
    import luminal_jl_b200 as L
    from importlib import import_module
    build = import_module("luminal_jl_b200._build")
    build.build_library()
    return L


@pytest.fixture(scope="session")
def device(lib_built):
    return lib_built.get_device()
