import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def oracle():
    from oracle import build_oracle, cpu

    build_oracle.build_restatement()
    return cpu


@pytest.fixture(scope="session")
def lib_built():
    """Make sure the CUDA library exists (compiles it when nvcc is here and it does not)."""
    import importlib.util

    path = os.path.join(ROOT, "llama.cl_b200", "build.py")
    spec = importlib.util.spec_from_file_location("_q4fc_build", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not os.path.exists(mod.LIB):
        mod.build()
    return mod.LIB
