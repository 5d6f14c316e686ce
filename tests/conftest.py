import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PACKAGE = "llm-assisted-kernel-dev_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (its directory name is not a Python identifier)."""
    build = importlib.import_module(PACKAGE + ".build")
    build.build()
    return importlib.import_module(PACKAGE)


@pytest.fixture(scope="session")
def oracle():
    from oracle import nvfp4_oracle
    return nvfp4_oracle


@pytest.fixture(scope="session")
def c_oracle():
    from oracle import c_oracle as mod
    mod.load()
    return mod


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))
