import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with `-m gpu` on the GPU box")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "kquant_golden.npz"))


@pytest.fixture(scope="session")
def cuda_lib():
    """The in-tree C-ABI library, built if needed (nvcc cross-compiles without a GPU)."""
    from llm_rs_b200 import build, load_library
    build.build()
    return load_library()


@pytest.fixture(scope="session")
def backend(cuda_lib):
    """A CudaBackend on cuda:0.  No fallback: without a B200 this raises and the test fails."""
    from llm_rs_b200 import CudaBackend
    be = CudaBackend(0)
    yield be
    be.close()
