import os
import shutil
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib_path():
    """Path of build/libnanoserve.so, compiled on demand when nvcc is available."""
    from nanoserve_b200 import build as b
    if shutil.which(os.environ.get("NVCC", "nvcc")):
        return b.build()
    if os.path.exists(b.LIB_PATH):
        return b.LIB_PATH
    pytest.fail("build/libnanoserve.so is missing and nvcc is not available to build it")


@pytest.fixture(scope="session")
def kernels(lib_path):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible (there is no CPU fallback)")
    from nanoserve_b200.ops import Kernels
    k = Kernels(lib_path)
    k.init()
    return k
