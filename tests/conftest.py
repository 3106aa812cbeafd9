import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without a GPU is an error of the invocation, not a skip: the
    # library has no CPU path. The driver selects with -m gpu / -m "not gpu".
    pass


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device (there is no CPU fallback)"
    assert torch.cuda.get_device_capability(0)[0] == 10, "kernels are built for sm_100a only"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _default_gemm_variant():
    """Every test starts and ends with the calling thread's tile-variant word at 0 (automatic selection), so that no
    test depends on what an earlier one left in the library. Skipped silently while the library is not built."""
    try:
        from rocmlir_b200 import _lib as L
        lib = L.lib()
    except Exception:
        yield
        return
    lib.rbSetGemmVariant(0)
    yield
    lib.rbSetGemmVariant(0)
