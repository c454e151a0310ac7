import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = None
    for item in items:
        if "gpu" in item.keywords:
            if n is None:
                n = _gpu_count()
            if n == 0:
                item.add_marker(pytest.mark.skip(reason="no CUDA device"))
            elif "multigpu" in item.keywords and n < 2:
                item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(scope="session")
def built_library():
    """The C-ABI library, built if stale (nvcc cross-compiles without a GPU)."""
    from saga_b200.build import build_library
    return build_library()


@pytest.fixture(scope="session")
def oracle(built_library):
    from oracle import oracle as orc
    orc.lib()
    return orc
