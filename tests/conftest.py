import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA GPU (run with -m gpu on a GPU box)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA GPUs")


def _gpu_count():
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = _gpu_count()
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA GPU"))
        want = int(os.environ.get("MEGRAY_TEST_NPROC", "2"))
        if "multigpu" in item.keywords and n < want:
            item.add_marker(pytest.mark.skip(reason=f"needs {want} GPUs"))


@pytest.fixture(scope="session", autouse=True)
def _native_library():
    """Build (if stale) and load libmegray.so once per session."""
    from megray_b200 import build, _lib

    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    _lib.load()
    yield
