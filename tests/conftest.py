import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# short waits everywhere in tests: a missing peer must surface in seconds
os.environ.setdefault("HCCL_CONNECT_TIMEOUT", "60")
os.environ.setdefault("HCCL_EXEC_TIMEOUT", "20")


def _has_cuda_early():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


# On a host without a GPU (where sources are edited) make sure the native library is current before it is loaded;
# on a GPU box the library that travelled with the tree is used as is.
if not _has_cuda_early():
    import importlib.util

    _spec = importlib.util.spec_from_file_location("_hccl_b200_build", ROOT / "hccl_b200" / "build.py")
    _mod = importlib.util.module_from_spec(_spec)
    _spec.loader.exec_module(_mod)
    _mod.build()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


@pytest.fixture(scope="session")
def native_lib():
    from hccl_b200 import _lib

    return _lib.lib


def _has_cuda():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
