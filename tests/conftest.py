import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native_lib():
    """The product library; built in-tree if stale (nvcc cross-compiles without a GPU)."""
    from jacq_b200 import build as _build
    _build.build()
    from jacq_b200 import _native
    return _native.lib()


@pytest.fixture(scope="session")
def ref_lib():
    """The reference's own CUDA, compiled unmodified into oracle/_ref (prebuilt where the
    reference checkout is absent)."""
    import ctypes
    path = ROOT / "oracle" / "_ref" / "libjacq_ref.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libjacq_ref.so not built (needs the reference checkout)")
    return ctypes.CDLL(str(path))
