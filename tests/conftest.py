import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The CUDA library and the oracle are built in-tree; build them when a fresh checkout lacks them."""
    from matxtract_b200 import build as mxbuild

    if not mxbuild.LIB.exists():
        mxbuild.build_all()
    import oracle

    if not (ROOT / "oracle" / "_build" / "liboracle.so").exists():
        oracle.build()
    yield


def has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False
