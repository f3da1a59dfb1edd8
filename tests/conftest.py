import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The C-ABI library and the oracle are built in-tree; build them when the shared objects are missing."""
    from hipster_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from hipster_b200 import build
        build.build()
    from oracle import orc
    if not os.path.exists(orc.LIB_PATH):
        orc.build()
    yield


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:
        has = False
    if not has:
        skip = pytest.mark.skip(reason="no CUDA device")
        for it in items:
            if "gpu" in it.keywords:
                it.add_marker(skip)
