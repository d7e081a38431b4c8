import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _library_options_follow_the_environment():
    """The library reads its FLASHMASK_B200_* switches once at load.  Tests that change them call
    ``_lib.reload_options()`` after setting the variable; this fixture is torn down after
    monkeypatch has restored the environment and makes the library read it again."""
    yield
    from flashmask_b200 import _lib
    if _lib._lib is not None:
        _lib.reload_options()
