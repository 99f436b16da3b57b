import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def reference_path(*parts: str) -> str:
    """Path inside a checkout of the reference project, for the tests that read its sample files when it is
    available: ``FBAM_REFERENCE_DIR``, else a directory named ``reference`` beside this repository."""
    import os
    base = os.environ.get("FBAM_REFERENCE_DIR") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    return os.path.join(base, *parts)
