"""pytest configuration: markers, import paths and per-test compiler reset."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for entry in (ROOT, ROOT / "fast-attnres_b200"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


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
        if item.get_closest_marker("gpu") is not None:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _fresh_compiler(request):
    """Each GPU test starts with an empty Dynamo cache (the reference does the same,
    tests/conftest.py:7-11) so recompile counters are per test."""
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        torch.compiler.reset()
    yield
