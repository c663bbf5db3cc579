import os
import sys

import pytest

# The engine hands products with few tiles to the library (they are faster there); the tiny models of these tests
# would then never reach the engine's own tcgen05 kernels, so the tests ask for them from the first tile on.
# test_engine_gpu.py::test_product_dispatch_by_tiles checks the rule itself.
os.environ.setdefault("IIAN_TCGEN05_MIN_TILES", "0")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
