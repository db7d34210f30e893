import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _build_native():
    """Compile libhapx.so when it is missing or stale and nvcc is here (it cross-compiles without a GPU)."""
    spec = importlib.util.spec_from_file_location("_hapx_build", os.path.join(ROOT, "hap_b200", "csrc", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    try:
        mod.build()
    except RuntimeError:
        if not os.path.exists(mod.LIB):
            raise


_build_native()

# Device-side waits on peers default to ten minutes (a late peer is not a dead one); a test that gets a
# collective wrong should fail in seconds instead.
os.environ.setdefault("HAPX_TIMEOUT_MS", "20000")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
