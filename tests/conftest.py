"""pytest configuration: the ``gpu`` marker, import paths, and a GPU-presence guard."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "cta-pipelining_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu(n): needs at least n CUDA devices; skipped on smaller boxes")


def pytest_collection_modifyitems(config, items):
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        mk = item.get_closest_marker("multigpu")
        if mk is not None and n < int(mk.args[0]):
            item.add_marker(pytest.mark.skip(reason=f"needs {mk.args[0]} CUDA devices, have {n}"))
