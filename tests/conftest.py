import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The largest logit error the engine tests saw, relative to the largest logit, per dtype."""
    mh = sys.modules.get("model_helpers")
    for dtype, ratio in sorted(getattr(mh, "OBSERVED", {}).items()):
        terminalreporter.write_line(f"largest logit error / largest logit, {dtype}: {ratio:.3e}")
