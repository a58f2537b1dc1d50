import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on a B200 with -m gpu)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where there is no GPU."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """How close the bfloat16 rows of this session came to their bound (1.0 would fail)."""
    try:
        from replay import LARGEST_EXCESS
    except Exception:
        return
    if LARGEST_EXCESS["rows"]:
        terminalreporter.write_line(f"bfloat16 rows compared with the plain implementation: {LARGEST_EXCESS['rows']}, "
                                    f"largest distance {LARGEST_EXCESS['value']:.2f} of the bound")
