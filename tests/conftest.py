import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The worst measured error of each kind of tensor over the session, next to its bound."""
    try:
        from tests.util import WORST
    except Exception:
        return
    if not WORST:
        return
    terminalreporter.write_line("worst measured errors (max-abs, rel-L2, fraction of the max-abs bound, where):")
    for key in sorted(WORST):
        ma, rl, frac, what = WORST[key]
        terminalreporter.write_line(f"  {key:<14s} {ma:.3e}  {rl:.3e}  {frac:5.2f}  {what}")
