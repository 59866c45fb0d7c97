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


@pytest.fixture(autouse=True)
def _library_state_does_not_leak(request):
    """Every GPU test starts from the library's defaults: kernel choice, options and dq path are
    process-wide settings, and the device status word is sticky until it is read.  With this reset
    no test depends on the order of collection (test_zz_no_alloc.py is named to run last only so
    that the fixed scratch array it uses is first touched after every other kernel has run)."""
    yield
    if "gpu" not in request.keywords:
        return
    import importlib
    import torch
    if not torch.cuda.is_available():
        return
    nsa = importlib.import_module("openbox-llm_b200")
    nsa.set_impl("auto")
    nsa.set_dq_accumulator(False)
    for name, value in (("sel_fwd_variant", 0), ("merged_boxes", 1), ("bwd_kernel", 1),
                        ("debug_starve_load", 0)):
        nsa.set_option(name, value)
    nsa.lib().nsa_device_status(None)          # reading clears the word


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
