import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


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


# Achieved parity errors, printed after the run (also with -q) so that a log of the GPU suite shows how far inside
# its stated tolerance every comparison landed.
_ACHIEVED = []


def report_achieved(case, **values):
    """Record named achieved errors of one parity comparison: report_achieved("c2 bf16", hist=1.2e-3, loss=4e-6)."""
    _ACHIEVED.append((case, values))


@pytest.fixture
def achieved():
    return report_achieved


def pytest_terminal_summary(terminalreporter):
    if not _ACHIEVED:
        return
    terminalreporter.section("achieved parity errors (rel = |x-ref|_F/|ref|_F unless named otherwise)")
    for case, values in _ACHIEVED:
        terminalreporter.write_line(case + ": " + "  ".join(
            f"{k}={v:.2e}" if isinstance(v, float) else f"{k}={v}" for k, v in values.items()))
