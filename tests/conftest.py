import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from kvmix_b200 import _lib
    _lib.lib()          # fail loudly if the library is not built
    return torch.device("cuda:0")


def pytest_terminal_summary(terminalreporter):
    """List the rounding-dominated rows admitted by the attention parity checks (tests/util.py)."""
    try:
        import util
    except Exception:
        return
    if util.ROUNDING_DOMINATED:
        terminalreporter.write_line("rounding-dominated rows admitted beyond 2e-3 (test, rows, worst error, upstream's own narrowing noise):")
        for rec in util.ROUNDING_DOMINATED:
            terminalreporter.write_line("  %s: %d row(s), %.3e (noise %.3e)" % rec)
