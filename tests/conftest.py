import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def pytest_terminal_summary(terminalreporter):
    """The differences the parity tests observed (helpers.observed), one line each."""
    try:
        from helpers import OBSERVED
    except ImportError:
        return
    if OBSERVED:
        terminalreporter.section("observed differences")
        for line in OBSERVED:
            terminalreporter.write_line(line)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O
