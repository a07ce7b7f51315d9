import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc
    orc.build()
    orc.lib()
    return orc


def pytest_terminal_summary(terminalreporter):
    """One line per test with the worst error it measured relative to its bar (see util.assert_close)."""
    try:
        import util
    except ImportError:
        return
    if not util.RECORDS:
        return
    terminalreporter.write_line("measured parity margins (worst |err| / bound per test; 1.0 = at the bar):")
    for test, (ratio, err, what) in sorted(util.RECORDS.items()):
        terminalreporter.write_line("  %-100s %8.3g  (|err| %.3g, %s)" % (test, ratio, err, what))
