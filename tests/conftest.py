import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_port():
    import oracle
    oracle.build()
    return oracle.port


@pytest.fixture(scope="session")
def oracle_ref():
    import oracle
    oracle.build()
    if not oracle.ref.available():
        pytest.skip("reference CPU build not present")
    return oracle.ref


def pytest_terminal_summary(terminalreporter):
    """The parity report: for every long FP32 reduction compared with the CPU path, how many elements miss the literal
    bound 1e-5 + 1e-4 |cpu| and what the test asserted instead (tests/util.py)."""
    try:
        from util import PARITY_REPORT
    except Exception:
        return
    if PARITY_REPORT:
        terminalreporter.section("parity report (device vs CPU path)")
        for line in PARITY_REPORT:
            terminalreporter.write_line(line)
