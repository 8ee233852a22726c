import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


# Figures the parity tests want shown even when they pass (error sizes, mismatch counts): collected here and
# printed once in the terminal summary, which "-q" keeps.
_PARITY_LINES = []


@pytest.fixture
def parity_report():
    """Callable that records one line for the "parity figures" section of the run's summary."""
    return _PARITY_LINES.append


def pytest_terminal_summary(terminalreporter):
    if _PARITY_LINES:
        terminalreporter.section("parity figures")
        for line in _PARITY_LINES:
            terminalreporter.write_line(line)
