import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


# Every GEMM call made by a test is followed by a check of the kernels' status word: a bounded wait that ran
# out inside a kernel (results incomplete, no hang) fails the test that caused it instead of passing unseen.
os.environ.setdefault("PTB_DEBUG_STATUS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return REPO / "tests" / "golden"
