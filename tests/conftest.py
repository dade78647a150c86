import os
import sys
from pathlib import Path

import pytest

os.environ.setdefault("SFM_CHECK_STATUS", "1")   # tests read the kernels' status word after every call
ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "monarch_golden.npz")
