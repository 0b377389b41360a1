import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "lut6_golden.npz"))


def golden_cases(prefix):
    """Case keys 'prefix_...'(without the trailing array name) present in the golden file."""
    z = np.load(os.path.join(ROOT, "tests", "golden", "lut6_golden.npz"))
    keys = sorted({k[: -len("_idx")] for k in z.files if k.startswith(prefix + "_") and k.endswith("_idx")})
    return keys
