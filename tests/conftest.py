import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
QTYPES = {10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_golden(qtype):
    import numpy as np
    return np.load(os.path.join(GOLDEN, f"kquant_{QTYPES[qtype]}.npz"))


@pytest.fixture(params=sorted(QTYPES))
def qtype(request):
    return request.param
