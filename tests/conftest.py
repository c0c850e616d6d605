import os
import sys

import pytest

# The reference's CPU engine calls a pthread OpenBLAS inside OpenMP loops (engine/src/conv_ops.cpp:109-175): one BLAS thread
# per OpenMP thread keeps its summation order fixed and stops the two thread pools from fighting over the cores.
os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def rel_l2(a, b):
    """||a - b|| / ||b|| in double precision (||b|| = 0 -> absolute norm)."""
    import numpy as np
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a))


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
