import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def gpu_packers():
    z = np.load(os.path.join(GOLDEN, "gpu_packers.npz"))
    cases = {}
    for k in z.files:
        c, name = k.split(".", 1)
        cases.setdefault(c, {})[name] = z[k]
    return cases


@pytest.fixture(scope="session")
def cpu_reference():
    return np.load(os.path.join(GOLDEN, "cpu_reference.npz"))


def random_ternary(rng, K, N, sparsity, dtype=np.int8):
    """i.i.d. P(0)=s, P(-1)=P(+1)=(1-s)/2 (the reference's non-uniform generator, TernaryLinear.py:79-83)."""
    r = rng.random((K, N))
    w = np.zeros((K, N), dtype)
    w[(r >= sparsity) & (r < (sparsity + 1) / 2)] = -1
    w[r >= (sparsity + 1) / 2] = 1
    return w
