import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pattern(idx):
    """The reference's deterministic test filler (src/selftest.rs:540-543,
    src/metal.rs:215-218): integer hash -> [-1, 1)."""
    i = np.asarray(idx, dtype=np.uint64)
    h = i * np.uint64(2654435761) + np.uint64(0x9E3779B9)
    return (((h >> np.uint64(13)) % np.uint64(2000)).astype(np.float32) / np.float32(1000.0)
            - np.float32(1.0)).astype(np.float32)


def pattern_matrix(rows, cols, offset=0):
    return pattern(np.arange(rows * cols, dtype=np.uint64) + np.uint64(offset)).reshape(rows, cols)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
