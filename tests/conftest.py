"""Test configuration: registers the `gpu` marker and puts the repository root on sys.path.

`-m "not gpu"` tests run on a CPU-only machine (oracle against the golden vectors, host logic, library exports);
`-m gpu` tests are the parity tests proper and need a B200 plus the built CUDA library (they fail, not skip, without it).
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")
if GOLDEN not in sys.path:
    sys.path.insert(0, GOLDEN)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200) and the built CUDA library")
