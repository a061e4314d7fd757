"""Shared test plumbing.

`-m "not gpu"` covers the CPU oracle (against hand-derived known answers and
the committed golden vectors), the host-side logic and the C-ABI surface;
`-m gpu` holds the parity tests proper, which call the CUDA library through
the C-ABI and compare with the oracle.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O

    O.load()
    return O


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def ops():
    """The product operators; importing them never falls back to anything."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import cannbench_operator_solutions_b200 as pkg

    pkg._lib.load()
    return pkg.ops
