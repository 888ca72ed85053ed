"""pytest configuration: the ``gpu`` marker and shared fixtures."""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Inputs and outputs produced by the reference's own code (see tests/golden/make_golden.py)."""
    with np.load(os.path.join(GOLDEN_DIR, "ref_vectors.npz")) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def golden_hashes():
    with open(os.path.join(GOLDEN_DIR, "ref_hashes.json")) as f:
        return json.load(f)
