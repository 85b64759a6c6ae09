"""Shared test configuration: the `gpu` marker, import paths, and the golden-vector loader."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE_DIR = os.path.join(ROOT, "latent-sparse-attention_b200")
for path in (ROOT, PACKAGE_DIR):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def golden(name: str):
    """Load one golden-vector file written by tests/golden/make_golden.py."""
    return np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))


@pytest.fixture(scope="session")
def oracle():
    import oracle as module

    module.build()
    return module
