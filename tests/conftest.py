"""Shared pytest configuration: the ``gpu`` marker, import paths and golden loaders."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "leanmoe-quant_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ops_golden():
    return dict(np.load(os.path.join(GOLDEN_DIR, "ops_golden.npz")))


@pytest.fixture(scope="session")
def hf_golden():
    return dict(np.load(os.path.join(GOLDEN_DIR, "hf_tiny_model_golden.npz")))
