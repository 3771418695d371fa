"""Shared pytest set-up: the ``gpu`` marker, the repo root on ``sys.path``, golden vectors."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    """Vectors produced by the reference's own CPU code (tests/golden/make_golden.py)."""
    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    with np.load(path) as data:
        return {key: data[key] for key in data.files}


@pytest.fixture(autouse=True)
def _release_cuda_between_tests():
    yield
    import torch

    if torch.cuda.is_available():
        import gc

        gc.collect()
        torch.cuda.empty_cache()
