"""Shared pytest configuration: registers the ``gpu`` marker, puts the repository root on
``sys.path`` and exposes the golden fixtures."""

import json
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


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_graphs():
    with open(os.path.join(GOLDEN, "intents.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_verdicts():
    with open(os.path.join(GOLDEN, "verdicts.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_vectors():
    with np.load(os.path.join(GOLDEN, "vectors.npz")) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def golden_edges():
    with np.load(os.path.join(GOLDEN, "edge_cases.npz")) as z:
        return {k: z[k] for k in z.files}
