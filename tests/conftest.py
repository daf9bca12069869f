"""Shared pytest configuration: the ``gpu`` marker and fixture loading."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Return a fixture as a dict of torch tensors / Python scalars."""
    with np.load(GOLDEN / f"{name}.npz") as data:
        result = {}
        for key in data.files:
            value = data[key]
            result[key] = value.item() if value.ndim == 0 else torch.from_numpy(value)
        return result
