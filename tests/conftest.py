"""Shared pytest set-up: marker registration, import path, golden-file loader."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict[str, torch.Tensor]:
    """Read one golden case as a dict of CPU tensors (bool masks stay bool)."""
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as data:
        return {k: torch.from_numpy(np.ascontiguousarray(data[k])) for k in data.files}


def params_of(case: dict[str, torch.Tensor], prefix: str = "p.") -> dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in case.items() if k.startswith(prefix)}
