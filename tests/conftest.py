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


@pytest.fixture(scope="session")
def nccl_group():
    """The NCCL process group of a torchrun launch, one per pytest session: set up on first use and torn down when
    the session ends (a second group created after a destroyed one can pick the first one's stale rendezvous keys
    out of the store).  Tests that need it are skipped by their own markers when WORLD_SIZE is unset."""
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    yield dist
    dist.barrier()
    dist.destroy_process_group()


def load_golden(name: str) -> dict[str, torch.Tensor]:
    """Read one golden case as a dict of CPU tensors (bool masks stay bool)."""
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as data:
        return {k: torch.from_numpy(np.ascontiguousarray(data[k])) for k in data.files}


def params_of(case: dict[str, torch.Tensor], prefix: str = "p.") -> dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in case.items() if k.startswith(prefix)}
