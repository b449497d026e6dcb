"""The scan kernels exist in several CTA shapes picked by a size heuristic (64 or 32 channels, 16 or 32
time-lanes, different ring depths).  The environment variables RGLRU_FWD_VARIANT / RGLRU_BWD_VARIANT force one
shape for a whole process, so each forced shape runs the odd-shape parity cases in a child interpreter."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["1", "2", "3"])
def test_forced_kernel_shape_passes_the_parity_cases(variant):
    env = dict(os.environ, RGLRU_FWD_VARIANT=variant, RGLRU_BWD_VARIANT=variant)
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_parity.py"), "-m", "gpu", "-q", "-x",
           "-k", "odd_shapes or config0 or bf16_io or golden", "-p", "no:cacheprovider"]
    res = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-1000:]
