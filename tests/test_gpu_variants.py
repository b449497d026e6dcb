"""The scan kernels exist in two variants each, picked by shape and dtype: the forward with 64- or 32-channel
tiles (variants 0 and 2), the backward with a producer warp or with the bulk copies issued by a compute thread
(variants 0 and 3).  The environment variables RGLRU_FWD_VARIANT / RGLRU_BWD_VARIANT force one variant for a
whole process, so each combination runs the parity cases in a child interpreter."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fwd,bwd", [("0", "0"), ("2", "3"), ("0", "3"), ("2", "0")])
def test_forced_kernel_variant_passes_the_parity_cases(fwd, bwd):
    env = dict(os.environ, RGLRU_FWD_VARIANT=fwd, RGLRU_BWD_VARIANT=bwd)
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_parity.py"), "-m", "gpu", "-q", "-x",
           "-k", "odd_shapes or config0 or bf16_io or golden", "-p", "no:cacheprovider"]
    res = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-1000:]
