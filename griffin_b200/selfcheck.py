"""Once-per-device known-answer check of the CUDA scan (the role of ``triton_scan_is_usable`` /
``_validate_triton_scan`` in the reference, griffin/triton_scan.py:139-204).

The reference validates its Triton kernels on closed-form inputs before it lets the automatic dispatch use
them and otherwise falls back to a portable scan.  This package has no other backend to fall back to, so the
check is an explicit diagnostic: ``cuda_scan_is_usable(device)`` answers False on anything that is not a CUDA
device with the library loaded and the kernels reproducing the recurrence; ``strict=True`` raises instead.
"""

from __future__ import annotations

import threading
import warnings

import torch

_LOCK = threading.Lock()
_CHECKED: dict[tuple[str, int], bool] = {}

STEPS, WIDTH = 7, 257     # one full 256-wide tile plus a partial one, as in the reference's self-test


def _known_answer_case(device: torch.device):
    k = torch.arange(STEPS * WIDTH, device=device, dtype=torch.float32)
    decay = (0.9 + 0.05 * torch.sin(k / 97.0)).reshape(1, STEPS, WIDTH)
    drive = (0.1 * torch.cos(k / 53.0)).reshape(1, STEPS, WIDTH)
    h0 = torch.sin(torch.arange(WIDTH, device=device, dtype=torch.float32) / 31.0)[None]
    upstream = torch.cos(k / 71.0).reshape(1, STEPS, WIDTH)
    return decay, drive, h0, upstream


def _loop_scan(decay, drive, h0):
    h, rows = h0, []
    for t in range(decay.size(1)):
        h = decay[:, t] * h + drive[:, t]
        rows.append(h)
    return torch.stack(rows, dim=1)


def _run_check(device: torch.device) -> None:
    from . import ops

    decay, drive, h0, upstream = _known_answer_case(device)
    want_in = [t.clone().requires_grad_(True) for t in (decay, drive, h0)]
    got_in = [t.clone().requires_grad_(True) for t in (decay, drive, h0)]
    want = _loop_scan(*want_in)
    got = ops.linear_scan(*got_in)
    want_grads = torch.autograd.grad(want, want_in, upstream)
    got_grads = torch.autograd.grad(got, got_in, upstream)
    torch.cuda.synchronize(device)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-5)
    for g, w in zip(got_grads, want_grads):
        torch.testing.assert_close(g, w, atol=3e-5, rtol=3e-5)


def cuda_scan_is_usable(device, *, strict: bool = False) -> bool:
    """Whether the CUDA scan kernels load and reproduce the recurrence on ``device`` (checked once per device)."""
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        if strict:
            raise RuntimeError("the CUDA scan needs a CUDA device; there is no CPU fallback")
        return False
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = (dev.type, dev.index)
    with _LOCK:
        if key not in _CHECKED:
            try:
                with torch.enable_grad(), torch.cuda.device(dev):
                    _run_check(dev)
                _CHECKED[key] = True
            except Exception as error:   # a missing library, a launch failure and a wrong answer all mean "unusable"
                _CHECKED[key] = False
                if strict:
                    raise RuntimeError(f"CUDA RG-LRU scan failed its self-check on {dev}: {error}") from error
                warnings.warn(f"CUDA RG-LRU scan failed its self-check on {dev}: {error}", RuntimeWarning, stacklevel=2)
        elif strict and not _CHECKED[key]:
            raise RuntimeError(f"CUDA RG-LRU scan failed its self-check on {dev} earlier in this process")
        return _CHECKED[key]
