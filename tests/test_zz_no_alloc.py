"""The allocation-free conv backward (rglru_conv_bwd_noalloc) against the ordinary one.

This file is collected last on purpose: a run that stops at the first failure has then already run
every other test.  The entry point serves hosts that may not allocate device memory where the
backward runs (a runtime that owns all device memory, a frozen serving memory plan, a callback in
which an allocation would synchronise); its scratch is a fixed array inside the library, shared by
all calls.  The test therefore calls it twice in a row with different inputs and sizes -- the second
call sees the first call's leftovers in the scratch -- and requires the same results as
rglru_conv_bwd with a caller-provided workspace, through the C ABI in both cases.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(B, T, D, dtype, seed, with_state, with_flags):
    gen = torch.Generator().manual_seed(seed)
    t = {
        "d_conv": torch.randn(B, T, D, generator=gen).to(dtype).to(DEV),
        "x_in": torch.randn(B, T, D, generator=gen).to(dtype).to(DEV),
        "w": (torch.randn(D, 4, generator=gen) * 0.5).to(DEV),
        "state": torch.randn(B, 3, D, generator=gen).to(dtype).to(DEV) if with_state else None,
        "tok": None,
    }
    if with_flags:
        seg = torch.arange(T)[None, :].repeat(B, 1)
        seg[:, T // 2:] = torch.arange(T - T // 2)
        t["tok"] = (3 - seg.clamp(max=3)).to(torch.uint8).to(DEV)
    return t


def _oracle_grads(t, B, T, D):
    """Gradients of sum(conv(x_in) * d_conv) from the CPU oracle in fp64; the token flags used here carry only
    the number of taps to cut (3 - min(position, 3)), so positions are recovered from them."""
    from oracle import rglru_oracle as orc
    x = t["x_in"].double().cpu().requires_grad_(True)
    w = t["w"].double().cpu().requires_grad_(True)
    b = torch.zeros(D, dtype=torch.float64, requires_grad=True)
    state = (torch.zeros(B, 3, D, dtype=torch.float64) if t["state"] is None else t["state"].double().cpu()).requires_grad_(True)
    seg = torch.full((B, T), 3, dtype=torch.long) if t["tok"] is None else 3 - (t["tok"].cpu().long() & 3)
    out, _ = orc.causal_conv_dense(x, w, b, state, seg)
    (out * t["d_conv"].double().cpu()).sum().backward()
    return {"dx": x.grad, "d_w": w.grad, "d_b": b.grad, "d_state": state.grad}


def _run(lib, name, t, B, T, D, io, with_ws):
    dtype = t["x_in"].dtype
    out = {
        "dx": torch.full((B, T, D), float("nan"), device=DEV, dtype=dtype),
        "d_w": torch.full((D, 4), float("nan"), device=DEV),
        "d_b": torch.full((D,), float("nan"), device=DEV),
        "d_state": torch.full((B, 3, D), float("nan"), device=DEV, dtype=dtype),
    }
    ptr = lambda x: None if x is None else x.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    head = (ptr(t["d_conv"]), ptr(t["x_in"]), ptr(t["w"]), ptr(t["state"]), ptr(t["tok"]), ptr(out["dx"]),
            ptr(out["d_w"]), ptr(out["d_b"]), ptr(out["d_state"]))
    if with_ws:
        nbytes = lib.rglru_conv_bwd_workspace_bytes(B, T, D)
        ws = torch.empty(nbytes, device=DEV, dtype=torch.uint8)
        rc = lib.rglru_conv_bwd(*head, ws.data_ptr(), nbytes, B, T, D, io, stream)
    else:
        rc = lib.rglru_conv_bwd_noalloc(*head, B, T, D, io, stream)
    assert rc == 0, (name, rc, lib.rglru_status_string(rc).decode())
    torch.cuda.synchronize()
    return out


def test_noalloc_conv_backward_matches_workspace_version_twice_in_a_row():
    from griffin_b200 import _lib
    from oracle.rglru_oracle import rel_l2
    lib = _lib.load()
    calls = [
        (3, 300, 136, torch.float32, _lib.F32, 11, True, True),
        (2, 70, 64, torch.bfloat16, _lib.BF16, 12, False, False),   # smaller: stale scratch beyond its rows
        (3, 300, 136, torch.float32, _lib.F32, 13, True, False),
    ]
    for B, T, D, dtype, io, seed, with_state, with_flags in calls:
        t = _case(B, T, D, dtype, seed, with_state, with_flags)
        got = _run(lib, "noalloc", t, B, T, D, io, with_ws=False)
        want = _run(lib, "workspace", t, B, T, D, io, with_ws=True)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for key in ("dx", "d_w", "d_b", "d_state"):
            assert torch.isfinite(got[key].float()).all(), key
            assert rel_l2(got[key], want[key]) <= tol, key
        # ... and against the oracle's conv (griffin/griffin.py:474-487 of the reference) differentiated by autograd
        ref = _oracle_grads(t, B, T, D)
        for key in ("dx", "d_w", "d_b") + (("d_state",) if with_state else ()):
            assert rel_l2(got[key], ref[key]) <= tol, (key, "oracle")


def test_noalloc_rejects_problems_beyond_its_fixed_scratch():
    from griffin_b200 import _lib
    lib = _lib.load()
    cap = lib.rglru_conv_bwd_noalloc_max_bytes()
    assert cap == 4 << 20
    B, T, D = 64, 8192, 5632   # needs far more than the fixed array; must be refused before any launch
    assert lib.rglru_conv_bwd_workspace_bytes(B, T, D) > cap
    tiny = torch.zeros(64, device=DEV)
    p = tiny.data_ptr()
    rc = lib.rglru_conv_bwd_noalloc(p, p, p, None, None, p, p, None, None, B, T, D, _lib.F32, None)
    assert rc == _lib.ERR_TOO_LARGE
    assert "capacity" in lib.rglru_status_string(rc).decode()
    with pytest.raises(ValueError):
        _lib.check(rc, "rglru_conv_bwd_noalloc")
    torch.cuda.synchronize()
