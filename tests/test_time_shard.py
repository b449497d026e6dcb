"""Time-sharded RG-LRU (griffin_b200/time_shard.py): the carry algebra on CPU against the oracle's sequential scan,
the three phases on one GPU against an unsplit call, and -- under a multi-process launch -- NCCL ranks holding time
slices against the oracle on the whole sequence (outputs and every gradient)."""

from __future__ import annotations

import os

import pytest
import torch

from oracle import rglru_oracle as orc

WORLD = int(os.environ.get("WORLD_SIZE", "1"))


def test_carry_fold_reproduces_the_unsplit_scan_on_cpu():
    from griffin_b200.time_shard import fold_entering_states
    torch.manual_seed(0)
    B, T, D = 2, 50, 6
    a = torch.rand(B, T, D, dtype=torch.float64) * 0.5 + 0.5
    b = torch.randn(B, T, D, dtype=torch.float64)
    h0 = torch.randn(B, D, dtype=torch.float64)
    states, last = orc.sequential_scan(a, b, h0)
    cuts = [0, 13, 14, 37, 50]
    prods, finals = [], []
    for lo, hi in zip(cuts, cuts[1:]):
        prods.append(a[:, lo:hi].prod(dim=1))
        finals.append(orc.sequential_scan(a[:, lo:hi], b[:, lo:hi], torch.zeros(B, D, dtype=torch.float64))[1])
    enter, end = fold_entering_states(prods, finals, h0)
    torch.testing.assert_close(end, last)
    for k, lo in enumerate(cuts[:-1]):
        want = h0 if lo == 0 else states[:, lo - 1]
        torch.testing.assert_close(enter[k], want)
    # reverse chain: g_{t-1} = a_t (dy_t + g_t); the carry entering a slice from its right equals the unsplit one
    dy = torch.randn(B, T, D, dtype=torch.float64)
    g = torch.zeros(B, D, dtype=torch.float64)
    carry_at = {}
    for t in range(T - 1, -1, -1):
        carry_at[t] = g
        g = a[:, t] * (dy[:, t] + g)
    locs = []
    for lo, hi in zip(cuts, cuts[1:]):
        gl = torch.zeros(B, D, dtype=torch.float64)
        for t in range(hi - 1, lo - 1, -1):
            gl = a[:, t] * (dy[:, t] + gl)
        locs.append(gl)
    enter_r, out_r = fold_entering_states(prods, locs, None, reverse=True)
    torch.testing.assert_close(out_r, g)
    for k, hi in enumerate(cuts[1:]):
        torch.testing.assert_close(enter_r[k], carry_at[hi - 1])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 4e-3)])
def test_slices_on_one_device_equal_the_unsplit_call(dtype, tol):
    from griffin_b200 import ops
    from griffin_b200.time_shard import run_slices_on_one_device
    gen = torch.Generator(device="cuda").manual_seed(5)
    B, T, D = 3, 700, 192
    x, u_r, u_i = (torch.randn(B, T, D, device="cuda", generator=gen).to(dtype) for _ in range(3))
    lam = orc.init_lambda(D, 8.0, torch.Generator().manual_seed(5)).cuda()
    h0 = torch.randn(B, D, device="cuda", generator=gen)
    with torch.no_grad():
        y, h_last = ops.rglru(x, u_r, u_i, lam, h0)
        cuts = [0, 130, 131, 450, 700]
        slices = [(x[:, lo:hi], u_r[:, lo:hi], u_i[:, lo:hi]) for lo, hi in zip(cuts, cuts[1:])]
        outs, last = run_slices_on_one_device(slices, lam, h0)
    assert orc.rel_l2(torch.cat(outs, dim=1), y) <= tol
    assert orc.rel_l2(last, h_last) <= 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 700, 192), (2, 150, 72)])       # the TMA-staged path and the plain-load path
def test_carry_only_passes_equal_the_full_calls_and_write_nothing_else(dtype, shape):
    """rglru_fwd_carry without y and rglru_bwd without gradient tensors return the carries of the full calls, and
    leave their inputs (over which their unused output descriptors are laid) untouched."""
    from griffin_b200 import check_device, ops
    from griffin_b200.time_shard import _reverse_carry, _scan_with_carry
    gen = torch.Generator(device="cuda").manual_seed(9)
    B, T, D = shape
    x, u_r, u_i, dy = (torch.randn(B, T, D, device="cuda", generator=gen).to(dtype) for _ in range(4))
    lam = orc.init_lambda(D, 8.0, torch.Generator().manual_seed(9)).cuda()
    h0, g_end = (torch.randn(B, D, device="cuda", generator=gen) for _ in range(2))
    keep = [t.clone() for t in (x, u_r, u_i, dy)]
    y, h_full, p_full, ws = _scan_with_carry(x, u_r, u_i, lam, h0, None, 8.0, True)
    none, h_c, p_c, ws_c = _scan_with_carry(x, u_r, u_i, lam, h0, None, 8.0, True, want_y=False)
    assert none is None and ws_c.numel() == 0
    # (the two calls may run different tile shapes, hence different summation orders inside a chunk)
    assert orc.rel_l2(h_c, h_full) <= 2e-6 and orc.rel_l2(p_c, p_full) <= 2e-6
    full = ops._rglru_bwd_impl(dy, g_end, x, u_r, u_i, lam, h0, None, ws, 8.0, True)
    carry = _reverse_carry(dy, g_end, x, u_r, u_i, lam, h0, None, ws, 8.0)
    assert orc.rel_l2(carry, full[4]) <= 2e-6
    for before, after in zip(keep, (x, u_r, u_i, dy)):
        assert torch.equal(before, after)
    again = ops._rglru_bwd_impl(dy, g_end, x, u_r, u_i, lam, h0, None, ws, 8.0, True)     # the workspace is still good
    for a, b in zip(full, again):
        assert torch.equal(a, b)
    check_device()


@pytest.mark.gpu
@pytest.mark.skipif(WORLD < 2, reason="needs a multi-process launch (torchrun)")
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_time_sharded_ranks_equal_the_oracle_on_the_whole_sequence(nccl_group, dtype, tol):
    from griffin_b200.time_shard import rglru_time_sharded
    dist = nccl_group
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    B, T, D = 2, 96 * world + 40, 128                 # uneven slices: the last rank gets 40 steps more
    gen = torch.Generator().manual_seed(23)
    x, u_r, u_i, dy = (torch.randn(B, T, D, generator=gen).to(dtype) for _ in range(4))
    lam = orc.init_lambda(D, 8.0, gen)
    h0, dh = torch.randn(B, D, generator=gen), torch.randn(B, D, generator=gen)
    want = orc.rglru_backward_linear(x.double(), u_r.double(), u_i.double(), lam.double(), dy.double(), h0=h0, dh_last=dh)

    lo = 96 * rank
    hi = T if rank == world - 1 else 96 * (rank + 1)
    xs, urs, uis = (t[:, lo:hi].to(dev).requires_grad_(True) for t in (x, u_r, u_i))
    lam_d = lam.to(dev).requires_grad_(True)
    h0_d = h0.to(dev).requires_grad_(True)
    y, h_end = rglru_time_sharded(xs, urs, uis, lam_d, h0_d)
    loss = (y.float() * dy[:, lo:hi].to(dev).float()).sum()
    if rank == world - 1:
        loss = loss + (h_end * dh.to(dev)).sum()      # the sequence's final state lives on the last rank
    loss.backward()
    dist.all_reduce(lam_d.grad)                        # parameter gradient: summed over the time slices
    h0_grad = h0_d.grad.clone()
    dist.broadcast(h0_grad, src=0)
    assert orc.rel_l2(y, want["y"][:, lo:hi]) <= tol
    if rank == world - 1:
        assert orc.rel_l2(h_end, want["h_last"]) <= tol
    assert orc.rel_l2(xs.grad, want["dx"][:, lo:hi]) <= tol
    assert orc.rel_l2(urs.grad, want["du_r"][:, lo:hi]) <= tol
    assert orc.rel_l2(uis.grad, want["du_i"][:, lo:hi]) <= tol
    assert orc.rel_l2(lam_d.grad, want["dLambda"]) <= tol
    assert orc.rel_l2(h0_grad, want["dh0"]) <= tol
    dist.barrier()
