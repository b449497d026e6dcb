"""World-size-2 CPU (gloo) check of the time split's multi-rank plumbing: the carry-only pass, the all-gather,
the fold and the full pass of griffin_b200.time_shard run on two ranks with the three kernel calls replaced by
the oracle's arithmetic (the kernels themselves are covered on GPUs); outputs and every gradient must equal the
oracle on the whole sequence."""

from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

B, D, CUT, T = 2, 12, 17, 40      # uneven slices: 17 and 23 steps


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case():
    from oracle import rglru_oracle as orc
    gen = torch.Generator().manual_seed(31)
    x, u_r, u_i, dy = (torch.randn(B, T, D, generator=gen, dtype=torch.float64) for _ in range(4))
    lam = orc.init_lambda(D, 8.0, gen).double()
    h0, dh = (torch.randn(B, D, generator=gen, dtype=torch.float64) for _ in range(2))
    return x, u_r, u_i, dy, lam, h0, dh


def _install_oracle_backends():
    """Stand-ins with the signatures of the three kernel wrappers time_shard calls."""
    from griffin_b200 import ops, time_shard
    from oracle import rglru_oracle as orc

    def scan_with_carry(x, u_r, u_i, lam, h0, tok, c, save, want_y=True):
        a, _ = orc.gate_epilogue(x, u_r, u_i, lam, c, None, None)
        r = orc.rglru_backward_linear(x, u_r, u_i, lam, torch.zeros_like(x), h0=h0, c=c)    # (its forward half, in fp64)
        return (r["y"] if want_y else None), r["h_last"], a.prod(dim=1), torch.empty(0)

    def full_backward(dy, g_end, x, u_r, u_i, lam, h0, tok, ws, c, want_dh0):
        r = orc.rglru_backward_linear(x, u_r, u_i, lam, dy, h0=h0, dh_last=g_end, c=c)
        return r["dx"], r["du_r"], r["du_i"], r["dLambda"], r["dh0"]

    def reverse_carry(dy, g_end, x, u_r, u_i, lam, h0, tok, ws, c):
        return full_backward(dy, g_end, x, u_r, u_i, lam, h0, tok, ws, c, True)[4]

    time_shard._scan_with_carry = scan_with_carry
    time_shard._reverse_carry = reverse_carry
    ops._rglru_bwd_impl = full_backward


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from griffin_b200 import time_shard
    _install_oracle_backends()
    x, u_r, u_i, dy, lam, h0, dh = _case()
    lo, hi = (0, CUT) if rank == 0 else (CUT, T)
    xs, urs, uis = (t[:, lo:hi].clone().requires_grad_(True) for t in (x, u_r, u_i))
    lam_r, h0_r = lam.clone().requires_grad_(True), h0.clone().requires_grad_(True)
    y, h_end = time_shard._TimeShardedRGLRU.apply(xs, urs, uis, lam_r, h0_r, None, 8.0, None)
    loss = (y * dy[:, lo:hi]).sum()
    if rank == world - 1:
        loss = loss + (h_end * dh).sum()          # the sequence's final state lives on the last rank
    loss.backward()
    dist.all_reduce(lam_r.grad)                    # parameter gradient: summed over the time slices
    torch.save({"y": y.detach(), "h_end": h_end.detach(), "dx": xs.grad, "du_r": urs.grad, "du_i": uis.grad,
                "dlam": lam_r.grad, "dh0": h0_r.grad}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_time_slices_on_gloo_ranks_equal_the_whole_sequence(tmp_path):
    from oracle import rglru_oracle as orc
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    x, u_r, u_i, dy, lam, h0, dh = _case()
    want = orc.rglru_backward_linear(x, u_r, u_i, lam, dy, h0=h0, dh_last=dh)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    close = dict(atol=2e-6, rtol=2e-6)      # Lambda and the carried states travel as fp32, as on the GPU
    torch.testing.assert_close(torch.cat([p["y"] for p in parts], dim=1), want["y"], **close)
    torch.testing.assert_close(parts[-1]["h_end"], want["h_last"], **close)
    for key in ("dx", "du_r", "du_i"):
        torch.testing.assert_close(torch.cat([p[key] for p in parts], dim=1), want[key], **close)
    for p in parts:                                # every rank holds the summed parameter gradient
        torch.testing.assert_close(p["dlam"], want["dLambda"], **close)
    torch.testing.assert_close(parts[0]["dh0"], want["dh0"], **close)      # produced on rank 0
    assert float(parts[1]["dh0"].abs().max()) == 0.0
