"""World-size-2 CPU (gloo) check of the batch-sharding rule: each rank runs the oracle on its own rows,
parameter gradients are summed with one all-reduce, and the result equals the unsharded run."""

from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import sys
    sys.path.insert(0, ROOT)
    from griffin_b200.sharding import allreduce_parameter_grads, batch_shard
    from oracle import rglru_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    case = orc.make_rglru_case(5, 24, 16, 4, seed=3)
    names = ("Lambda", "recurrence_gate.weight", "recurrence_gate.bias", "input_gate.weight", "input_gate.bias")
    holder = torch.nn.ParameterDict({k.replace(".", "_"): torch.nn.Parameter(case[k].clone()) for k in names})
    params = {k: holder[k.replace(".", "_")] for k in names}
    lo, hi = batch_shard(5, rank, world)
    x = case["x"][lo:hi].clone().requires_grad_(True)
    y, h_last = orc.rglru_layer(x, params)
    (y * case["dy"][lo:hi]).sum().backward()
    allreduce_parameter_grads(holder)
    torch.save({"y": y.detach(), "dx": x.grad, "h_last": h_last.detach(), "lo": lo, "hi": hi,
                "grads": {k: params[k].grad for k in names}}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_batch_shard_ranges():
    from griffin_b200.sharding import batch_shard
    for batch in (0, 1, 5, 8, 64):
        for world in (1, 2, 3, 8):
            spans = [batch_shard(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_sharded_gradients_equal_unsharded(tmp_path):
    from oracle import rglru_oracle as orc
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    case = orc.make_rglru_case(5, 24, 16, 4, seed=3)
    names = ("Lambda", "recurrence_gate.weight", "recurrence_gate.bias", "input_gate.weight", "input_gate.bias")
    params = {k: case[k].clone().requires_grad_(True) for k in names}
    x = case["x"].clone().requires_grad_(True)
    y, h_last = orc.rglru_layer(x, params)
    (y * case["dy"]).sum().backward()
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    torch.testing.assert_close(torch.cat([p["y"] for p in parts]), y.detach(), atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(torch.cat([p["dx"] for p in parts]), x.grad, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(torch.cat([p["h_last"] for p in parts]), h_last.detach(), atol=1e-6, rtol=1e-6)
    for r in range(world):  # every rank holds the full sum
        for k in names:
            torch.testing.assert_close(parts[r]["grads"][k], params[k].grad, atol=2e-5, rtol=2e-5)
