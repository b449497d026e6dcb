"""Batch sharding of the CUDA path over the GPUs of one box, checked against the unsharded oracle.

Run under a launcher, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        -m pytest tests/test_gpu_sharded_nccl.py -m gpu -q

Each rank runs ``RG_LRU(scan_mode="cuda")`` / ``RecurrentBlock`` forward and backward on its rows of a seeded
batch; the parameter gradients are summed with one NCCL all-reduce (``allreduce_parameter_grads``); every rank
compares its slice of the outputs and input gradients, and the summed parameter gradients, with the oracle
run on the WHOLE batch.  There is no collective on the data path and no peer access.  Without a launcher
(WORLD_SIZE unset or 1) the tests are skipped.
"""

from __future__ import annotations

import os

import pytest
import torch

from oracle import rglru_oracle as orc

WORLD = int(os.environ.get("WORLD_SIZE", "1"))
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(WORLD < 2, reason="needs a multi-process launch (torchrun)")]


@pytest.fixture(scope="module")
def group(nccl_group):
    return nccl_group


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_sharded_layer_equals_unsharded_oracle(group, dtype, tol):
    from griffin_b200 import RG_LRU
    from griffin_b200.sharding import allreduce_parameter_grads, batch_shard
    rank, world = group.get_rank(), group.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    B, T, D, G = 8, 320, 256, 4
    case = orc.make_rglru_case(B, T, D, G, seed=11)
    names = ("Lambda", "recurrence_gate.weight", "recurrence_gate.bias", "input_gate.weight", "input_gate.bias")
    params = {k: case[k].to(dtype).float() for k in names}
    x_all, dy_all = case["x"].to(dtype), case["dy"].to(dtype)

    ref_params = {k: v.clone().requires_grad_(True) for k, v in params.items()}
    xr = x_all.float().clone().requires_grad_(True)
    yr, hr = orc.rglru_layer_linear_backward(xr, ref_params)
    (yr * dy_all.float()).sum().backward()

    lo, hi = batch_shard(B, rank, world)
    module = RG_LRU(D, gate_blocks=G, scan_mode="cuda")
    module.load_state_dict(params)
    module = module.to(dev, dtype)
    x = x_all[lo:hi].detach().to(dev).requires_grad_(True)
    y, h_last = module(x, return_state=True)
    (y.float() * dy_all[lo:hi].to(dev).float()).sum().backward()
    allreduce_parameter_grads(module)

    assert orc.rel_l2(y, yr[lo:hi]) <= tol
    assert orc.rel_l2(h_last, hr[lo:hi]) <= tol
    assert orc.rel_l2(x.grad, xr.grad[lo:hi]) <= tol
    got = dict(module.named_parameters())
    for k in names:
        assert orc.rel_l2(got[k].grad, ref_params[k].grad) <= tol, (k, rank)


def test_sharded_block_equals_unsharded_oracle(group):
    from griffin_b200 import RecurrentBlock
    from griffin_b200.sharding import allreduce_parameter_grads, batch_shard
    rank, world = group.get_rank(), group.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(17)                       # the same parameters and data on every rank
    B, T, DM, DR = 8, 200, 32, 256
    blk = RecurrentBlock(DM, DR, gate_blocks=4, scan_mode="cuda", fold_merge=True)
    with torch.no_grad():
        blk.temporal_conv.weight.normal_(0.0, 0.5)
    params = {k: v.detach().clone().requires_grad_(True) for k, v in blk.state_dict().items()}
    x_all, dout = torch.randn(B, T, DM), torch.randn(B, T, DM)
    xr = x_all.clone().requires_grad_(True)
    ref, _ = orc.recurrent_block(xr, params, linear_backward=True)
    (ref * dout).sum().backward()

    lo, hi = batch_shard(B, rank, world)
    blk = blk.to(dev)
    x = x_all[lo:hi].to(dev).requires_grad_(True)
    out = blk(x)
    (out * dout[lo:hi].to(dev)).sum().backward()
    allreduce_parameter_grads(blk)
    assert orc.rel_l2(out, ref[lo:hi]) <= 1e-5
    assert orc.rel_l2(x.grad, xr.grad[lo:hi]) <= 1e-5
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad, params[key].grad) <= 2e-5, (key, rank)
