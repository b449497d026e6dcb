"""Batch sharding of the RG-LRU path across the GPUs of one box.

Batch rows are independent recurrences, so rank k of n simply owns rows
[k*B/n, (k+1)*B/n) of every [B, T, D] tensor in its own HBM and the scan needs no
collective.  The only cross-rank sums are those of parameter gradients (Lambda, the gate
projections, the conv taps), which are reductions over the batch.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def batch_shard(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [begin, end) of ``rank``; the first ``batch % world`` ranks take one extra row."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"invalid rank {rank} for world size {world}")
    if batch < 0:
        raise ValueError("batch must be non-negative")
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def allreduce_parameter_grads(module: torch.nn.Module, group=None) -> None:
    """Sum parameter gradients over ranks in place (one flat fp32 all-reduce), for checking sharded
    gradients against an unsharded run or for plain data-parallel training without DDP."""
    grads = [p.grad for p in module.parameters() if p.grad is not None]
    if not grads or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    flat = torch.cat([g.reshape(-1).to(torch.float32) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    offset = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[offset:offset + n].view_as(g))
        offset += n
