"""RG-LRU over a sequence that is split along TIME across the GPUs of one box.

Batch sharding (``griffin_b200.sharding``) needs no communication, but it cannot help when a single
sequence is too long for one GPU.  Here rank k of n holds time slice k of every ``[B, T, D]`` tensor.
A slice of the recurrence is an affine map of the state that enters it,

    h_out = P * h_in + h_local,      P = prod_t a_t,  h_local = the final state from h_in = 0,

(the associative operator of the reference's ``_associative_scan``, griffin/griffin.py:291-306, applied
to whole slices), so the slices are chained with ONE small exchange: every rank scans its slice from a
zero state in a carry-only pass (``rglru_fwd_carry`` without an output tensor: it reads its inputs and
returns P and h_local, nothing else leaves the chip), the ``[B, D]`` pairs ``(P, h_local)`` are all-gathered,
every rank folds the pairs of the ranks before it into the state entering its own slice, and scans again,
in full, from that state.  The backward does the same in reverse: a carry-only pass of ``rglru_bwd`` (no
gradient tensors, only ``dh0_local``), one all-gather, the full pass with the true incoming carry.  The price
of the time split is the carry-only pass (3/4 of a forward's traffic, 4/7 of a backward's) on every rank;
the exchange is ``3 * B * D`` floats per rank and step.  A group of one runs the ordinary single pass.

The reference has no counterpart.  Collectives are plain ``torch.distributed`` all-gathers (NCCL on GPUs);
there is no peer access.  The carry algebra is separated from the communication so that it can be tested
without GPUs (``fold_entering_states``) and on one GPU (``run_slices_on_one_device``).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import Tensor

from . import _lib, ops


def fold_entering_states(decay_prod: Sequence[Tensor], local_final: Sequence[Tensor], first: Optional[Tensor],
                         reverse: bool = False) -> tuple[list[Tensor], Tensor]:
    """Chain the per-slice pairs (P_k, state left by slice k when it starts from zero).

    Forward order (``reverse=False``): ``enter[0] = first`` (or zero) and ``enter[k+1] = P_k * enter[k] + local_k``.
    ``reverse=True`` chains from the last slice towards the first (the backward's carry).  Returns the state
    entering every slice and the state that leaves the chain's far end.
    """
    n = len(decay_prod)
    order = range(n - 1, -1, -1) if reverse else range(n)
    state = torch.zeros_like(local_final[0]) if first is None else first.to(local_final[0].dtype)
    enter: list[Optional[Tensor]] = [None] * n
    for k in order:
        enter[k] = state
        state = torch.addcmul(local_final[k], decay_prod[k], state)
    return enter, state  # type: ignore[return-value]


def _scan_with_carry(x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor],
                     c: float, save: bool, want_y: bool = True) -> tuple[Optional[Tensor], Tensor, Tensor, Tensor]:
    """(y, h_last, decay_prod, workspace) of one slice through ``rglru_fwd_carry``; ``want_y=False`` is the
    carry-only pass (y is None and no workspace is written)."""
    lib = _lib.load()
    dt = ops._io_dtype(x, "time-sharded forward")
    B, T, D = x.shape
    y = torch.empty_like(x) if want_y else None
    h_last = torch.empty(B, D, device=x.device, dtype=torch.float32)
    prod = torch.empty(B, D, device=x.device, dtype=torch.float32)
    save = save and want_y
    nbytes = lib.rglru_workspace_bytes(B, T, D, dt) if save else 0
    ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
    with ops._on(x, "rglru_fwd_carry"):
        rc = lib.rglru_fwd_carry(ops._ptr(x), ops._ptr(u_r), ops._ptr(u_i), ops._ptr(lam), ops._ptr(h0), ops._ptr(tok),
                                 ops._ptr(y), ops._ptr(h_last), ops._ptr(prod), ops._ptr(ws) if save else None, nbytes,
                                 B, T, D, c, dt, ops._stream(x))
    _lib.check(rc, "rglru_fwd_carry")
    return y, h_last, prod, ws


def _reverse_carry(dy: Tensor, g_end: Optional[Tensor], x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Tensor,
                   tok: Optional[Tensor], ws: Tensor, c: float) -> Tensor:
    """dh0 of one slice from a carry-only ``rglru_bwd`` call (no gradient tensors are written)."""
    lib = _lib.load()
    dt = ops._io_dtype(x, "time-sharded backward")
    B, T, D = x.shape
    dh0 = torch.empty(B, D, device=x.device, dtype=torch.float32)
    with ops._on(x, "rglru_bwd"):
        rc = lib.rglru_bwd(ops._ptr(dy), ops._ptr(g_end), ops._ptr(x), ops._ptr(u_r), ops._ptr(u_i), ops._ptr(lam),
                           ops._ptr(h0), ops._ptr(tok), ops._ptr(ws), ws.numel(), None, None, None, None, ops._ptr(dh0),
                           B, T, D, c, dt, ops._stream(x))
    _lib.check(rc, "rglru_bwd (carry only)")
    return dh0


def _all_gather(t: Tensor, group) -> Tensor:
    """[world, *t.shape]: every rank's ``t`` (one collective; a group of one needs none)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return t.unsqueeze(0)
    out = torch.empty((world * t.shape[0],) + tuple(t.shape[1:]), device=t.device, dtype=t.dtype)   # concatenated form
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out.view((world,) + tuple(t.shape))


class _TimeShardedRGLRU(torch.autograd.Function):
    """One rank's slice of the time-sharded layer (gate pre-activations given)."""

    @staticmethod
    def forward(ctx, x, u_r, u_i, lam, h0, tok, c, group):
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        x, u_r, u_i = x.contiguous(), u_r.contiguous(), u_i.contiguous()
        lam32 = lam.to(torch.float32).contiguous()
        first = None if h0 is None else h0.to(torch.float32).contiguous()
        save = any(ctx.needs_input_grad)
        if world == 1:
            y, h_last, _, ws = _scan_with_carry(x, u_r, u_i, lam32, first, tok, c, save)
            h_in, prods = first, x.new_empty((1, 0), dtype=torch.float32)
        else:
            # pass 1, carry only, from a zero state (rank 0 from the sequence's own initial state)
            start = first if rank == 0 else None
            _, h_local, prod, _ = _scan_with_carry(x, u_r, u_i, lam32, start, tok, c, False, want_y=False)
            pairs = _all_gather(torch.stack((prod, h_local)), group)       # [world, 2, B, D]: one exchange
            prods, finals = pairs[:, 0], pairs[:, 1]
            # rank 0's pair already contains `first`, so the fold starts at rank 1's entry = finals[0]
            enter = fold_entering_states(prods[1:], finals[1:], finals[0])[0]
            h_in = start if rank == 0 else enter[rank - 1].contiguous()
            y, h_last, _, ws = _scan_with_carry(x, u_r, u_i, lam32, h_in, tok, c, save)   # pass 2: in full, from the true state
        ctx.save_for_backward(x, u_r, u_i, lam32, h_in, tok, ws, prods)
        ctx.c, ctx.group, ctx.has_h0 = c, group, h0 is not None
        ctx.lam_dtype = lam.dtype
        return y, h_last

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy, dh_last):
        import torch.distributed as dist
        x, u_r, u_i, lam32, h_in, tok, ws, prods = ctx.saved_tensors    # prods: every rank's decay product, from the forward
        group = ctx.group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        dy = torch.zeros_like(x) if dy is None else dy.to(x.dtype).contiguous()
        # the gradient on the returned final state belongs to the LAST slice's end (every rank returns its own
        # slice-final state; only the last rank's is the sequence's)
        g_end = None if dh_last is None else dh_last.to(torch.float32).contiguous()
        B, T, D = x.shape
        h0_arg = h_in if h_in is not None else torch.zeros(B, D, device=x.device, dtype=torch.float32)

        g_total = g_end
        if world > 1:
            # pass 1, carry only: what this slice hands to the one before it, given its own end gradient alone
            locals_ = _all_gather(_reverse_carry(dy, g_end, x, u_r, u_i, lam32, h0_arg, tok, ws, ctx.c), group)
            if rank < world - 1:
                # carry entering slice k from the slices after it: fold (P_j, dh0_local_j) for j = world-1 .. k+1; what
                # leaves that chain at slice k+1's start is the gradient of the state at slice k's end
                _, g_in = fold_entering_states(prods[rank + 1:], locals_[rank + 1:], None, reverse=True)
                g_total = (g_in if g_end is None else g_in + g_end).contiguous()
        # pass 2 (the only pass of a group of one): in full, with the true incoming carry
        dx, du_r, du_i, dlam, dh0 = ops._rglru_bwd_impl(dy, g_total, x, u_r, u_i, lam32, h0_arg, tok, ws, ctx.c, True)
        # dLambda is a parameter gradient: summed over ranks by the caller's data-parallel machinery or explicitly
        dh0_out = dh0 if (ctx.has_h0 and rank == 0) else (torch.zeros_like(dh0) if ctx.has_h0 else None)
        return dx, du_r, du_i, dlam.to(ctx.lam_dtype), dh0_out, None, None, None


def rglru_time_sharded(x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Optional[Tensor] = None,
                       tok: Optional[Tensor] = None, c: float = 8.0, group=None) -> tuple[Tensor, Tensor]:
    """This rank's time slice of RG-LRU(x | u_r, u_i): returns (y of the slice, state at the slice's end).

    Every rank of ``group`` calls it with its own slice (slices may differ in length); ``h0`` is the state
    entering the WHOLE sequence (used by rank 0).  Gradients: ``dx, du_r, du_i`` of the slice; ``dLambda`` is this
    rank's share and must be summed over the group like any data-parallel parameter gradient; the gradient of
    ``h0`` is produced on rank 0.  A gradient on the returned state is honoured on the last rank (the sequence's
    end) and, for intermediate ranks, treated as a gradient on that intermediate state.
    """
    if x.dim() != 3 or u_r.shape != x.shape or u_i.shape != x.shape:
        raise ValueError("x, u_r and u_i must share shape [batch, sequence, width]")
    if not x.is_cuda:
        raise RuntimeError("CUDA RG-LRU kernels require CUDA tensors (there is no CPU path)")
    import torch.distributed as dist
    if not dist.is_initialized():
        raise RuntimeError("rglru_time_sharded needs an initialised torch.distributed process group")
    return _TimeShardedRGLRU.apply(x, u_r, u_i, lam, h0, None if tok is None else tok.contiguous(), float(c), group)


def run_slices_on_one_device(slices: Sequence[tuple[Tensor, Tensor, Tensor]], lam: Tensor, h0: Optional[Tensor] = None,
                             c: float = 8.0) -> tuple[list[Tensor], Tensor]:
    """The same three phases with the "ranks" played one after another on ONE device (forward only): a check of
    the carry algebra against an unsplit call, and a way to push a sequence through in pieces when its slices do
    not fit in memory together.  Returns the per-slice outputs and the final state."""
    lam32 = lam.to(torch.float32).contiguous()
    first = None if h0 is None else h0.to(torch.float32).contiguous()
    prods, finals = [], []
    for k, (x, u_r, u_i) in enumerate(slices):
        _, h_last, prod, _ = _scan_with_carry(x.contiguous(), u_r.contiguous(), u_i.contiguous(), lam32,
                                              first if k == 0 else None, None, c, False, want_y=False)
        prods.append(prod)
        finals.append(h_last)
    enter = [first] + (fold_entering_states(prods[1:], finals[1:], finals[0])[0] if len(slices) > 1 else [])
    outs, last = [], None
    for k, (x, u_r, u_i) in enumerate(slices):
        y, last, _, _ = _scan_with_carry(x.contiguous(), u_r.contiguous(), u_i.contiguous(), lam32, enter[k], None, c, False)
        outs.append(y)
    return outs, last
