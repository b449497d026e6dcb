"""Host-side mirror of the reference's RG-LRU modules, backed only by the CUDA kernels.

``RG_LRU``, ``RecurrentBlock``, ``BlockDiagonalLinear`` and ``RecurrentBlockCache``
keep the constructor arguments, forward signatures, parameter names/shapes and
error behaviour of the reference (griffin/griffin.py:26-33, 129-154, 157-306,
361-529) so reference checkpoints load unchanged.  The one difference is the
scan backend: ``scan_mode="cuda"`` (also what ``"auto"`` resolves to here) runs
the hand-written sm_100a kernels; the reference's "sequential", "associative" and
"fused" (Triton) backends are not part of this package and are rejected, and
there is no CPU fallback -- a CPU tensor raises ``RuntimeError``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Literal, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import _lib, ops

ScanMode = Literal["auto", "cuda"]
_REFERENCE_ONLY_MODES = ("sequential", "associative", "fused")


def _check_scan_mode(scan_mode: str) -> str:
    if scan_mode in ("auto", "cuda"):
        return "cuda"
    if scan_mode in _REFERENCE_ONLY_MODES:
        raise ValueError(
            f"scan_mode={scan_mode!r} is a backend of the reference implementation; this package provides only "
            "scan_mode='cuda' (the sm_100a kernels)")
    raise ValueError(f"Unknown RG-LRU scan mode: {scan_mode}")


@dataclass
class RecurrentBlockCache:
    """State needed to continue a recurrent block on a later chunk (griffin/griffin.py:26-33)."""

    rnn_state: Tensor          # [B, D] fp32
    conv_state: Tensor         # [B, 3, D] activation dtype
    segment_position: Tensor   # [B] int64, position of the last real token


def _largest_block_count(width: int, requested: int) -> int:
    if width <= 0 or requested <= 0:
        raise ValueError("width and requested_blocks must be positive")
    count = min(width, requested)
    while width % count:
        count -= 1
    return count


class BlockDiagonalLinear(nn.Module):
    """Gate projection with independent diagonal blocks (griffin/griffin.py:129-154).

    Stays an ordinary batched GEMM; only its output feeds the CUDA kernels.
    ``weight`` is [blocks, out, in], ``bias`` [blocks, out].
    """

    def __init__(self, width: int, num_blocks: int = 16):
        super().__init__()
        self.width = width
        self.num_blocks = _largest_block_count(width, num_blocks)
        self.block_width = width // self.num_blocks
        self.weight = nn.Parameter(torch.empty(self.num_blocks, self.block_width, self.block_width))
        self.bias = nn.Parameter(torch.empty(self.num_blocks, self.block_width))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0.0, std=math.sqrt(1.0 / self.block_width))
        nn.init.zeros_(self.bias)

    def forward(self, x: Tensor) -> Tensor:
        lead = x.shape[:-1]
        rows = x.reshape(-1, self.num_blocks, self.block_width).transpose(0, 1)   # [G, N, in]
        out = torch.baddbmm(self.bias[:, None, :], rows, self.weight.transpose(1, 2))  # [G, N, out]
        return out.transpose(0, 1).reshape(*lead, self.width)


def token_flags(batch: int, steps: int, device, *, reset: Optional[Tensor] = None, active: Optional[Tensor] = None,
                segment_pos: Optional[Tensor] = None, padded: Optional[Tensor] = None) -> Optional[Tensor]:
    """Pack the per-token masks into the flag byte the kernels read ([B, T] uint8), or None if all are absent."""
    if reset is None and active is None and segment_pos is None:
        return None
    flags = torch.zeros(batch, steps, device=device, dtype=torch.uint8)
    if segment_pos is not None:
        cut = (3 - segment_pos.clamp(min=0, max=3)).to(torch.uint8)
        flags = flags | cut
    if reset is not None:
        flags = flags | (reset.to(torch.uint8) * _lib.TOK_RESET)
    if active is not None:
        flags = flags | ((~active).to(torch.uint8) * _lib.TOK_INACTIVE)
    if padded is not None and segment_pos is not None and active is not None:
        wipe = (segment_pos == 0) & active & padded
        flags = flags | (wipe.to(torch.uint8) * _lib.TOK_ZERO_HISTORY)
    return flags


_PLAIN_FLAGS: dict = {}


def _build_plain_flags(batch: int, steps: int, device) -> Tensor:
    flags = torch.zeros(batch, steps, device=device, dtype=torch.uint8)
    flags[:, 0] = 3 | _lib.TOK_RESET
    if steps > 1:
        flags[:, 1] = 2
    if steps > 2:
        flags[:, 2] = 1
    return flags


def _plain_flags(batch: int, steps: int, device) -> Tensor:
    """Flag bytes of rows that are one fresh document each (positions 0..T-1): a reset at token 0 and the first
    three tokens short of taps.  Built with device-side fills only (no host copy, so the block can be captured
    into a CUDA graph), once per (batch, steps, device), and shared read-only between calls.

    The shared tensor must be usable from any later context, so it is created as an ordinary tensor even when
    the first caller runs under ``torch.inference_mode`` (an inference tensor could not be saved for a later
    backward), the creating stream is drained once so that other streams may read it, and nothing is cached
    while a CUDA graph is being captured (a tensor born in a capture belongs to the graph's memory pool and
    holds data only after a replay): such calls get a tensor of their own."""
    if ops._library_ops_active():      # being traced (torch.compile, fake tensors): plain ops, no cache, no CUDA runtime calls
        return _build_plain_flags(batch, steps, device)
    device = torch.device(device)
    capturing = device.type == "cuda" and torch.cuda.is_current_stream_capturing()
    key = (batch, steps, str(device))
    flags = None if capturing else _PLAIN_FLAGS.get(key)
    if flags is None:
        with torch.inference_mode(False):
            flags = _build_plain_flags(batch, steps, device)
        if capturing:
            return flags
        if device.type == "cuda":
            torch.cuda.current_stream(device).synchronize()
        if len(_PLAIN_FLAGS) > 64:
            _PLAIN_FLAGS.clear()
        _PLAIN_FLAGS[key] = flags
    return flags


class RG_LRU(nn.Module):
    """Real-gated linear recurrent unit on the CUDA kernels (reference: griffin/griffin.py:157-306)."""

    def __init__(self, rnn_width: int, c: float = 8.0, gate_blocks: int = 16, scan_mode: str = "cuda", *,
                 group_gates: bool = True):
        super().__init__()
        # group_gates (not in the reference): where the shape allows, both gate projections run as one grouped
        # GEMM whose output the kernels read in place (same arithmetic, fewer passes over memory).
        self.group_gates = group_gates
        self.rnn_width = rnn_width
        self.c = c
        self.scan_mode = _check_scan_mode(scan_mode)
        self.recurrence_gate = BlockDiagonalLinear(rnn_width, gate_blocks)
        self.input_gate = BlockDiagonalLinear(rnn_width, gate_blocks)
        self.Lambda = nn.Parameter(torch.empty(rnn_width))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """sigmoid(Lambda)^c uniform in [0.9, 0.999] (griffin/griffin.py:179-188)."""
        self.recurrence_gate.reset_parameters()
        self.input_gate.reset_parameters()
        with torch.no_grad():
            target = torch.empty_like(self.Lambda).uniform_(0.9, 0.999)
            self.Lambda.copy_(torch.logit(target.pow(1.0 / self.c)))

    def forward(self, xt: Tensor, ht_minus_1: Optional[Tensor] = None, *, reset_mask: Optional[Tensor] = None,
                active_mask: Optional[Tensor] = None, return_state: bool = False, _flags: Optional[Tensor] = None,
                _branch: Optional[Tensor] = None):
        if xt.dim() != 3:
            raise ValueError(f"RG_LRU expects [batch, sequence, width], got {tuple(xt.shape)}")
        batch, steps, width = xt.shape
        if width != self.rnn_width:
            raise ValueError(f"Expected width {self.rnn_width}, got {width}")
        if reset_mask is not None:
            if reset_mask.shape != (batch, steps):
                raise ValueError(f"reset_mask must have shape ({batch}, {steps}), got {tuple(reset_mask.shape)}")
            reset_mask = reset_mask.to(device=xt.device, dtype=torch.bool)
        if active_mask is not None:
            if active_mask.shape != (batch, steps):
                raise ValueError(f"active_mask must have shape ({batch}, {steps}), got {tuple(active_mask.shape)}")
            active_mask = active_mask.to(device=xt.device, dtype=torch.bool)
        if ht_minus_1 is not None:
            if ht_minus_1.shape != (batch, width):
                raise ValueError(f"ht_minus_1 must have shape ({batch}, {width}), got {tuple(ht_minus_1.shape)}")
            ht_minus_1 = ht_minus_1.to(device=xt.device, dtype=torch.float32)
        if not xt.is_cuda:
            raise RuntimeError("scan_mode='cuda' requires CUDA tensors; there is no CPU fallback")
        if xt.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"scan_mode='cuda' supports float32 and bfloat16 activations, got {xt.dtype}")

        flags = _flags if _flags is not None else token_flags(batch, steps, xt.device, reset=reset_mask, active=active_mask)
        if self.group_gates and ops.grouped_gates_supported(xt, self.recurrence_gate.block_width):
            yt, h_last = ops.rglru_grouped(xt, self.recurrence_gate.weight, self.recurrence_gate.bias,
                                           self.input_gate.weight, self.input_gate.bias, self.Lambda, ht_minus_1, flags,
                                           self.c, _branch)
            return (yt, h_last) if return_state else yt
        u_r = self.recurrence_gate(xt).to(xt.dtype)
        u_i = self.input_gate(xt).to(xt.dtype)
        if _branch is not None:   # the caller's GeLU branch, multiplied in by the kernels
            yt, h_last = ops.rglru_merged(xt, u_r, u_i, _branch, self.Lambda, ht_minus_1, flags, self.c)
        else:
            yt, h_last = ops.rglru(xt, u_r, u_i, self.Lambda, ht_minus_1, flags, self.c)
        if return_state:
            return yt, h_last
        return yt


def _positions(x: Tensor, segment_pos: Optional[Tensor], previous: Optional[Tensor], active: Optional[Tensor]) -> Tensor:
    """Per-token position inside its document (behaviour of griffin/griffin.py:309-338)."""
    batch, steps = x.shape[:2]
    if steps == 0:
        raise ValueError("Empty token sequences are not supported")
    if segment_pos is not None:
        if segment_pos.shape != (batch, steps):
            raise ValueError(f"segment_pos must have shape ({batch}, {steps}), got {tuple(segment_pos.shape)}")
        return segment_pos.to(device=x.device, dtype=torch.long)
    if previous is None:
        start = torch.full((batch, 1), -1, device=x.device, dtype=torch.long)
    else:
        if previous.shape != (batch,):
            raise ValueError("Cached segment positions have an incompatible shape")
        start = previous.to(device=x.device, dtype=torch.long)[:, None]
    if active is None:
        return start + torch.arange(1, steps + 1, device=x.device, dtype=torch.long)[None, :]
    return start + active.to(torch.long).cumsum(dim=1)


def _last_real_position(segment_pos: Tensor, active: Optional[Tensor], previous: Optional[Tensor]) -> Tensor:
    """Position of each row's last non-padding token, without a host loop (griffin/griffin.py:341-358)."""
    batch, steps = segment_pos.shape
    if active is None:
        return segment_pos[:, -1].clone()
    index = torch.arange(1, steps + 1, device=segment_pos.device)[None, :] * active.to(torch.long)
    last = index.max(dim=1).values                       # 0 when the row is all padding
    picked = segment_pos.gather(1, (last - 1).clamp(min=0)[:, None])[:, 0]
    if previous is None:
        fallback = torch.full((batch,), -1, device=segment_pos.device, dtype=torch.long)
    else:
        fallback = previous.to(device=segment_pos.device, dtype=torch.long)
    return torch.where(last > 0, picked, fallback)


def _stable_partition(active: Tensor) -> tuple[Tensor, Tensor]:
    """Indices that move every row's real tokens to the front, order kept (and the padding behind them, order kept):
    ``order[b, j]`` is the token that lands at place j, ``restore[b, t]`` the place token t lands at.  Two running
    counts and one scatter instead of two sorts: a real token's place is the number of real tokens before it, a
    padding token's the row's real count plus the padding before it."""
    real = active.to(torch.long)
    before_real = real.cumsum(dim=1) - real                    # real tokens strictly before t
    pad = 1 - real
    before_pad = pad.cumsum(dim=1) - pad
    restore = torch.where(active, before_real, real.sum(dim=1, keepdim=True) + before_pad)
    steps = torch.arange(active.shape[1], device=active.device, dtype=torch.long).expand_as(restore)
    order = torch.empty_like(restore).scatter_(1, restore, steps)
    return order, restore


def _flat_rows(index: Tensor) -> Tensor:
    """Per-row sequence indices [B, T] as indices into the flattened [B * T] tokens."""
    batch, steps = index.shape
    return (index + torch.arange(batch, device=index.device, dtype=index.dtype)[:, None] * steps).reshape(-1)


class _PermuteRows(torch.autograd.Function):
    """Move whole tokens of a [B, T, D] tensor by a permutation of every row, given as flat token indices
    (``_flat_rows``) together with those of the inverse permutation: one index per token (``index_select`` on the
    flattened tokens, not an index per element), and a backward that is the same move with the inverse permutation,
    not the atomic scatter-add autograd would use for a gather."""

    @staticmethod
    def forward(ctx, x, flat_index, flat_inverse):
        ctx.save_for_backward(flat_inverse)
        return x.reshape(flat_index.numel(), -1).index_select(0, flat_index).view(x.shape)

    @staticmethod
    def backward(ctx, grad):
        (flat_inverse,) = ctx.saved_tensors
        return grad.reshape(flat_inverse.numel(), -1).index_select(0, flat_inverse).view(grad.shape), None, None


def _memo_stamp(t: Tensor):
    """(weak reference, version) identifying a tensor object in its present state, or None where that cannot be had
    (inference tensors track no version; some subclasses take no weak references): then nothing is remembered."""
    import weakref
    try:
        return weakref.ref(t), t._version
    except (RuntimeError, TypeError):
        return None


def _memo_hit(stamp, t: Tensor) -> bool:
    try:
        return stamp[0]() is t and stamp[1] == t._version
    except RuntimeError:
        return False


_PADDING_KIND: dict = {}     # id(mask tensor) -> ((weak reference, version), answer)


def _needs_partition(active: Tensor, owner: Tensor) -> bool:
    """Whether some row has a real token after padding (anything but right padding).  The answer costs a
    device-to-host read, so it is remembered per mask OBJECT (``owner``: the tensor the caller passed, of which
    ``active`` is the boolean copy on the right device) and version: a model hands the same mask tensor to every one
    of its blocks, and only the first of them waits for the device."""
    key = id(owner)
    hit = _PADDING_KIND.get(key)
    if hit is not None and _memo_hit(hit[0], owner):
        return hit[1]
    answer = bool((active[:, 1:] & ~active[:, :-1]).any())
    stamp = _memo_stamp(owner)
    if stamp is not None:
        if len(_PADDING_KIND) > 64:
            _PADDING_KIND.clear()
        _PADDING_KIND[key] = (stamp, answer)
    return answer


_MASK_PLANS: dict = {}


def _shared_between_blocks(owners: tuple, device, build):
    """``build()``, remembered per (owner tensor OBJECTS, their versions, device).  A model hands the same
    ``segment_pos`` / ``active_mask`` tensors to every one of its recurrent blocks, and what a block derives from them
    (positions, flag bytes, the row partition) is the same for all: the first block builds it, the others take it.
    Nothing is remembered while tracing, under ``torch.inference_mode`` (an inference tensor could not be saved for
    a later backward) or while a CUDA graph is being captured (a tensor born in a capture holds data only after a
    replay).  The shared tensors are read-only and live on the stream that built them, like the inputs they come
    from."""
    live = tuple(o for o in owners if o is not None)
    if (not live or ops._library_ops_active() or torch.is_inference_mode_enabled()
            or (device.type == "cuda" and torch.cuda.is_current_stream_capturing())):
        return build()
    key = tuple(0 if o is None else id(o) for o in owners) + (str(device),)
    hit = _MASK_PLANS.get(key)
    if hit is not None and all(_memo_hit(stamp, o) for stamp, o in zip(hit[0], live)):
        return hit[1]
    value = build()
    stamps = tuple(_memo_stamp(o) for o in live)
    if all(stamp is not None for stamp in stamps):
        if len(_MASK_PLANS) > 16:
            _MASK_PLANS.clear()
        _MASK_PLANS[key] = (stamps, value)
    return value


def _project(layer: nn.Module, x: Tensor) -> Tensor:
    """One of the block's three projections.  A stock ``nn.Linear`` without hooks goes through ``ops.linear`` (same
    GEMMs; the bias gradient comes from the library's column-sum kernel); anything else — a replaced layer, a layer
    with hooks — is called as the module it is."""
    if type(layer) is nn.Linear and not (layer._forward_hooks or layer._forward_pre_hooks or layer._backward_hooks
                                         or layer._backward_pre_hooks):
        return ops.linear(x, layer.weight, layer.bias)
    return layer(x)


class RecurrentBlock(nn.Module):
    """Causal conv + RG-LRU temporal-mixing block with cached decoding (griffin/griffin.py:361-529).

    The two input projections, the GeLU branch and the output projection are ordinary
    torch GEMMs; the conv, the RG-LRU and the single-token decode run on the CUDA kernels.
    The kernels take padding (``active_mask``) as right padding; any other mask (left padding, holes) is
    handled by moving each row's real tokens to the front for the conv and the scan and moving the results
    back, which is exactly the reference's rule that padding neither enters the conv history nor moves the
    state (griffin/griffin.py:488-510).
    """

    def __init__(self, input_dim: int, rnn_width: int, conv_kernel_size: int = 4, gate_blocks: int = 16,
                 final_w_init_variance_scale: float = 1.0, scan_mode: str = "cuda", *, fold_conv: bool = False,
                 fold_merge: bool = False):
        super().__init__()
        # fold_merge (not in the reference): the product with the GeLU branch is formed in the scan kernels' store
        # stage and differentiated in the backward kernel's load stage; combines with fold_conv.
        self.fold_merge = fold_merge
        # fold_conv (not in the reference): run conv, gates and scan as one autograd node whose scan kernels
        # apply the conv while loading, so the conv output is not kept for backward (recomputed there instead).
        self.fold_conv = fold_conv
        if conv_kernel_size <= 0:
            raise ValueError("conv_kernel_size must be positive")
        if conv_kernel_size != 4:
            raise ValueError("scan_mode='cuda' implements the temporal convolution for conv_kernel_size=4 only")
        self.rnn_width = rnn_width
        self.conv_kernel_size = conv_kernel_size
        self.linear_x = nn.Linear(input_dim, rnn_width)
        self.linear_y = nn.Linear(input_dim, rnn_width)
        self.temporal_conv = nn.Conv1d(rnn_width, rnn_width, kernel_size=conv_kernel_size, padding=0, groups=rnn_width)
        self.rg_lru = RG_LRU(rnn_width, gate_blocks=gate_blocks, scan_mode=scan_mode)
        self.linear_out = nn.Linear(rnn_width, input_dim)
        self.final_w_init_variance_scale = final_w_init_variance_scale
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Initialisation of griffin/griffin.py:393-407."""
        nn.init.normal_(self.linear_x.weight, std=math.sqrt(1.0 / self.linear_x.in_features))
        nn.init.normal_(self.linear_y.weight, std=math.sqrt(1.0 / self.linear_y.in_features))
        nn.init.normal_(self.linear_out.weight, std=math.sqrt(self.final_w_init_variance_scale / self.linear_out.in_features))
        nn.init.normal_(self.temporal_conv.weight, std=math.sqrt(0.01 / self.conv_kernel_size))
        for bias in (self.linear_x.bias, self.linear_y.bias, self.linear_out.bias, self.temporal_conv.bias):
            nn.init.zeros_(bias)

    def forward(self, x: Tensor, cache: Optional[RecurrentBlockCache] = None, segment_pos: Optional[Tensor] = None, *,
                active_mask: Optional[Tensor] = None, return_cache: bool = False):
        if x.dim() != 3:
            raise ValueError(f"RecurrentBlock expects [batch, sequence, width], got {tuple(x.shape)}")
        batch, steps = x.shape[:2]
        caller_mask = active_mask        # the caller's own tensor object: what the padding-kind memo is keyed on
        if active_mask is not None:
            if active_mask.shape != (batch, steps):
                raise ValueError("active_mask must match the input [batch, sequence] dimensions")
            active_mask = active_mask.to(device=x.device, dtype=torch.bool)
        previous = None if cache is None else cache.segment_position
        plain = segment_pos is None and cache is None and active_mask is None
        if plain and steps == 0:
            raise ValueError("Empty token sequences are not supported")
        caller_pos = segment_pos
        device = x.device

        def mask_plan():
            """(positions, flag bytes, flat indices of the row partition or None) for this call's masks."""
            # rows that are one fresh document each need no position tensor unless a cache is asked for
            pos = None if plain and not return_cache else _positions(x, segment_pos, previous, active_mask)
            if plain:
                # contiguous positions 0..T-1: only the first three tokens lose taps, token 0 is a reset
                return pos, _plain_flags(batch, steps, device), None
            moves = None
            kernel_pos, kernel_active = pos, active_mask
            if active_mask is not None and steps > 1 and _needs_partition(active_mask, caller_mask):
                # a real token follows padding somewhere: stable partition of every row, real tokens first
                order, restore = _stable_partition(active_mask)
                moves = (_flat_rows(order), _flat_rows(restore))
                kernel_pos, kernel_active = pos.gather(1, order), active_mask.gather(1, order)
            padded = None if kernel_active is None else ~kernel_active.all()
            flags = token_flags(batch, steps, device, reset=kernel_pos == 0, active=kernel_active,
                                segment_pos=kernel_pos, padded=padded)
            return pos, flags, moves

        if plain or cache is not None:      # (the plain flags have a memo of their own; a cache differs per block)
            pos, flags, moves = mask_plan()
        else:
            pos, flags, moves = _shared_between_blocks((caller_pos, caller_mask), device, mask_plan)

        y_branch = _project(self.linear_y, x)
        if not self.fold_merge:
            y_branch = F.gelu(y_branch, approximate="tanh")
        x_in = _project(self.linear_x, x)
        if moves is not None:
            x_in = _PermuteRows.apply(x_in, moves[0], moves[1])
            if self.fold_merge:   # the kernels multiply by the branch, so it travels with its tokens
                y_branch = _PermuteRows.apply(y_branch, moves[0], moves[1])
        conv_state = None if cache is None else cache.conv_state
        if conv_state is not None and conv_state.shape != (batch, self.conv_kernel_size - 1, self.rnn_width):
            raise ValueError("Recurrent convolution cache has an incompatible shape")

        conv_w = self.temporal_conv.weight[:, 0, :]
        rnn_state = None if cache is None else cache.rnn_state
        if steps == 1 and cache is not None and not torch.is_grad_enabled() and x_in.is_cuda:
            # Cached single-token decode (inference): the two in-place decode kernels on copies of the cached
            # states (the cache stays a value: the caller's old cache is not modified).
            if rnn_state.shape != (batch, self.rnn_width):
                raise ValueError(f"ht_minus_1 must have shape ({batch}, {self.rnn_width}), got {tuple(rnn_state.shape)}")
            lru = self.rg_lru
            tok = flags[:, 0].contiguous()
            new_conv = conv_state.to(x_in.dtype).clone()
            bias = self.temporal_conv.bias
            x_conv = ops.decode_conv(x_in[:, 0].contiguous(), conv_w.float().contiguous(),
                                     None if bias is None else bias.float().contiguous(), new_conv, tok)
            u_r = lru.recurrence_gate(x_conv).to(x_conv.dtype)
            u_i = lru.input_gate(x_conv).to(x_conv.dtype)
            new_rnn = rnn_state.to(device=x_in.device, dtype=torch.float32).clone()
            y = ops.decode_step(x_conv, u_r, u_i, lru.Lambda.float().contiguous(), new_rnn, tok, lru.c)[:, None, :]
            if self.fold_merge:
                y = y * F.gelu(y_branch, approximate="tanh")
        elif self.fold_conv:
            if not x_in.is_cuda:
                raise RuntimeError("scan_mode='cuda' requires CUDA tensors; there is no CPU fallback")
            if rnn_state is not None and rnn_state.shape != (batch, self.rnn_width):
                raise ValueError(f"ht_minus_1 must have shape ({batch}, {self.rnn_width}), got {tuple(rnn_state.shape)}")
            lru = self.rg_lru
            y, new_rnn, new_conv = ops.recurrent_core(
                x_in, conv_w, self.temporal_conv.bias, conv_state, lru.recurrence_gate.weight, lru.recurrence_gate.bias,
                lru.input_gate.weight, lru.input_gate.bias, lru.Lambda, rnn_state, flags, lru.c,
                y_branch if self.fold_merge else None)
        else:
            x_conv, new_conv = ops.causal_conv(x_in, conv_w, self.temporal_conv.bias, conv_state, flags,
                                               want_state=return_cache)
            y, new_rnn = self.rg_lru(x_conv, rnn_state, return_state=True, _flags=flags,
                                     _branch=y_branch if self.fold_merge else None)
        if moves is not None:
            y = _PermuteRows.apply(y, moves[1], moves[0])
        out = _project(self.linear_out, y if self.fold_merge else y * y_branch)
        if active_mask is not None:
            out = torch.where(active_mask[..., None], out, 0.0)     # (a scalar: no tensor of zeros to write and read)
        if return_cache:
            return out, RecurrentBlockCache(new_rnn, new_conv, _last_real_position(pos, active_mask, previous))
        return out
