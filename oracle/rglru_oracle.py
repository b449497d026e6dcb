"""CPU oracle for the RG-LRU hot path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This file restates, in plain CPU torch, the arithmetic that the reference
(peytontolbert/Griffin) performs on the path that the CUDA kernels replace.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it; the shipped package never does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the unmodified
reference (``scan_mode="sequential"``) on seeded inputs and stores its outputs
and gradients; ``tests/test_oracle_golden.py`` checks every function below
against those vectors.

Each function names the reference lines it follows (paths are relative to the
reference project root).

Two families live here:

* autograd-based functions (``rglru_layer``, ``recurrent_block``) that use the
  same torch primitives as the reference, so their gradients are produced by
  the same mechanism the reference relies on (including its O(T^2) backward
  cost on CPU, which is what the CPU baseline times);
* ``rglru_backward_linear``: a hand-derived O(T) reverse pass used where the
  autograd route is too slow or too large (long sequences), itself validated
  against the autograd route at small sizes.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor

SQRT_SLOPE_CAP = 1000.0  # griffin/griffin.py:51


class _CappedSlopeSqrt(torch.autograd.Function):
    """sqrt(v) whose derivative is limited to SQRT_SLOPE_CAP.

    Follows griffin/griffin.py:48-65 (``_SqrtBoundDerivative``): forward is the
    exact square root; backward divides by sqrt(max(4 v, 1/cap^2)).
    """

    @staticmethod
    def forward(ctx, v: Tensor) -> Tensor:
        ctx.save_for_backward(v)
        return v.sqrt()

    @staticmethod
    def backward(ctx, grad: Tensor):
        (v,) = ctx.saved_tensors
        floor = 1.0 / (SQRT_SLOPE_CAP * SQRT_SLOPE_CAP)
        return (grad / (4.0 * v).clamp(min=floor).sqrt(),)


def capped_sqrt(v: Tensor) -> Tensor:
    return _CappedSlopeSqrt.apply(v)


def block_diagonal_linear(x: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
    """Gate pre-activation: G independent (bw x bw) maps over the last axis.

    griffin/griffin.py:149-154.  ``weight`` is [G, out, in], ``bias`` [G, out].
    """
    groups, width_out, width_in = weight.shape
    lead = x.shape[:-1]
    parts = x.reshape(*lead, groups, width_in)
    mapped = torch.einsum("...gi,goi->...go", parts, weight) + bias
    return mapped.reshape(*lead, groups * width_out)


def gate_epilogue(
    x: Tensor,
    u_r: Tensor,
    u_i: Tensor,
    lam: Tensor,
    c: float,
    reset: Tensor | None,
    active: Tensor | None,
) -> tuple[Tensor, Tensor]:
    """Decay ``a`` and driven input ``b`` of the recurrence, in ``x``'s dtype.

    griffin/griffin.py:237-255.  ``u_r``/``u_i`` are the gate pre-activations.
    """
    r = torch.sigmoid(u_r)
    i = torch.sigmoid(u_i)
    log_base = F.logsigmoid(lam).to(x.dtype)  # :239
    log_a = c * r * log_base  # :240
    a = torch.exp(log_a)  # :241
    gamma_sq = torch.clamp(-torch.expm1(2.0 * log_a), min=0.0)  # :244
    gamma = capped_sqrt(gamma_sq)  # :245
    if reset is not None:
        rm = reset[..., None]
        a = torch.where(rm, torch.zeros_like(a), a)  # :248
        gamma = torch.where(rm, torch.ones_like(gamma), gamma)  # :249
    b = gamma * i * x  # :250
    if active is not None:
        am = active[..., None]
        a = torch.where(am, a, torch.ones_like(a))  # :252
        b = torch.where(am, b, torch.zeros_like(b))  # :253-255
    return a, b


def state_dtype(io_dtype: torch.dtype) -> torch.dtype:
    """fp32 state for half-precision I/O, otherwise the I/O type (griffin.py:226)."""
    return torch.float32 if io_dtype in (torch.float16, torch.bfloat16) else io_dtype


def sequential_scan(a: Tensor, b: Tensor, h0: Tensor) -> tuple[Tensor, Tensor]:
    """h_t = a_t * h_{t-1} + b_t walked in time order (griffin/griffin.py:280-284).

    Returns the stacked states [B, T, D] and the last state [B, D].
    """
    h = h0
    steps = []
    for t in range(a.shape[1]):
        h = a[:, t] * h + b[:, t]
        steps.append(h)
    return torch.stack(steps, dim=1), h


def rglru_core(
    x: Tensor,
    u_r: Tensor,
    u_i: Tensor,
    lam: Tensor,
    h0: Tensor | None = None,
    reset: Tensor | None = None,
    active: Tensor | None = None,
    c: float = 8.0,
) -> tuple[Tensor, Tensor]:
    """Gate epilogue + sequential scan given the gate pre-activations.

    This is the part of ``RG_LRU.forward`` that the CUDA forward kernel
    computes (griffin/griffin.py:226-235 state set-up, :237-258 epilogue,
    :280-286 scan and cast back).  Returns ``(y in x.dtype, h_last in state dtype)``.
    """
    acc = state_dtype(x.dtype)
    batch, _, width = x.shape
    if h0 is None:
        h0 = torch.zeros(batch, width, dtype=acc)
    else:
        h0 = h0.to(acc)
    a, b = gate_epilogue(x, u_r, u_i, lam, c, reset, active)
    states, last = sequential_scan(a.to(acc), b.to(acc), h0)
    return states.to(x.dtype), last


def rglru_layer(
    x: Tensor,
    params: dict[str, Tensor],
    h0: Tensor | None = None,
    reset: Tensor | None = None,
    active: Tensor | None = None,
    c: float = 8.0,
) -> tuple[Tensor, Tensor]:
    """Whole ``RG_LRU.forward`` including the two gate projections.

    ``params`` uses the reference's state-dict names: ``Lambda``,
    ``recurrence_gate.weight/bias``, ``input_gate.weight/bias``
    (griffin/griffin.py:174-176).
    """
    u_r = block_diagonal_linear(x, params["recurrence_gate.weight"], params["recurrence_gate.bias"])
    u_i = block_diagonal_linear(x, params["input_gate.weight"], params["input_gate.bias"])
    return rglru_core(x, u_r, u_i, params["Lambda"], h0, reset, active, c)


def rglru_backward_linear(
    x: Tensor,
    u_r: Tensor,
    u_i: Tensor,
    lam: Tensor,
    dy: Tensor,
    h0: Tensor | None = None,
    dh_last: Tensor | None = None,
    reset: Tensor | None = None,
    active: Tensor | None = None,
    c: float = 8.0,
) -> dict[str, Tensor]:
    """O(T) reverse pass of ``rglru_core`` written out by hand.

    The reference has no explicit backward for the fused gate epilogue (it
    relies on autograd over griffin/griffin.py:237-286 plus the capped slope of
    :59-65); this is the closed form of that autograd graph.  With
    g_t = dy_t + a_{t+1} g_{t+1} (g_{T-1} also receives dh_last):

      db_t = g_t,  da_t = g_t h_{t-1}            (zero where inactive; da also zero at reset)
      dx   = db * gamma * i                      (direct path only, gates excluded)
      du_i = db * gamma * x * i (1 - i)
      dgam = db * i * x  (zero at reset);  dgam2 = dgam / sqrt(max(4 gamma^2, 1e-6))
      dl   = da * a_raw - 2 a_raw^2 dgam2        (a_raw = exp(l), before masking)
      du_r = dl * c * logsigmoid(Lambda) * r (1 - r)
      dLambda = sigmoid(-Lambda) * c * sum_{b,t} dl * r
      dh0  = a_0 g_0

    All arithmetic is carried out in ``x.dtype`` promoted to at least fp32.
    Returns dx (direct), du_r, du_i, dLambda, dh0, plus y and h_last.
    """
    work = torch.float64 if x.dtype == torch.float64 else torch.float32
    xf, urf, uif, dyf = (t.to(work) for t in (x, u_r, u_i, dy))
    lamf = lam.to(work)
    batch, steps, width = xf.shape
    r = torch.sigmoid(urf)
    i = torch.sigmoid(uif)
    log_base = F.logsigmoid(lamf)
    log_a = c * r * log_base
    a_raw = torch.exp(log_a)
    gamma_sq = torch.clamp(-torch.expm1(2.0 * log_a), min=0.0)
    gamma = gamma_sq.sqrt()
    keep = torch.ones(batch, steps, 1, dtype=work)
    live = torch.ones(batch, steps, 1, dtype=work)
    a = a_raw
    gam = gamma
    if reset is not None:
        rm = reset[..., None]
        a = torch.where(rm, torch.zeros_like(a), a)
        gam = torch.where(rm, torch.ones_like(gam), gam)
        keep = (~rm).to(work)
    b = gam * i * xf
    if active is not None:
        am = active[..., None]
        a = torch.where(am, a, torch.ones_like(a))
        b = torch.where(am, b, torch.zeros_like(b))
        live = am.to(work)

    h = torch.zeros(batch, width, dtype=work) if h0 is None else h0.to(work)
    h_prev = torch.empty(batch, steps, width, dtype=work)
    y = torch.empty(batch, steps, width, dtype=work)
    for t in range(steps):
        h_prev[:, t] = h
        h = a[:, t] * h + b[:, t]
        y[:, t] = h
    h_last = h

    g = torch.zeros(batch, width, dtype=work) if dh_last is None else dh_last.to(work).clone()
    db = torch.empty_like(y)
    for t in range(steps - 1, -1, -1):
        g = g + dyf[:, t]
        db[:, t] = g
        g = g * a[:, t]
    dh0 = g

    da = db * h_prev * live * keep
    db = db * live
    dx = db * gam * i
    du_i = db * gam * xf * i * (1.0 - i)
    dgam = db * i * xf * keep
    floor = 1.0 / (SQRT_SLOPE_CAP * SQRT_SLOPE_CAP)
    dgam_sq = dgam / torch.sqrt(torch.clamp(4.0 * gamma_sq, min=floor))
    dlog = da * a_raw - 2.0 * a_raw * a_raw * dgam_sq
    du_r = dlog * (c * log_base) * r * (1.0 - r)
    dlam = torch.sigmoid(-lamf) * c * (dlog * r).sum(dim=(0, 1))
    return {
        "y": y,
        "h_last": h_last,
        "dx": dx,
        "du_r": du_r,
        "du_i": du_i,
        "dLambda": dlam,
        "dh0": dh0,
    }


class _CoreLinearBackward(torch.autograd.Function):
    """``rglru_core`` as one autograd node whose backward is ``rglru_backward_linear``.

    Same forward values as the sequential loop of griffin/griffin.py:280-286 (fp32 state for half-precision
    I/O); the gradient is the hand-derived O(T) reverse pass instead of autograd's O(T^2) one, so that whole
    blocks can be differentiated at sequence lengths in the thousands.  The closed form is itself held to
    the reference's autograd results by tests/test_oracle_golden.py.
    """

    @staticmethod
    def forward(ctx, x, u_r, u_i, lam, h0, reset, active, c):
        with torch.no_grad():
            y, h_last = rglru_core(x, u_r, u_i, lam, h0, reset, active, c)
        ctx.save_for_backward(x, u_r, u_i, lam, h0, reset, active)
        ctx.c = c
        return y, h_last

    @staticmethod
    def backward(ctx, dy, dh_last):
        x, u_r, u_i, lam, h0, reset, active = ctx.saved_tensors
        got = rglru_backward_linear(x, u_r, u_i, lam, dy, h0=h0, dh_last=dh_last, reset=reset, active=active, c=ctx.c)
        dh0 = None if h0 is None else got["dh0"].to(h0.dtype)
        return (got["dx"].to(x.dtype), got["du_r"].to(u_r.dtype), got["du_i"].to(u_i.dtype), got["dLambda"].to(lam.dtype),
                dh0, None, None, None)


def rglru_layer_linear_backward(
    x: Tensor,
    params: dict[str, Tensor],
    h0: Tensor | None = None,
    reset: Tensor | None = None,
    active: Tensor | None = None,
    c: float = 8.0,
) -> tuple[Tensor, Tensor]:
    """``rglru_layer`` with the O(T) closed-form backward through the gate epilogue and the scan (the gate
    projections stay ordinary autograd)."""
    u_r = block_diagonal_linear(x, params["recurrence_gate.weight"], params["recurrence_gate.bias"])
    u_i = block_diagonal_linear(x, params["input_gate.weight"], params["input_gate.bias"])
    return _CoreLinearBackward.apply(x, u_r, u_i, params["Lambda"], h0, reset, active, c)


def linear_scan(decay: Tensor, drive: Tensor, h0: Tensor) -> Tensor:
    """The raw affine scan operator (griffin/triton_scan.py:130-137, 274-276)."""
    return sequential_scan(decay, drive, h0)[0]


def selftest_vectors(steps: int = 7, width: int = 257) -> dict[str, Tensor]:
    """Closed-form inputs of the reference's per-device scan self-test.

    griffin/triton_scan.py:142-153: decay 0.9 + 0.05 sin(k/97), drive
    0.1 cos(k/53), initial state sin(j/31), upstream cos(k/71).
    """
    k = torch.arange(steps * width, dtype=torch.float32)
    return {
        "decay": (0.9 + 0.05 * torch.sin(k / 97.0)).reshape(1, steps, width),
        "drive": (0.1 * torch.cos(k / 53.0)).reshape(1, steps, width),
        "h0": torch.sin(torch.arange(width) / 31.0)[None],
        "upstream": torch.cos(k / 71.0).reshape(1, steps, width),
    }


# --------------------------------------------------------------------------
# Causal depthwise convolution in front of the RG-LRU and the cached block
# --------------------------------------------------------------------------


def resolve_positions(
    batch: int,
    steps: int,
    segment_pos: Tensor | None,
    previous: Tensor | None,
    active: Tensor | None,
) -> Tensor:
    """Per-token position inside its document (griffin/griffin.py:309-338)."""
    if segment_pos is not None:
        return segment_pos.to(torch.long)
    if active is None:
        active = torch.ones(batch, steps, dtype=torch.bool)
    if previous is None:
        previous = torch.full((batch,), -1, dtype=torch.long)
    return previous.to(torch.long)[:, None] + active.to(torch.long).cumsum(dim=1)


def last_position(segment_pos: Tensor, active: Tensor, previous: Tensor | None) -> Tensor:
    """Position of the last non-padding token of each row (griffin/griffin.py:341-358)."""
    batch = segment_pos.shape[0]
    out = torch.full((batch,), -1, dtype=torch.long) if previous is None else previous.to(torch.long).clone()
    for row in range(batch):
        seen = segment_pos[row][active[row]]
        if seen.numel():
            out[row] = seen[-1]
    return out


def causal_conv_dense(
    x_in: Tensor,
    weight: Tensor,
    bias: Tensor | None,
    conv_state: Tensor,
    segment_pos: Tensor,
) -> tuple[Tensor, Tensor]:
    """Depthwise causal convolution with document-boundary tap masking.

    griffin/griffin.py:474-487.  ``weight`` is [D, K] with column K-1 applied to
    the current token; ``conv_state`` [B, K-1, D] supplies tokens before t=0.
    Returns the convolved sequence and the next conv state (last K-1 rows).
    """
    taps = weight.shape[1]
    hist = taps - 1
    steps = x_in.shape[1]
    padded = torch.cat([conv_state.to(x_in), x_in], dim=1)
    out = x_in.new_zeros(x_in.shape)
    if bias is not None:
        out = out + bias[None, None, :]
    for lag in range(taps):
        window = padded[:, hist - lag : hist - lag + steps]
        same_doc = (segment_pos >= lag).to(window.dtype)
        out = out + window * same_doc[..., None] * weight[None, None, :, taps - 1 - lag]
    new_state = padded[:, -hist:] if hist else padded[:, :0]
    return out, new_state


def causal_conv_padded(
    x_in: Tensor,
    weight: Tensor,
    bias: Tensor | None,
    conv_state: Tensor,
    segment_pos: Tensor,
    active: Tensor,
) -> tuple[Tensor, Tensor]:
    """Variable-length variant: padding neither produces output nor enters history.

    griffin/griffin.py:488-510.
    """
    taps = weight.shape[1]
    hist = taps - 1
    state = conv_state.to(x_in)
    rows = []
    for t in range(x_in.shape[1]):
        on = active[:, t, None]
        start = (segment_pos[:, t] == 0)[:, None, None] & on[:, :, None]
        state = torch.where(start, torch.zeros_like(state), state)
        cur = x_in[:, t]
        if hist:
            val = torch.einsum("bkd,dk->bd", state, weight[:, :hist])
        else:
            val = torch.zeros_like(cur)
        val = val + cur * weight[:, -1]
        if bias is not None:
            val = val + bias
        rows.append(torch.where(on, val, torch.zeros_like(val)))
        if hist:
            moved = torch.cat([state[:, 1:], cur[:, None, :]], dim=1)
            state = torch.where(on[:, :, None], moved, state)
    return torch.stack(rows, dim=1), state


@dataclass
class BlockCache:
    """Mirror of ``RecurrentBlockCache`` (griffin/griffin.py:26-33)."""

    rnn_state: Tensor
    conv_state: Tensor
    segment_position: Tensor


def recurrent_block(
    x: Tensor,
    params: dict[str, Tensor],
    cache: BlockCache | None = None,
    segment_pos: Tensor | None = None,
    active: Tensor | None = None,
    c: float = 8.0,
    linear_backward: bool = False,
) -> tuple[Tensor, BlockCache]:
    """``RecurrentBlock.forward`` (griffin/griffin.py:439-529).

    ``params`` uses the reference's state-dict names (``linear_x.weight`` ...,
    ``temporal_conv.weight`` [D,1,K], ``rg_lru.Lambda`` ...).  ``linear_backward``
    swaps autograd's O(T^2) backward of the scan for the O(T) closed form (same values).
    """
    batch, steps = x.shape[:2]
    everyone = active is None
    if active is None:
        active = torch.ones(batch, steps, dtype=torch.bool)
    previous = None if cache is None else cache.segment_position
    pos = resolve_positions(batch, steps, segment_pos, previous, active)

    gate_branch = F.gelu(F.linear(x, params["linear_y.weight"], params["linear_y.bias"]), approximate="tanh")
    x_in = F.linear(x, params["linear_x.weight"], params["linear_x.bias"])
    conv_w = params["temporal_conv.weight"][:, 0, :]
    conv_b = params.get("temporal_conv.bias")
    taps = conv_w.shape[1]
    width = conv_w.shape[0]
    conv_state = x_in.new_zeros(batch, taps - 1, width) if cache is None else cache.conv_state
    if everyone or bool(active.all()):
        xc, new_conv = causal_conv_dense(x_in, conv_w, conv_b, conv_state, pos)
    else:
        xc, new_conv = causal_conv_padded(x_in, conv_w, conv_b, conv_state, pos, active)

    rnn_params = {k[len("rg_lru.") :]: v for k, v in params.items() if k.startswith("rg_lru.")}
    h0 = None if cache is None else cache.rnn_state
    layer = rglru_layer_linear_backward if linear_backward else rglru_layer
    y, h_last = layer(xc, rnn_params, h0, reset=pos == 0, active=active, c=c)
    out = F.linear(y * gate_branch, params["linear_out.weight"], params["linear_out.bias"])
    out = torch.where(active[..., None], out, torch.zeros_like(out))
    return out, BlockCache(h_last, new_conv, last_position(pos, active, previous))


# --------------------------------------------------------------------------
# Seeded workload builders shared by tests, the golden generator and the bench
# --------------------------------------------------------------------------


def init_lambda(width: int, c: float, gen: torch.Generator) -> Tensor:
    """Lambda with sigmoid(Lambda)^c uniform in [0.9, 0.999] (griffin/griffin.py:183-188)."""
    target = torch.empty(width).uniform_(0.9, 0.999, generator=gen)
    return torch.logit(target.pow(1.0 / c))


def make_rglru_case(
    batch: int,
    steps: int,
    width: int,
    gate_blocks: int,
    seed: int = 0,
    c: float = 8.0,
) -> dict[str, Tensor]:
    """Seeded fp32 inputs and parameters with the benchmark's value distributions.

    x ~ N(0,1); gate weights ~ N(0, 1/bw), zero gate biases
    (griffin/griffin.py:144-147); Lambda as ``init_lambda``; upstream ~ N(0,1).
    Everything is drawn on the CPU generator so the CUDA path and the oracle
    see identical bits.
    """
    gen = torch.Generator().manual_seed(seed)
    bw = width // gate_blocks
    std = math.sqrt(1.0 / bw)
    return {
        "x": torch.randn(batch, steps, width, generator=gen),
        "dy": torch.randn(batch, steps, width, generator=gen),
        "recurrence_gate.weight": torch.randn(gate_blocks, bw, bw, generator=gen) * std,
        "recurrence_gate.bias": torch.zeros(gate_blocks, bw),
        "input_gate.weight": torch.randn(gate_blocks, bw, bw, generator=gen) * std,
        "input_gate.bias": torch.zeros(gate_blocks, bw),
        "Lambda": init_lambda(width, c, gen),
    }


def rel_l2(test: Tensor, ref: Tensor) -> float:
    """Norm-wise relative error ||test - ref|| / ||ref|| in fp64."""
    t = test.detach().to(torch.float64).cpu()
    r = ref.detach().to(torch.float64).cpu()
    denom = r.norm().item()
    num = (t - r).norm().item()
    if denom == 0.0:
        return num
    return num / denom
