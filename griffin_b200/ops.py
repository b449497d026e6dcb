"""Differentiable torch operators over the C ABI.

Each operator is registered with ``torch.library`` (namespace ``griffin_b200``)
with an explicit backward, so autograd, DDP and ``torch.compile`` see ordinary
ops.  Tensors are passed to the library as raw device pointers on the current
CUDA stream; nothing here computes on the CPU.

* ``rglru``        -- gate epilogue + scan (griffin/griffin.py:237-286 of the reference)
* ``linear_scan``  -- raw affine scan, the counterpart of ``fused_rglru_scan``
                      (griffin/triton_scan.py:274-276)
* ``causal_conv``  -- width-4 depthwise causal conv (griffin/griffin.py:474-510)
* ``decode_conv`` / ``decode_step`` -- single-token updates (no autograd)
"""

from __future__ import annotations

import contextlib
import os
from typing import Optional

import torch
from torch import Tensor

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def _io_dtype(t: Tensor, what: str) -> int:
    if t.dtype not in _DTYPES:
        raise TypeError(f"CUDA RG-LRU {what} expects float32 or bfloat16 activations, got {t.dtype}")
    return _DTYPES[t.dtype]


def _require_cuda(*tensors: Optional[Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("CUDA RG-LRU kernels require CUDA tensors (scan_mode='cuda' has no CPU path)")


_NVTX = os.environ.get("RGLRU_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def _on_traced(t: Tensor, name: str):
    with torch.cuda.device(t.device):
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()


def _on(t: Tensor, name: str):
    """Context that makes ``t``'s device current for one library call; with RGLRU_NVTX=1 the call also sits in an
    NVTX range named after the entry point, so a profiler's timeline or range filter shows the operators."""
    return _on_traced(t, name) if _NVTX else torch.cuda.device(t.device)


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


# ----------------------------------------------------------------------------- rglru
@torch.library.custom_op("griffin_b200::rglru_fwd", mutates_args=())
def _rglru_fwd(x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor],
               c: float, save: bool) -> tuple[Tensor, Tensor, Tensor]:
    lib = _lib.load()
    _require_cuda(x, u_r, u_i, lam, h0, tok)
    dt = _io_dtype(x, "forward")
    B, T, D = x.shape
    y = torch.empty_like(x)
    h_last = torch.empty(B, D, device=x.device, dtype=torch.float32)
    nbytes = lib.rglru_workspace_bytes(B, T, D, dt) if save else 0
    ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
    with _on(x, "rglru_fwd"):
        rc = lib.rglru_fwd(_ptr(x), _ptr(u_r), _ptr(u_i), _ptr(lam), _ptr(h0), _ptr(tok), _ptr(y), _ptr(h_last),
                           _ptr(ws) if save else None, nbytes, B, T, D, c, dt, _stream(x))
    _lib.check(rc, "rglru_fwd")
    return y, h_last, ws


@_rglru_fwd.register_fake
def _(x, u_r, u_i, lam, h0, tok, c, save):
    B, T, D = x.shape
    return (torch.empty_like(x), x.new_empty((B, D), dtype=torch.float32), x.new_empty((0,), dtype=torch.uint8))


@torch.library.custom_op("griffin_b200::rglru_bwd", mutates_args=())
def _rglru_bwd(dy: Tensor, dh_last: Optional[Tensor], x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor,
               h0: Optional[Tensor], tok: Optional[Tensor], ws: Tensor, c: float, want_dh0: bool
               ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    lib = _lib.load()
    dt = _io_dtype(x, "backward")
    B, T, D = x.shape
    dx = torch.empty_like(x)
    du_r = torch.empty_like(x)
    du_i = torch.empty_like(x)
    dlam = torch.empty(D, device=x.device, dtype=torch.float32)
    dh0 = torch.empty((B, D) if want_dh0 else (0,), device=x.device, dtype=torch.float32)
    with _on(x, "rglru_bwd"):
        rc = lib.rglru_bwd(_ptr(dy), _ptr(dh_last), _ptr(x), _ptr(u_r), _ptr(u_i), _ptr(lam), _ptr(h0), _ptr(tok),
                           _ptr(ws), ws.numel(), _ptr(dx), _ptr(du_r), _ptr(du_i), _ptr(dlam),
                           _ptr(dh0) if want_dh0 else None, B, T, D, c, dt, _stream(x))
    _lib.check(rc, "rglru_bwd")
    return dx, du_r, du_i, dlam, dh0


@_rglru_bwd.register_fake
def _(dy, dh_last, x, u_r, u_i, lam, h0, tok, ws, c, want_dh0):
    B, T, D = x.shape
    return (torch.empty_like(x), torch.empty_like(x), torch.empty_like(x), x.new_empty((D,), dtype=torch.float32),
            x.new_empty((B, D) if want_dh0 else (0,), dtype=torch.float32))


def _rglru_setup(ctx, inputs, output):
    x, u_r, u_i, lam, h0, tok, c, save = inputs
    _, _, ws = output
    ctx.save_for_backward(x, u_r, u_i, lam, h0, tok, ws)
    ctx.c = c
    ctx.saved = save
    ctx.want_dh0 = h0 is not None and ctx.needs_input_grad[4]


def _rglru_backward(ctx, dy, dh_last, _dws):
    if not ctx.saved:
        raise RuntimeError("rglru was run with save=False (inference); its backward is unavailable")
    x, u_r, u_i, lam, h0, tok, ws = ctx.saved_tensors
    if dy is None:
        dy = torch.zeros_like(x)
    dy = dy.contiguous()
    if dh_last is not None:
        dh_last = dh_last.to(torch.float32).contiguous()
    dx, du_r, du_i, dlam, dh0 = _rglru_bwd(dy, dh_last, x, u_r, u_i, lam, h0, tok, ws, ctx.c, ctx.want_dh0)
    return dx, du_r, du_i, dlam, (dh0 if ctx.want_dh0 else None), None, None, None


_rglru_fwd.register_autograd(_rglru_backward, setup_context=_rglru_setup)


def rglru(x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Optional[Tensor] = None,
          tok: Optional[Tensor] = None, c: float = 8.0) -> tuple[Tensor, Tensor]:
    """y, h_last = RG-LRU(x | gate pre-activations u_r, u_i).  ``lam`` and ``h0`` are fp32."""
    if x.dim() != 3 or u_r.shape != x.shape or u_i.shape != x.shape:
        raise ValueError("x, u_r and u_i must share shape [batch, sequence, width]")
    if u_r.dtype != x.dtype or u_i.dtype != x.dtype:
        raise TypeError("x, u_r and u_i must share one dtype")
    if lam.shape != (x.shape[2],):
        raise ValueError("Lambda must have shape [width]")
    save = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (x, u_r, u_i, lam, h0))
    y, h_last, _ = _rglru_fwd(x.contiguous(), u_r.contiguous(), u_i.contiguous(),
                              lam.to(torch.float32).contiguous(),
                              None if h0 is None else h0.to(torch.float32).contiguous(),
                              None if tok is None else tok.contiguous(), float(c), save)
    return y, h_last


# ----------------------------------------------------------------------------- raw affine scan
@torch.library.custom_op("griffin_b200::linear_scan_fwd", mutates_args=())
def _scan_fwd(decay: Tensor, drive: Tensor, h0: Tensor) -> Tensor:
    lib = _lib.load()
    B, T, D = decay.shape
    out = torch.empty_like(drive)
    with _on(decay, "rglru_linear_scan_fwd"):
        rc = lib.rglru_linear_scan_fwd(_ptr(decay), _ptr(drive), _ptr(h0), _ptr(out), B, T, D, _stream(decay))
    _lib.check(rc, "rglru_linear_scan_fwd")
    return out


@_scan_fwd.register_fake
def _(decay, drive, h0):
    return torch.empty_like(drive)


@torch.library.custom_op("griffin_b200::linear_scan_bwd", mutates_args=())
def _scan_bwd(d_out: Tensor, decay: Tensor, h0: Tensor, out: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    lib = _lib.load()
    B, T, D = decay.shape
    d_decay = torch.empty_like(decay)
    d_drive = torch.empty_like(decay)
    d_h0 = torch.empty_like(h0)
    with _on(decay, "rglru_linear_scan_bwd"):
        rc = lib.rglru_linear_scan_bwd(_ptr(d_out), _ptr(decay), _ptr(h0), _ptr(out), _ptr(d_decay), _ptr(d_drive),
                                       _ptr(d_h0), B, T, D, _stream(decay))
    _lib.check(rc, "rglru_linear_scan_bwd")
    return d_decay, d_drive, d_h0


@_scan_bwd.register_fake
def _(d_out, decay, h0, out):
    return torch.empty_like(decay), torch.empty_like(decay), torch.empty_like(h0)


def _scan_setup(ctx, inputs, output):
    decay, _, h0 = inputs
    ctx.save_for_backward(decay, h0, output)


def _scan_backward(ctx, d_out):
    decay, h0, out = ctx.saved_tensors
    return _scan_bwd(d_out.contiguous(), decay, h0, out)


_scan_fwd.register_autograd(_scan_backward, setup_context=_scan_setup)


def linear_scan(decay: Tensor, current_input: Tensor, initial_state: Tensor) -> Tensor:
    """h_t = decay_t * h_{t-1} + current_input_t; same contract as the reference's
    ``fused_rglru_scan`` (griffin/triton_scan.py:211-224, 274-276)."""
    if not decay.is_cuda or not current_input.is_cuda or not initial_state.is_cuda:
        raise RuntimeError("CUDA linear scan requires CUDA tensors")
    if decay.shape != current_input.shape or decay.dim() != 3:
        raise ValueError("decay and current_input must share shape [batch, sequence, width]")
    if initial_state.shape != (decay.size(0), decay.size(2)):
        raise ValueError("initial_state must have shape [batch, width]")
    if decay.dtype != torch.float32 or current_input.dtype != torch.float32:
        raise TypeError("CUDA linear scan expects fp32 decay and normalized input")
    if initial_state.dtype != torch.float32:
        raise TypeError("CUDA linear scan expects fp32 recurrent state")
    return _scan_fwd(decay.contiguous(), current_input.contiguous(), initial_state.contiguous())


# ----------------------------------------------------------------------------- causal conv
@torch.library.custom_op("griffin_b200::conv_fwd", mutates_args=())
def _conv_fwd(x_in: Tensor, w: Tensor, b: Optional[Tensor], state: Optional[Tensor], tok: Optional[Tensor]
              ) -> tuple[Tensor, Tensor]:
    lib = _lib.load()
    _require_cuda(x_in, w, b, state, tok)
    dt = _io_dtype(x_in, "conv")
    B, T, D = x_in.shape
    out = torch.empty_like(x_in)
    new_state = torch.empty(B, 3, D, device=x_in.device, dtype=x_in.dtype)
    with _on(x_in, "rglru_conv_fwd"):
        rc = lib.rglru_conv_fwd(_ptr(x_in), _ptr(w), _ptr(b), _ptr(state), _ptr(tok), _ptr(out), _ptr(new_state),
                                B, T, D, dt, _stream(x_in))
    _lib.check(rc, "rglru_conv_fwd")
    return out, new_state


@_conv_fwd.register_fake
def _(x_in, w, b, state, tok):
    B, T, D = x_in.shape
    return torch.empty_like(x_in), x_in.new_empty((B, 3, D))


@torch.library.custom_op("griffin_b200::conv_bwd", mutates_args=())
def _conv_bwd(d_conv: Tensor, x_in: Tensor, w: Tensor, state: Optional[Tensor], tok: Optional[Tensor],
              want_state: bool) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    lib = _lib.load()
    dt = _io_dtype(x_in, "conv backward")
    B, T, D = x_in.shape
    dx = torch.empty_like(x_in)
    d_w = torch.empty(D, 4, device=x_in.device, dtype=torch.float32)
    d_b = torch.empty(D, device=x_in.device, dtype=torch.float32)
    d_state = torch.empty((B, 3, D) if want_state else (0,), device=x_in.device, dtype=x_in.dtype)
    nbytes = lib.rglru_conv_bwd_workspace_bytes(B, T, D)
    ws = torch.empty(nbytes, device=x_in.device, dtype=torch.uint8)
    with _on(x_in, "rglru_conv_bwd"):
        rc = lib.rglru_conv_bwd(_ptr(d_conv), _ptr(x_in), _ptr(w), _ptr(state), _ptr(tok), _ptr(dx), _ptr(d_w),
                                _ptr(d_b), _ptr(d_state) if want_state else None, _ptr(ws), nbytes, B, T, D, dt,
                                _stream(x_in))
    _lib.check(rc, "rglru_conv_bwd")
    return dx, d_w, d_b, d_state


@_conv_bwd.register_fake
def _(d_conv, x_in, w, state, tok, want_state):
    B, T, D = x_in.shape
    return (torch.empty_like(x_in), x_in.new_empty((D, 4), dtype=torch.float32),
            x_in.new_empty((D,), dtype=torch.float32), x_in.new_empty((B, 3, D) if want_state else (0,)))


def _conv_setup(ctx, inputs, output):
    x_in, w, b, state, tok = inputs
    ctx.save_for_backward(x_in, w, state, tok)
    ctx.has_bias = b is not None
    ctx.want_state = state is not None and ctx.needs_input_grad[3]


def _conv_backward(ctx, d_out, _d_new_state):
    x_in, w, state, tok = ctx.saved_tensors
    dx, d_w, d_b, d_state = _conv_bwd(d_out.contiguous(), x_in, w, state, tok, ctx.want_state)
    return dx, d_w, (d_b if ctx.has_bias else None), (d_state if ctx.want_state else None), None


_conv_fwd.register_autograd(_conv_backward, setup_context=_conv_setup)


def causal_conv(x_in: Tensor, weight: Tensor, bias: Optional[Tensor], conv_state: Optional[Tensor] = None,
                tok: Optional[Tensor] = None) -> tuple[Tensor, Tensor]:
    """Width-4 depthwise causal convolution; ``weight`` is [D, 4] with column 3 on the current token.

    Returns the convolved sequence and the next conv state [B, 3, D].  The gradient with
    respect to the returned state is not propagated (the reference never differentiates it).
    """
    if x_in.dim() != 3:
        raise ValueError("conv input must be [batch, sequence, width]")
    if weight.shape != (x_in.shape[2], 4):
        raise ValueError("CUDA causal conv supports kernel width 4 with weight [width, 4]")
    w = weight.to(torch.float32).contiguous()
    b = None if bias is None else bias.to(torch.float32).contiguous()
    st = None if conv_state is None else conv_state.to(x_in.dtype).contiguous()
    return _conv_fwd(x_in.contiguous(), w, b, st, None if tok is None else tok.contiguous())


# ----------------------------------------------------------------------------- conv folded into the scan
def conv_scan_fwd(x_in: Tensor, conv_w: Tensor, conv_b: Optional[Tensor], conv_state: Optional[Tensor], u_r: Tensor,
                  u_i: Tensor, lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor], c: float, save: bool
                  ) -> tuple[Tensor, Tensor, Tensor]:
    """y, h_last, workspace = RG-LRU(conv(x_in) | u_r, u_i) with the conv applied while chunks are loaded
    (``rglru_conv_scan_fwd``).  All tensors contiguous; ``conv_w`` [D,4] / ``conv_b`` / ``lam`` / ``h0`` fp32."""
    lib = _lib.load()
    _require_cuda(x_in, conv_w, conv_b, conv_state, u_r, u_i, lam, h0, tok)
    dt = _io_dtype(x_in, "conv-scan forward")
    B, T, D = x_in.shape
    y = torch.empty_like(x_in)
    h_last = torch.empty(B, D, device=x_in.device, dtype=torch.float32)
    nbytes = lib.rglru_workspace_bytes(B, T, D, dt) if save else 0
    ws = torch.empty(nbytes, device=x_in.device, dtype=torch.uint8)
    with _on(x_in, "rglru_conv_scan_fwd"):
        rc = lib.rglru_conv_scan_fwd(_ptr(x_in), _ptr(conv_w), _ptr(conv_b), _ptr(conv_state), _ptr(u_r), _ptr(u_i),
                                     _ptr(lam), _ptr(h0), _ptr(tok), _ptr(y), _ptr(h_last),
                                     _ptr(ws) if save else None, nbytes, B, T, D, c, dt, _stream(x_in))
    _lib.check(rc, "rglru_conv_scan_fwd")
    return y, h_last, ws


def conv_scan_bwd(dy: Tensor, dh_last: Optional[Tensor], x_in: Tensor, conv_w: Tensor, conv_b: Optional[Tensor],
                  conv_state: Optional[Tensor], u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Optional[Tensor],
                  tok: Optional[Tensor], ws: Tensor, c: float, want_dh0: bool
                  ) -> tuple[Tensor, Tensor, Tensor, Tensor, Optional[Tensor]]:
    """Backward of :func:`conv_scan_fwd`: (d x_conv direct path, d u_r, d u_i, d Lambda, d h0)."""
    lib = _lib.load()
    dt = _io_dtype(x_in, "conv-scan backward")
    B, T, D = x_in.shape
    dxc, du_r, du_i = torch.empty_like(x_in), torch.empty_like(x_in), torch.empty_like(x_in)
    dlam = torch.empty(D, device=x_in.device, dtype=torch.float32)
    dh0 = torch.empty(B, D, device=x_in.device, dtype=torch.float32) if want_dh0 else None
    with _on(x_in, "rglru_conv_scan_bwd"):
        rc = lib.rglru_conv_scan_bwd(_ptr(dy), _ptr(dh_last), _ptr(x_in), _ptr(conv_w), _ptr(conv_b), _ptr(conv_state),
                                     _ptr(u_r), _ptr(u_i), _ptr(lam), _ptr(h0), _ptr(tok), _ptr(ws), ws.numel(),
                                     _ptr(dxc), _ptr(du_r), _ptr(du_i), _ptr(dlam), _ptr(dh0), B, T, D, c, dt,
                                     _stream(x_in))
    _lib.check(rc, "rglru_conv_scan_bwd")
    return dxc, du_r, du_i, dlam, dh0


# ----------------------------------------------------------------------------- GeLU branch merged into the scan
def merge_scan_fwd(x: Tensor, conv_w: Optional[Tensor], conv_b: Optional[Tensor], conv_state: Optional[Tensor],
                   u_r: Tensor, u_i: Tensor, branch: Tensor, lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor],
                   c: float, save: bool) -> tuple[Tensor, Tensor, Tensor]:
    """out, h_last, workspace with out = RG-LRU(...) * gelu_tanh(branch) formed in the scan's store stage
    (``rglru_merge_fwd``).  With ``conv_w`` given, ``x`` is the conv input and the conv is applied while loading."""
    lib = _lib.load()
    _require_cuda(x, conv_w, conv_b, conv_state, u_r, u_i, branch, lam, h0, tok)
    dt = _io_dtype(x, "merged scan forward")
    B, T, D = x.shape
    out = torch.empty_like(x)
    h_last = torch.empty(B, D, device=x.device, dtype=torch.float32)
    nbytes = lib.rglru_workspace_bytes(B, T, D, dt) if save else 0
    ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
    with _on(x, "rglru_merge_fwd"):
        rc = lib.rglru_merge_fwd(_ptr(x), _ptr(conv_w), _ptr(conv_b), _ptr(conv_state), _ptr(u_r), _ptr(u_i),
                                 _ptr(branch), _ptr(lam), _ptr(h0), _ptr(tok), _ptr(out), _ptr(h_last),
                                 _ptr(ws) if save else None, nbytes, B, T, D, c, dt, _stream(x))
    _lib.check(rc, "rglru_merge_fwd")
    return out, h_last, ws


def merge_scan_bwd(dout: Tensor, dh_last: Optional[Tensor], x: Tensor, conv_w: Optional[Tensor],
                   conv_b: Optional[Tensor], conv_state: Optional[Tensor], u_r: Tensor, u_i: Tensor, branch: Tensor,
                   lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor], ws: Tensor, c: float, want_dh0: bool
                   ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Optional[Tensor]]:
    """Backward of :func:`merge_scan_fwd`: (d x direct path, d u_r, d u_i, d branch, d Lambda, d h0)."""
    lib = _lib.load()
    dt = _io_dtype(x, "merged scan backward")
    B, T, D = x.shape
    dx, du_r, du_i, dbranch = (torch.empty_like(x) for _ in range(4))
    dlam = torch.empty(D, device=x.device, dtype=torch.float32)
    dh0 = torch.empty(B, D, device=x.device, dtype=torch.float32) if want_dh0 else None
    with _on(x, "rglru_merge_bwd"):
        rc = lib.rglru_merge_bwd(_ptr(dout), _ptr(dh_last), _ptr(x), _ptr(conv_w), _ptr(conv_b), _ptr(conv_state),
                                 _ptr(u_r), _ptr(u_i), _ptr(branch), _ptr(lam), _ptr(h0), _ptr(tok), _ptr(ws),
                                 ws.numel(), _ptr(dx), _ptr(du_r), _ptr(du_i), _ptr(dbranch), _ptr(dlam), _ptr(dh0),
                                 B, T, D, c, dt, _stream(x))
    _lib.check(rc, "rglru_merge_bwd")
    return dx, du_r, du_i, dbranch, dlam, dh0


class _MergedScan(torch.autograd.Function):
    """RG-LRU whose output is multiplied by gelu_tanh(branch) inside the scan kernels (no conv fold)."""

    @staticmethod
    def forward(ctx, x, u_r, u_i, branch, lam, h0, tok, c):
        lam32 = lam.to(torch.float32).contiguous()
        h032 = None if h0 is None else h0.to(torch.float32).contiguous()
        x, u_r, u_i, branch = x.contiguous(), u_r.contiguous(), u_i.contiguous(), branch.to(x.dtype).contiguous()
        save = any(ctx.needs_input_grad)
        out, h_last, ws = merge_scan_fwd(x, None, None, None, u_r, u_i, branch, lam32, h032, tok, float(c), save)
        ctx.save_for_backward(x, u_r, u_i, branch, lam32, h032, tok, ws)
        ctx.c, ctx.lam_dtype = float(c), lam.dtype
        return out, h_last

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dout, dh_last):
        x, u_r, u_i, branch, lam32, h032, tok, ws = ctx.saved_tensors
        if ws.numel() == 0:
            raise RuntimeError("merged scan was run without saving its workspace; backward is unavailable")
        dh_last = None if dh_last is None else dh_last.to(torch.float32).contiguous()
        want_dh0 = h032 is not None and ctx.needs_input_grad[5]
        dx, du_r, du_i, dbranch, dlam, dh0 = merge_scan_bwd(dout.contiguous(), dh_last, x, None, None, None, u_r, u_i,
                                                            branch, lam32, h032, tok, ws, ctx.c, want_dh0)
        return dx, du_r, du_i, dbranch, dlam.to(ctx.lam_dtype), dh0, None, None


def rglru_merged(x: Tensor, u_r: Tensor, u_i: Tensor, branch: Tensor, lam: Tensor, h0: Optional[Tensor] = None,
                 tok: Optional[Tensor] = None, c: float = 8.0) -> tuple[Tensor, Tensor]:
    """(RG-LRU(x | u_r, u_i) * gelu(branch, approximate="tanh"), h_last): the recurrent block's branch merge
    (griffin/griffin.py:464, 520 of the reference) formed and differentiated inside the scan kernels."""
    if x.dim() != 3 or u_r.shape != x.shape or u_i.shape != x.shape or branch.shape != x.shape:
        raise ValueError("x, u_r, u_i and branch must share shape [batch, sequence, width]")
    if u_r.dtype != x.dtype or u_i.dtype != x.dtype:
        raise TypeError("x, u_r and u_i must share one dtype")
    if lam.shape != (x.shape[2],):
        raise ValueError("Lambda must have shape [width]")
    return _MergedScan.apply(x, u_r, u_i, branch, lam, h0, None if tok is None else tok.contiguous(), c)


# ----------------------------------------------------------------------------- both gates from one grouped GEMM
def grouped_gates_supported(x: Tensor, gate_width: int) -> bool:
    """Whether the grouped gate layout can be used: CUDA, a gate head that is a whole number of 64-channel
    tiles, and rows the copy engine can address."""
    return x.is_cuda and gate_width % 64 == 0 and (x.shape[-1] * x.element_size()) % 16 == 0


def _aligned16(t: Optional[Tensor]) -> Optional[Tensor]:
    return t if t is None or t.data_ptr() % 16 == 0 else t.clone()


class _GroupedRGLRU(torch.autograd.Function):
    """Gate projections + RG-LRU (+ optional GeLU-branch product) as one node around ONE grouped GEMM.

    The two [G, bw, bw] gate weights are stacked per head and a single batched GEMM writes both gate
    pre-activations straight into a [B, T, G, 2 bw] tensor (cuBLAS takes the strided output, so there is no
    re-layout pass); the kernels read that layout, add the biases themselves and return the gradient in the
    same layout, from which two more batched GEMMs give the input and weight gradients.
    Reference: BlockDiagonalLinear griffin/griffin.py:129-154 called twice at :237-238."""

    @staticmethod
    def forward(ctx, x, w_r, b_r, w_i, b_i, lam, h0, tok, c, branch):
        lib = _lib.load()
        with torch.autocast("cuda", enabled=False):
            x = _aligned16(x.contiguous())
            B, T, D = x.shape
            G, bw, _ = w_r.shape
            dt = _io_dtype(x, "grouped forward")
            wcat = torch.cat([w_r, w_i], dim=1).to(x.dtype)                                   # [G, 2 bw, bw]
            bias = torch.cat([b_r, b_i], dim=1).to(torch.float32).reshape(-1).contiguous()    # [2 D]
            rows = x.view(B * T, G, bw).transpose(0, 1)                                       # [G, N, bw] view
            u = torch.empty(B, T, 2 * D, device=x.device, dtype=x.dtype)
            torch.bmm(rows, wcat.transpose(1, 2), out=u.view(B * T, G, 2 * bw).transpose(0, 1))
            lam32 = lam.to(torch.float32).contiguous()
            h032 = None if h0 is None else h0.to(torch.float32).contiguous()
            branch = None if branch is None else _aligned16(branch.to(x.dtype).contiguous())
            save = any(ctx.needs_input_grad)
            out = torch.empty_like(x)
            h_last = torch.empty(B, D, device=x.device, dtype=torch.float32)
            nbytes = lib.rglru_workspace_bytes(B, T, D, dt) if save else 0
            ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
            with _on(x, "rglru_grouped_fwd"):
                rc = lib.rglru_grouped_fwd(_ptr(x), _ptr(u), _ptr(bias), _ptr(branch), _ptr(lam32), _ptr(h032), _ptr(tok),
                                           _ptr(out), _ptr(h_last), _ptr(ws) if save else None, nbytes, B, T, D, bw,
                                           float(c), dt, _stream(x))
            _lib.check(rc, "rglru_grouped_fwd")
        ctx.save_for_backward(x, u, wcat, bias, lam32, h032, tok, ws, branch)
        ctx.c = float(c)
        ctx.meta = (w_r.dtype, b_r.dtype, w_i.dtype, b_i.dtype, lam.dtype)
        return out, h_last

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dout, dh_last):
        lib = _lib.load()
        x, u, wcat, bias, lam32, h032, tok, ws, branch = ctx.saved_tensors
        if ws.numel() == 0:
            raise RuntimeError("grouped RG-LRU was run without saving its workspace; backward is unavailable")
        with torch.autocast("cuda", enabled=False):
            B, T, D = x.shape
            G, bw2, bw = wcat.shape
            dt = _io_dtype(x, "grouped backward")
            dout = _aligned16(dout.to(x.dtype).contiguous())
            dh_last = None if dh_last is None else dh_last.to(torch.float32).contiguous()
            want_dh0 = h032 is not None and ctx.needs_input_grad[6]
            dx = torch.empty_like(x)
            du = torch.empty_like(u)
            dbranch = None if branch is None else torch.empty_like(x)
            dlam = torch.empty(D, device=x.device, dtype=torch.float32)
            dh0 = torch.empty(B, D, device=x.device, dtype=torch.float32) if want_dh0 else None
            with _on(x, "rglru_grouped_bwd"):
                rc = lib.rglru_grouped_bwd(_ptr(dout), _ptr(dh_last), _ptr(x), _ptr(u), _ptr(bias), _ptr(branch),
                                           _ptr(lam32), _ptr(h032), _ptr(tok), _ptr(ws), ws.numel(), _ptr(dx), _ptr(du),
                                           _ptr(dbranch), _ptr(dlam), _ptr(dh0), B, T, D, bw, ctx.c, dt, _stream(x))
            _lib.check(rc, "rglru_grouped_bwd")
            dg = du.view(B * T, G, bw2).transpose(0, 1)                    # [G, N, 2 bw] view
            rows = x.view(B * T, G, bw).transpose(0, 1)                    # [G, N, bw] view
            dx.view(B * T, G, bw).transpose(0, 1).baddbmm_(dg, wcat)       # gate path added onto the direct path
            dwcat = torch.bmm(dg.transpose(1, 2), rows)                    # [G, 2 bw, bw]
            dbias = du.view(B * T, G, bw2).sum(dim=0, dtype=torch.float32)  # [G, 2 bw]
        wr_dt, br_dt, wi_dt, bi_dt, lam_dt = ctx.meta
        return (dx, dwcat[:, :bw].to(wr_dt), dbias[:, :bw].to(br_dt), dwcat[:, bw:].to(wi_dt), dbias[:, bw:].to(bi_dt),
                dlam.to(lam_dt), dh0, None, None, dbranch)


def rglru_grouped(x: Tensor, w_r: Tensor, b_r: Tensor, w_i: Tensor, b_i: Tensor, lam: Tensor,
                  h0: Optional[Tensor] = None, tok: Optional[Tensor] = None, c: float = 8.0,
                  branch: Optional[Tensor] = None) -> tuple[Tensor, Tensor]:
    """y, h_last = RG-LRU(x) with both block-diagonal gate projections (weights [G, out, in], biases [G, out])
    computed inside the node by one grouped GEMM; with ``branch`` the first result is y * gelu_tanh(branch)."""
    if x.dim() != 3:
        raise ValueError("x must be [batch, sequence, width]")
    G, bw, bw_in = w_r.shape
    if bw != bw_in or w_i.shape != w_r.shape or G * bw != x.shape[2] or b_r.shape != (G, bw) or b_i.shape != (G, bw):
        raise ValueError("gate weights must be [heads, width/heads, width/heads] and biases [heads, width/heads]")
    if lam.shape != (x.shape[2],):
        raise ValueError("Lambda must have shape [width]")
    if branch is not None and branch.shape != x.shape:
        raise ValueError("branch must have the shape of x")
    if not grouped_gates_supported(x, bw):
        raise ValueError("the grouped gate layout needs CUDA tensors, gate heads of a multiple of 64 channels and "
                         "rows that are a multiple of 16 bytes")
    return _GroupedRGLRU.apply(x, w_r, b_r, w_i, b_i, lam, h0, None if tok is None else tok.contiguous(), c, branch)


def _gate(x: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
    """Block-diagonal projection [.., G*in] -> [.., G*out] in x's dtype (weight [G, out, in])."""
    g, wo, wi = weight.shape
    rows = x.reshape(-1, g, wi).transpose(0, 1)
    out = torch.baddbmm(bias.to(x.dtype)[:, None, :], rows, weight.to(x.dtype).transpose(1, 2))
    return out.transpose(0, 1).reshape(*x.shape[:-1], g * wo).contiguous()   # reshape may return a strided view


def _gate_backward(du: Tensor, x: Tensor, weight: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    """(d x, d weight, d bias) of :func:`_gate`."""
    g, wo, wi = weight.shape
    rows = x.reshape(-1, g, wi).transpose(0, 1)            # [G, N, in]
    d = du.reshape(-1, g, wo).transpose(0, 1)              # [G, N, out]
    dx = torch.bmm(d, weight.to(du.dtype)).transpose(0, 1).reshape(x.shape).contiguous()
    dw = torch.bmm(d.transpose(1, 2), rows).to(weight.dtype)
    db = d.sum(dim=1, dtype=torch.float32)
    return dx, dw, db


class _RecurrentCore(torch.autograd.Function):
    """conv -> gate projections -> RG-LRU as one autograd node that keeps only the conv INPUT.

    Forward materialises the conv output once for the two gate GEMMs and drops it; the scan kernels read the
    conv input and redo the four taps in their load stage.  Backward recomputes the conv output (one streaming
    pass) for the gate-weight gradients, sums the direct and gate paths and runs a single conv backward.
    """

    @staticmethod
    def forward(ctx, x_in, conv_w, conv_b, conv_state, w_r, b_r, w_i, b_i, lam, h0, tok, c, branch):
        x_in = x_in.contiguous()
        cw = conv_w.to(torch.float32).contiguous()
        cb = None if conv_b is None else conv_b.to(torch.float32).contiguous()
        cs = None if conv_state is None else conv_state.to(x_in.dtype).contiguous()
        lam32 = lam.to(torch.float32).contiguous()
        h032 = None if h0 is None else h0.to(torch.float32).contiguous()
        x_conv, new_state = _conv_fwd(x_in, cw, cb, cs, tok)
        u_r = _gate(x_conv, w_r, b_r)
        u_i = _gate(x_conv, w_i, b_i)
        del x_conv
        save = any(ctx.needs_input_grad)
        if branch is None:
            y, h_last, ws = conv_scan_fwd(x_in, cw, cb, cs, u_r, u_i, lam32, h032, tok, float(c), save)
        else:
            branch = branch.to(x_in.dtype).contiguous()
            y, h_last, ws = merge_scan_fwd(x_in, cw, cb, cs, u_r, u_i, branch, lam32, h032, tok, float(c), save)
        ctx.save_for_backward(x_in, cw, cb, cs, w_r, w_i, lam32, h032, tok, u_r, u_i, ws, branch)
        ctx.c = float(c)
        ctx.meta = (conv_w.dtype, None if conv_b is None else conv_b.dtype, b_r.dtype, b_i.dtype, lam.dtype)
        ctx.mark_non_differentiable(new_state)
        return y, h_last, new_state

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy, dh_last, _d_state):
        x_in, cw, cb, cs, w_r, w_i, lam32, h032, tok, u_r, u_i, ws, branch = ctx.saved_tensors
        if ws.numel() == 0:
            raise RuntimeError("recurrent core was run without saving its workspace; backward is unavailable")
        dy = dy.contiguous()
        dh_last = None if dh_last is None else dh_last.to(torch.float32).contiguous()
        want_dh0 = h032 is not None and ctx.needs_input_grad[9]
        dbranch = None
        if branch is None:
            dxc, du_r, du_i, dlam, dh0 = conv_scan_bwd(dy, dh_last, x_in, cw, cb, cs, u_r, u_i, lam32, h032, tok, ws,
                                                       ctx.c, want_dh0)
        else:
            dxc, du_r, du_i, dbranch, dlam, dh0 = merge_scan_bwd(dy, dh_last, x_in, cw, cb, cs, u_r, u_i, branch, lam32,
                                                                 h032, tok, ws, ctx.c, want_dh0)
        x_conv, _ = _conv_fwd(x_in, cw, cb, cs, tok)          # recomputed, not saved
        dx_r, dw_r, db_r = _gate_backward(du_r, x_conv, w_r)
        dx_i, dw_i, db_i = _gate_backward(du_i, x_conv, w_i)
        total = (dxc + dx_r + dx_i).contiguous()
        want_state = cs is not None and ctx.needs_input_grad[3]
        dx_in, d_w, d_b, d_state = _conv_bwd(total, x_in, cw, cs, tok, want_state)
        wdt, bdt, brdt, bidt, ldt = ctx.meta
        return (dx_in, d_w.to(wdt), None if cb is None else d_b.to(bdt), d_state if want_state else None,
                dw_r, db_r.to(brdt), dw_i, db_i.to(bidt), dlam.to(ldt), dh0, None, None, dbranch)


def recurrent_core(x_in: Tensor, conv_w: Tensor, conv_b: Optional[Tensor], conv_state: Optional[Tensor],
                   w_r: Tensor, b_r: Tensor, w_i: Tensor, b_i: Tensor, lam: Tensor, h0: Optional[Tensor] = None,
                   tok: Optional[Tensor] = None, c: float = 8.0, branch: Optional[Tensor] = None
                   ) -> tuple[Tensor, Tensor, Tensor]:
    """(y, h_last, new_conv_state) of conv k=4 -> block-diagonal gates -> RG-LRU, keeping only ``x_in`` for backward.

    With ``branch`` (the pre-activation of the block's GeLU branch, same shape as ``x_in``) the first result is
    ``y * gelu(branch, approximate="tanh")``, formed inside the scan kernels in both directions."""
    if branch is not None and branch.shape != x_in.shape:
        raise ValueError("branch must have the shape of x_in")
    if x_in.dim() != 3 or conv_w.shape != (x_in.shape[2], 4):
        raise ValueError("x_in must be [batch, sequence, width] and conv_w [width, 4]")
    return _RecurrentCore.apply(x_in, conv_w, conv_b, conv_state, w_r, b_r, w_i, b_i, lam, h0,
                                None if tok is None else tok.contiguous(), c, branch)


# ----------------------------------------------------------------------------- decode (in-place state, no autograd)
def decode_conv(x_in: Tensor, weight: Tensor, bias: Optional[Tensor], conv_state: Tensor,
                tok: Optional[Tensor] = None) -> Tensor:
    """One token of the causal conv; ``conv_state`` [B,3,D] is updated in place."""
    lib = _lib.load()
    _require_cuda(x_in, weight, bias, conv_state, tok)
    dt = _io_dtype(x_in, "decode conv")
    B, D = x_in.shape
    if conv_state.shape != (B, 3, D) or conv_state.dtype != x_in.dtype or not conv_state.is_contiguous():
        raise ValueError("conv_state must be a contiguous [batch, 3, width] tensor of the activation dtype")
    out = torch.empty_like(x_in)
    with _on(x_in, "rglru_decode_conv"):
        rc = lib.rglru_decode_conv(_ptr(x_in.contiguous()), _ptr(weight), _ptr(bias), _ptr(conv_state), _ptr(tok),
                                   _ptr(out), B, D, dt, _stream(x_in))
    _lib.check(rc, "rglru_decode_conv")
    return out


def decode_step(x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h: Tensor, tok: Optional[Tensor] = None,
                c: float = 8.0) -> Tensor:
    """One token of the RG-LRU; the fp32 state ``h`` [B,D] is updated in place, returns y."""
    lib = _lib.load()
    _require_cuda(x, u_r, u_i, lam, h, tok)
    dt = _io_dtype(x, "decode step")
    B, D = x.shape
    if h.shape != (B, D) or h.dtype != torch.float32 or not h.is_contiguous():
        raise ValueError("h must be a contiguous fp32 [batch, width] tensor")
    y = torch.empty_like(x)
    with _on(x, "rglru_decode_step"):
        rc = lib.rglru_decode_step(_ptr(x.contiguous()), _ptr(u_r.contiguous()), _ptr(u_i.contiguous()), _ptr(lam),
                                   _ptr(h), _ptr(tok), _ptr(y), B, D, float(c), dt, _stream(x))
    _lib.check(rc, "rglru_decode_step")
    return y
