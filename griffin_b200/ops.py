"""Differentiable torch operators over the C ABI.

Every differentiable operator here -- the plain, merged, grouped and conv-folded scans, the raw
affine scan and the conv -- is a ``torch.library`` custom op (namespace ``griffin_b200``) with an
explicit backward op and a fake (shape-only) implementation, so autograd, DDP and ``torch.compile``
see ordinary ops.  Tensors are passed to the library as raw device pointers on the current
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


_SAME_DEVICE = contextlib.nullcontext()


def _on(t: Tensor, name: str):
    """Context that makes ``t``'s device current for one library call (nothing to do when it already is); with
    RGLRU_NVTX=1 the call also sits in an NVTX range named after the entry point, so a profiler's timeline or
    range filter shows the operators."""
    if _NVTX:
        return _on_traced(t, name)
    if t.device.index == torch.cuda.current_device():
        return _SAME_DEVICE
    return torch.cuda.device(t.device)


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: Tensor) -> int:
    """The current stream of ``t``'s device as the integer handle the C ABI takes."""
    if _raw_stream is not None:
        return _raw_stream(t.device.index)
    return torch.cuda.current_stream(t.device).cuda_stream


# Every differentiable operator exists in two forms over the same implementation functions: a ``torch.library``
# custom op (with fake implementation and registered backward), which is what ``torch.compile`` and other
# tracers see, and a plain ``torch.autograd.Function``, which is what eager calls use because it costs a
# fraction of the dispatcher round trip per call (the block is launch-bound on the host at these sizes).
_FORCE_LIBRARY_OPS = False


@contextlib.contextmanager
def library_ops(enabled: bool = True):
    """Route eager calls through the ``torch.library`` custom ops as well (tracing with fake tensors, opcheck)."""
    global _FORCE_LIBRARY_OPS
    previous, _FORCE_LIBRARY_OPS = _FORCE_LIBRARY_OPS, enabled
    try:
        yield
    finally:
        _FORCE_LIBRARY_OPS = previous


def _library_ops_active() -> bool:
    return _FORCE_LIBRARY_OPS or torch.compiler.is_compiling()


def _eager_node(name: str, fwd_impl, setup, backward_rule, bwd_impl):
    """The autograd.Function twin of a custom op: same forward implementation, same set-up and backward rule."""

    class Node(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *args):
            ctx.set_materialize_grads(False)     # results nobody differentiates (workspace, gate tensor) stay None
            out = fwd_impl(*args)
            setup(ctx, args, out)
            return out

        @staticmethod
        @torch.autograd.function.once_differentiable
        def backward(ctx, *grads):
            return backward_rule(ctx, *grads, _bwd=bwd_impl)

    Node.__name__ = Node.__qualname__ = name
    return Node


# ----------------------------------------------------------------------------- rglru
def _rglru_fwd_impl(x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor],
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


def workspace_bytes(B, T, D):
    """Bytes of the scan workspace (``rglru_workspace_bytes``) as plain arithmetic, for shape inference: the
    states entering every 64-step chunk, one row of dLambda partial sums per batch row, a 256-byte tail, and one row
    of gate-sum partials [2 D] per batch row."""
    return (B * ((T + 63) // 64) * D + B * D) * 4 + 256 + B * 2 * D * 4


_rglru_fwd = torch.library.custom_op("griffin_b200::rglru_fwd", _rglru_fwd_impl, mutates_args=())


@_rglru_fwd.register_fake
def _(x, u_r, u_i, lam, h0, tok, c, save):
    B, T, D = x.shape
    return (torch.empty_like(x), x.new_empty((B, D), dtype=torch.float32),
            x.new_empty((workspace_bytes(B, T, D) if save else 0,), dtype=torch.uint8))


def _rglru_bwd_impl(dy: Tensor, dh_last: Optional[Tensor], x: Tensor, u_r: Tensor, u_i: Tensor, lam: Tensor,
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


_rglru_bwd = torch.library.custom_op("griffin_b200::rglru_bwd", _rglru_bwd_impl, mutates_args=())


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


def _rglru_backward(ctx, dy, dh_last, _dws, _bwd=None):
    if not ctx.saved:
        raise RuntimeError("rglru was run with save=False (inference); its backward is unavailable")
    x, u_r, u_i, lam, h0, tok, ws = ctx.saved_tensors
    if dy is None:
        dy = torch.zeros_like(x)
    dy = dy.contiguous()
    if dh_last is not None:
        dh_last = dh_last.to(torch.float32).contiguous()
    dx, du_r, du_i, dlam, dh0 = (_bwd or _rglru_bwd)(dy, dh_last, x, u_r, u_i, lam, h0, tok, ws, ctx.c, ctx.want_dh0)
    return dx, du_r, du_i, dlam, (dh0 if ctx.want_dh0 else None), None, None, None


_rglru_fwd.register_autograd(_rglru_backward, setup_context=_rglru_setup)
_RglruNode = _eager_node("RglruScan", _rglru_fwd_impl, _rglru_setup, _rglru_backward, _rglru_bwd_impl)


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
    y, h_last, _ = (_rglru_fwd if _library_ops_active() else _RglruNode.apply)(
        x.contiguous(), u_r.contiguous(), u_i.contiguous(),
                              lam.to(torch.float32).contiguous(),
                              None if h0 is None else h0.to(torch.float32).contiguous(),
                              None if tok is None else tok.contiguous(), float(c), save)
    return y, h_last


# ----------------------------------------------------------------------------- raw affine scan
def _scan_fwd_impl(decay: Tensor, drive: Tensor, h0: Tensor) -> Tensor:
    lib = _lib.load()
    B, T, D = decay.shape
    out = torch.empty_like(drive)
    with _on(decay, "rglru_linear_scan_fwd"):
        rc = lib.rglru_linear_scan_fwd(_ptr(decay), _ptr(drive), _ptr(h0), _ptr(out), B, T, D, _stream(decay))
    _lib.check(rc, "rglru_linear_scan_fwd")
    return out


_scan_fwd = torch.library.custom_op("griffin_b200::linear_scan_fwd", _scan_fwd_impl, mutates_args=())


@_scan_fwd.register_fake
def _(decay, drive, h0):
    return torch.empty_like(drive)


def _scan_bwd_impl(d_out: Tensor, decay: Tensor, h0: Tensor, out: Tensor) -> tuple[Tensor, Tensor, Tensor]:
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


_scan_bwd = torch.library.custom_op("griffin_b200::linear_scan_bwd", _scan_bwd_impl, mutates_args=())


@_scan_bwd.register_fake
def _(d_out, decay, h0, out):
    return torch.empty_like(decay), torch.empty_like(decay), torch.empty_like(h0)


def _scan_setup(ctx, inputs, output):
    decay, _, h0 = inputs
    ctx.save_for_backward(decay, h0, output)


def _scan_backward(ctx, d_out, _bwd=None):
    decay, h0, out = ctx.saved_tensors
    if d_out is None:
        d_out = torch.zeros_like(out)
    return (_bwd or _scan_bwd)(d_out.contiguous(), decay, h0, out)


_scan_fwd.register_autograd(_scan_backward, setup_context=_scan_setup)
_ScanNode = _eager_node("LinearScan", _scan_fwd_impl, _scan_setup, _scan_backward, _scan_bwd_impl)


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
    return (_scan_fwd if _library_ops_active() else _ScanNode.apply)(
        decay.contiguous(), current_input.contiguous(), initial_state.contiguous())


# ----------------------------------------------------------------------------- causal conv
def _conv_fwd_impl(x_in: Tensor, w: Tensor, b: Optional[Tensor], state: Optional[Tensor], tok: Optional[Tensor],
                   want_state: bool = True) -> tuple[Tensor, Tensor]:
    """(conv output, next conv state [B,3,D]); without ``want_state`` the second result is empty and the small kernel
    that gathers it is not launched (a training step that keeps no cache has no use for it)."""
    lib = _lib.load()
    _require_cuda(x_in, w, b, state, tok)
    dt = _io_dtype(x_in, "conv")
    B, T, D = x_in.shape
    out = torch.empty_like(x_in)
    new_state = torch.empty((B, 3, D) if want_state else (0,), device=x_in.device, dtype=x_in.dtype)
    with _on(x_in, "rglru_conv_fwd"):
        rc = lib.rglru_conv_fwd(_ptr(x_in), _ptr(w), _ptr(b), _ptr(state), _ptr(tok), _ptr(out),
                                _ptr(new_state) if want_state else None, B, T, D, dt, _stream(x_in))
    _lib.check(rc, "rglru_conv_fwd")
    return out, new_state


_conv_fwd = torch.library.custom_op("griffin_b200::conv_fwd", _conv_fwd_impl, mutates_args=())


@_conv_fwd.register_fake
def _(x_in, w, b, state, tok, want_state=True):
    B, T, D = x_in.shape
    return torch.empty_like(x_in), x_in.new_empty((B, 3, D) if want_state else (0,))


def _conv_bwd_impl(d_conv: Tensor, x_in: Tensor, w: Tensor, state: Optional[Tensor], tok: Optional[Tensor],
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


_conv_bwd = torch.library.custom_op("griffin_b200::conv_bwd", _conv_bwd_impl, mutates_args=())


@_conv_bwd.register_fake
def _(d_conv, x_in, w, state, tok, want_state):
    B, T, D = x_in.shape
    return (torch.empty_like(x_in), x_in.new_empty((D, 4), dtype=torch.float32),
            x_in.new_empty((D,), dtype=torch.float32), x_in.new_empty((B, 3, D) if want_state else (0,)))


def _conv_setup(ctx, inputs, output):
    x_in, w, b, state, tok = inputs[:5]
    ctx.save_for_backward(x_in, w, state, tok)
    ctx.has_bias = b is not None
    ctx.want_state = state is not None and ctx.needs_input_grad[3]


def _conv_backward(ctx, d_out, _d_new_state, _bwd=None):
    x_in, w, state, tok = ctx.saved_tensors
    if d_out is None:
        d_out = torch.zeros_like(x_in)
    dx, d_w, d_b, d_state = (_bwd or _conv_bwd)(d_out.contiguous(), x_in, w, state, tok, ctx.want_state)
    return dx, d_w, (d_b if ctx.has_bias else None), (d_state if ctx.want_state else None), None, None


_conv_fwd.register_autograd(_conv_backward, setup_context=_conv_setup)
_ConvNode = _eager_node("CausalConv", _conv_fwd_impl, _conv_setup, _conv_backward, _conv_bwd_impl)


def causal_conv(x_in: Tensor, weight: Tensor, bias: Optional[Tensor], conv_state: Optional[Tensor] = None,
                tok: Optional[Tensor] = None, want_state: bool = True) -> tuple[Tensor, Tensor]:
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
    return (_conv_fwd if _library_ops_active() else _ConvNode.apply)(
        x_in.contiguous(), w, b, st, None if tok is None else tok.contiguous(), want_state)


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


def _merged_fwd_impl(x: Tensor, u_r: Tensor, u_i: Tensor, branch: Tensor, lam: Tensor, h0: Optional[Tensor],
                tok: Optional[Tensor], c: float, save: bool) -> tuple[Tensor, Tensor, Tensor]:
    return merge_scan_fwd(x, None, None, None, u_r, u_i, branch, lam, h0, tok, c, save)


_merged_fwd = torch.library.custom_op("griffin_b200::merged_fwd", _merged_fwd_impl, mutates_args=())


@_merged_fwd.register_fake
def _(x, u_r, u_i, branch, lam, h0, tok, c, save):
    B, T, D = x.shape
    return (torch.empty_like(x), x.new_empty((B, D), dtype=torch.float32),
            x.new_empty((workspace_bytes(B, T, D) if save else 0,), dtype=torch.uint8))


def _merged_bwd_impl(dout: Tensor, dh_last: Optional[Tensor], x: Tensor, u_r: Tensor, u_i: Tensor, branch: Tensor,
                lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor], ws: Tensor, c: float, want_dh0: bool
                ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    dx, du_r, du_i, dbranch, dlam, dh0 = merge_scan_bwd(dout, dh_last, x, None, None, None, u_r, u_i, branch, lam, h0,
                                                        tok, ws, c, want_dh0)
    return dx, du_r, du_i, dbranch, dlam, (dh0 if want_dh0 else x.new_empty((0,), dtype=torch.float32))


_merged_bwd = torch.library.custom_op("griffin_b200::merged_bwd", _merged_bwd_impl, mutates_args=())


@_merged_bwd.register_fake
def _(dout, dh_last, x, u_r, u_i, branch, lam, h0, tok, ws, c, want_dh0):
    B, T, D = x.shape
    return (torch.empty_like(x), torch.empty_like(x), torch.empty_like(x), torch.empty_like(x),
            x.new_empty((D,), dtype=torch.float32), x.new_empty((B, D) if want_dh0 else (0,), dtype=torch.float32))


def _merged_setup(ctx, inputs, output):
    x, u_r, u_i, branch, lam, h0, tok, c, save = inputs
    ctx.save_for_backward(x, u_r, u_i, branch, lam, h0, tok, output[2])
    ctx.c, ctx.saved = c, save
    ctx.want_dh0 = h0 is not None and ctx.needs_input_grad[5]


def _merged_backward(ctx, dout, dh_last, _dws, _bwd=None):
    if not ctx.saved:
        raise RuntimeError("merged scan was run without saving its workspace; backward is unavailable")
    x, u_r, u_i, branch, lam, h0, tok, ws = ctx.saved_tensors
    dout = torch.zeros_like(x) if dout is None else dout.to(x.dtype).contiguous()
    dh_last = None if dh_last is None else dh_last.to(torch.float32).contiguous()
    dx, du_r, du_i, dbranch, dlam, dh0 = (_bwd or _merged_bwd)(dout, dh_last, x, u_r, u_i, branch, lam, h0, tok, ws,
                                                               ctx.c, ctx.want_dh0)
    return dx, du_r, du_i, dbranch, dlam, (dh0 if ctx.want_dh0 else None), None, None, None


_merged_fwd.register_autograd(_merged_backward, setup_context=_merged_setup)
_MergedNode = _eager_node("MergedScan", _merged_fwd_impl, _merged_setup, _merged_backward, _merged_bwd_impl)


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
    save = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, u_r, u_i, branch, lam, h0))
    out, h_last, _ = (_merged_fwd if _library_ops_active() else _MergedNode.apply)(
        x.contiguous(), u_r.contiguous(), u_i.contiguous(), branch.to(x.dtype).contiguous(),
        lam.to(torch.float32).contiguous(), None if h0 is None else h0.to(torch.float32).contiguous(),
        None if tok is None else tok.contiguous(), float(c), save)
    return out, h_last


# ----------------------------------------------------------------------------- both gates from one grouped GEMM
def grouped_gates_supported(x: Tensor, gate_width: int) -> bool:
    """Whether the grouped gate layout can be used: CUDA, a gate head that is a whole number of 64-channel
    tiles, and rows the copy engine can address."""
    return x.is_cuda and gate_width % 64 == 0 and (x.shape[-1] * x.element_size()) % 16 == 0


def _aligned16(t: Optional[Tensor]) -> Optional[Tensor]:
    return t if t is None or t.data_ptr() % 16 == 0 else t.clone()


def _stacked_gates(x: Tensor, w_r: Tensor, b_r: Tensor, w_i: Tensor, b_i: Tensor) -> tuple[Tensor, Tensor]:
    """The two [G, bw, bw] gate weights stacked per head in the activation dtype, and the biases [2 D] fp32 in the
    same column layout."""
    wcat = torch.cat([w_r, w_i], dim=1).to(x.dtype)                                   # [G, 2 bw, bw]
    bias = torch.cat([b_r, b_i], dim=1).to(torch.float32).reshape(-1).contiguous()    # [2 D]
    return wcat, bias


def _grouped_fwd_impl(x: Tensor, w_r: Tensor, b_r: Tensor, w_i: Tensor, b_i: Tensor, lam: Tensor, h0: Optional[Tensor],
                 tok: Optional[Tensor], c: float, branch: Optional[Tensor], save: bool
                 ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Gate projections + RG-LRU (+ optional GeLU-branch product) around ONE grouped GEMM.

    The two [G, bw, bw] gate weights are stacked per head and a single batched GEMM writes both gate
    pre-activations straight into a [B, T, G, 2 bw] tensor (cuBLAS takes the strided output, so there is no
    re-layout pass); the kernels read that layout, add the biases themselves and return the gradient in the
    same layout, from which two more batched GEMMs give the input and weight gradients.
    Reference: BlockDiagonalLinear griffin/griffin.py:129-154 called twice at :237-238.
    Returns (out, h_last, the gate tensor u, the workspace, the stacked weights, the stacked biases); the last four
    are what the backward needs beside the inputs."""
    lib = _lib.load()
    with torch.autocast("cuda", enabled=False):
        x = _aligned16(x)
        B, T, D = x.shape
        G, bw, _ = w_r.shape
        dt = _io_dtype(x, "grouped forward")
        wcat, bias = _stacked_gates(x, w_r, b_r, w_i, b_i)
        rows = x.view(B * T, G, bw).transpose(0, 1)                                       # [G, N, bw] view
        u = torch.empty(B, T, 2 * D, device=x.device, dtype=x.dtype)
        torch.bmm(rows, wcat.transpose(1, 2), out=u.view(B * T, G, 2 * bw).transpose(0, 1))
        branch = _aligned16(branch)
        out = torch.empty_like(x)
        h_last = torch.empty(B, D, device=x.device, dtype=torch.float32)
        nbytes = lib.rglru_workspace_bytes(B, T, D, dt) if save else 0
        ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
        with _on(x, "rglru_grouped_fwd"):
            rc = lib.rglru_grouped_fwd(_ptr(x), _ptr(u), _ptr(bias), _ptr(branch), _ptr(lam), _ptr(h0), _ptr(tok),
                                       _ptr(out), _ptr(h_last), _ptr(ws) if save else None, nbytes, B, T, D, bw,
                                       c, dt, _stream(x))
        _lib.check(rc, "rglru_grouped_fwd")
    return out, h_last, u, ws, wcat, bias


_grouped_fwd = torch.library.custom_op("griffin_b200::grouped_fwd", _grouped_fwd_impl, mutates_args=())


@_grouped_fwd.register_fake
def _(x, w_r, b_r, w_i, b_i, lam, h0, tok, c, branch, save):
    B, T, D = x.shape
    G, bw, _ = w_r.shape
    return (torch.empty_like(x), x.new_empty((B, D), dtype=torch.float32), x.new_empty((B, T, 2 * D)),
            x.new_empty((workspace_bytes(B, T, D) if save else 0,), dtype=torch.uint8),
            x.new_empty((G, 2 * bw, bw)), x.new_empty((2 * D,), dtype=torch.float32))


def _grouped_bwd_impl(dout: Tensor, dh_last: Optional[Tensor], x: Tensor, u: Tensor, wcat: Tensor, bias: Tensor,
                 branch: Optional[Tensor], lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor],
                 ws: Tensor, c: float, want_dh0: bool
                 ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(dx, d stacked weights [G, 2 bw, bw], d stacked biases [G, 2 bw] fp32, dLambda, dh0, dbranch) from the stacked
    weights and biases the forward built; absent results are empty tensors.  The caller slices the two stacked
    gradients into the gates' own."""
    lib = _lib.load()
    with torch.autocast("cuda", enabled=False):
        x = _aligned16(x)
        B, T, D = x.shape
        G, bw2, bw = wcat.shape
        dt = _io_dtype(x, "grouped backward")
        dout = _aligned16(dout)
        branch = _aligned16(branch)
        dx = torch.empty_like(x)
        du = torch.empty_like(u)
        dbranch = torch.empty_like(x) if branch is not None else x.new_empty((0,))
        dlam = torch.empty(D, device=x.device, dtype=torch.float32)
        dh0 = torch.empty((B, D) if want_dh0 else (0,), device=x.device, dtype=torch.float32)
        dbias = torch.empty(G, bw2, device=x.device, dtype=torch.float32)    # [2 D] in the gate tensor's column layout
        with _on(x, "rglru_grouped_bwd"):
            rc = lib.rglru_grouped_bwd(_ptr(dout), _ptr(dh_last), _ptr(x), _ptr(u), _ptr(bias), _ptr(branch),
                                       _ptr(lam), _ptr(h0), _ptr(tok), _ptr(ws), ws.numel(), _ptr(dx), _ptr(du),
                                       _ptr(dbranch) if branch is not None else None, _ptr(dlam),
                                       _ptr(dh0) if want_dh0 else None, _ptr(dbias), B, T, D, bw, c, dt, _stream(x))
        _lib.check(rc, "rglru_grouped_bwd")
        dg = du.view(B * T, G, bw2).transpose(0, 1)                    # [G, N, 2 bw] view
        rows = x.view(B * T, G, bw).transpose(0, 1)                    # [G, N, bw] view
        dx.view(B * T, G, bw).transpose(0, 1).baddbmm_(dg, wcat)       # gate path added onto the direct path
        dwcat = torch.bmm(dg.transpose(1, 2), rows)                    # [G, 2 bw, bw]
    return dx, dwcat, dbias, dlam, dh0, dbranch


_grouped_bwd = torch.library.custom_op("griffin_b200::grouped_bwd", _grouped_bwd_impl, mutates_args=())


@_grouped_bwd.register_fake
def _(dout, dh_last, x, u, wcat, bias, branch, lam, h0, tok, ws, c, want_dh0):
    B, T, D = x.shape
    G, bw2, _ = wcat.shape
    return (torch.empty_like(x), torch.empty_like(wcat), x.new_empty((G, bw2), dtype=torch.float32),
            x.new_empty((D,), dtype=torch.float32), x.new_empty((B, D) if want_dh0 else (0,), dtype=torch.float32),
            torch.empty_like(x) if branch is not None else x.new_empty((0,)))


def _grouped_setup(ctx, inputs, output):
    x, w_r, b_r, w_i, b_i, lam, h0, tok, c, branch, save = inputs
    _, _, u, ws, wcat, bias = output
    ctx.save_for_backward(x, u, wcat, bias, branch, lam, h0, tok, ws)
    ctx.c, ctx.saved = c, save
    ctx.param_dtypes = (w_r.dtype, b_r.dtype, w_i.dtype, b_i.dtype)
    ctx.want_dh0 = h0 is not None and ctx.needs_input_grad[6]


def _grouped_backward(ctx, dout, dh_last, _du, _dws, _dwcat, _dbias, _bwd=None):
    if not ctx.saved:
        raise RuntimeError("grouped RG-LRU was run without saving its workspace; backward is unavailable")
    x, u, wcat, bias, branch, lam, h0, tok, ws = ctx.saved_tensors
    dout = torch.zeros_like(x) if dout is None else dout.to(x.dtype).contiguous()
    dh_last = None if dh_last is None else dh_last.to(torch.float32).contiguous()
    dx, dwcat, dbias, dlam, dh0, dbranch = (_bwd or _grouped_bwd)(
        dout, dh_last, x, u, wcat, bias, branch, lam, h0, tok, ws, ctx.c, ctx.want_dh0)
    bw = wcat.shape[2]
    dt_wr, dt_br, dt_wi, dt_bi = ctx.param_dtypes
    return (dx, dwcat[:, :bw].to(dt_wr), dbias[:, :bw].to(dt_br), dwcat[:, bw:].to(dt_wi), dbias[:, bw:].to(dt_bi),
            dlam, (dh0 if ctx.want_dh0 else None), None, None, (dbranch if branch is not None else None), None)


_grouped_fwd.register_autograd(_grouped_backward, setup_context=_grouped_setup)
_GroupedNode = _eager_node("GroupedRGLRU", _grouped_fwd_impl, _grouped_setup, _grouped_backward, _grouped_bwd_impl)


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
    save = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (x, w_r, b_r, w_i, b_i, lam, h0, branch))
    out, h_last, _, _, _, _ = (_grouped_fwd if _library_ops_active() else _GroupedNode.apply)(
        x.contiguous(), w_r, b_r, w_i, b_i, lam.to(torch.float32).contiguous(),
        None if h0 is None else h0.to(torch.float32).contiguous(), None if tok is None else tok.contiguous(), float(c),
        None if branch is None else branch.to(x.dtype).contiguous(), save)
    return out, h_last


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


def _core_fwd_impl(x_in: Tensor, conv_w: Tensor, conv_b: Optional[Tensor], conv_state: Optional[Tensor], w_r: Tensor,
              b_r: Tensor, w_i: Tensor, b_i: Tensor, lam: Tensor, h0: Optional[Tensor], tok: Optional[Tensor], c: float,
              branch: Optional[Tensor], save: bool) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """conv -> gate projections -> RG-LRU as one operator that keeps only the conv INPUT for its backward.

    The conv output is materialised once for the two gate GEMMs and dropped; the scan kernels read the conv
    input and redo the four taps in their load stage.  ``conv_w`` [D,4], ``conv_b``, ``lam``, ``h0`` fp32.
    Returns (y, h_last, next conv state, u_r, u_i, workspace)."""
    with torch.autocast("cuda", enabled=False):
        x_conv, new_state = _conv_fwd_impl(x_in, conv_w, conv_b, conv_state, tok)
        u_r = _gate(x_conv, w_r, b_r)
        u_i = _gate(x_conv, w_i, b_i)
        del x_conv
        if branch is None:
            y, h_last, ws = conv_scan_fwd(x_in, conv_w, conv_b, conv_state, u_r, u_i, lam, h0, tok, c, save)
        else:
            y, h_last, ws = merge_scan_fwd(x_in, conv_w, conv_b, conv_state, u_r, u_i, branch, lam, h0, tok, c, save)
    return y, h_last, new_state, u_r, u_i, ws


_core_fwd = torch.library.custom_op("griffin_b200::core_fwd", _core_fwd_impl, mutates_args=())


@_core_fwd.register_fake
def _(x_in, conv_w, conv_b, conv_state, w_r, b_r, w_i, b_i, lam, h0, tok, c, branch, save):
    B, T, D = x_in.shape
    return (torch.empty_like(x_in), x_in.new_empty((B, D), dtype=torch.float32), x_in.new_empty((B, 3, D)),
            torch.empty_like(x_in), torch.empty_like(x_in),
            x_in.new_empty((workspace_bytes(B, T, D) if save else 0,), dtype=torch.uint8))


def _core_bwd_impl(dy: Tensor, dh_last: Optional[Tensor], x_in: Tensor, conv_w: Tensor, conv_b: Optional[Tensor],
              conv_state: Optional[Tensor], w_r: Tensor, w_i: Tensor, lam: Tensor, h0: Optional[Tensor],
              tok: Optional[Tensor], u_r: Tensor, u_i: Tensor, ws: Tensor, branch: Optional[Tensor], c: float,
              want_dh0: bool, want_state: bool
              ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Backward of ``core_fwd``: recomputes the conv output (one streaming pass) for the gate-weight gradients,
    sums the direct and gate paths and runs a single conv backward.  Returns (dx_in, d conv_w, d conv_b,
    d conv_state, dw_r, db_r, dw_i, db_i, dLambda, dh0, dbranch); absent results are empty tensors."""
    with torch.autocast("cuda", enabled=False):
        empty = x_in.new_empty((0,))
        dbranch = empty
        if branch is None:
            dxc, du_r, du_i, dlam, dh0 = conv_scan_bwd(dy, dh_last, x_in, conv_w, conv_b, conv_state, u_r, u_i, lam, h0,
                                                       tok, ws, c, want_dh0)
        else:
            dxc, du_r, du_i, dbranch, dlam, dh0 = merge_scan_bwd(dy, dh_last, x_in, conv_w, conv_b, conv_state, u_r, u_i,
                                                                 branch, lam, h0, tok, ws, c, want_dh0)
        x_conv, _ = _conv_fwd_impl(x_in, conv_w, conv_b, conv_state, tok, False)     # recomputed, not saved
        dx_r, dw_r, db_r = _gate_backward(du_r, x_conv, w_r)
        dx_i, dw_i, db_i = _gate_backward(du_i, x_conv, w_i)
        total = (dxc + dx_r + dx_i).contiguous()
        dx_in, d_w, d_b, d_state = _conv_bwd_impl(total, x_in, conv_w, conv_state, tok, want_state)
    return (dx_in, d_w, d_b, d_state, dw_r, db_r, dw_i, db_i, dlam,
            dh0 if want_dh0 else x_in.new_empty((0,), dtype=torch.float32), dbranch)


_core_bwd = torch.library.custom_op("griffin_b200::core_bwd", _core_bwd_impl, mutates_args=())


@_core_bwd.register_fake
def _(dy, dh_last, x_in, conv_w, conv_b, conv_state, w_r, w_i, lam, h0, tok, u_r, u_i, ws, branch, c, want_dh0, want_state):
    B, T, D = x_in.shape
    g, wo, _ = w_r.shape
    f32 = torch.float32
    return (torch.empty_like(x_in), x_in.new_empty((D, 4), dtype=f32), x_in.new_empty((D,), dtype=f32),
            x_in.new_empty((B, 3, D) if want_state else (0,)), torch.empty_like(w_r), x_in.new_empty((g, wo), dtype=f32),
            torch.empty_like(w_i), x_in.new_empty((g, wo), dtype=f32), x_in.new_empty((D,), dtype=f32),
            x_in.new_empty((B, D) if want_dh0 else (0,), dtype=f32),
            torch.empty_like(x_in) if branch is not None else x_in.new_empty((0,)))


def _core_setup(ctx, inputs, output):
    x_in, conv_w, conv_b, conv_state, w_r, b_r, w_i, b_i, lam, h0, tok, c, branch, save = inputs
    _, _, new_state, u_r, u_i, ws = output
    ctx.save_for_backward(x_in, conv_w, conv_b, conv_state, w_r, w_i, lam, h0, tok, u_r, u_i, ws, branch)
    ctx.c, ctx.saved = c, save
    ctx.bias_dtypes = (b_r.dtype, b_i.dtype)
    ctx.want_dh0 = h0 is not None and ctx.needs_input_grad[9]
    ctx.want_state = conv_state is not None and ctx.needs_input_grad[3]
    ctx.mark_non_differentiable(new_state)


def _core_backward(ctx, dy, dh_last, _d_state, _du_r, _du_i, _dws, _bwd=None):
    if not ctx.saved:
        raise RuntimeError("recurrent core was run without saving its workspace; backward is unavailable")
    x_in, conv_w, conv_b, conv_state, w_r, w_i, lam, h0, tok, u_r, u_i, ws, branch = ctx.saved_tensors
    dy = torch.zeros_like(x_in) if dy is None else dy.to(x_in.dtype).contiguous()
    dh_last = None if dh_last is None else dh_last.to(torch.float32).contiguous()
    (dx_in, d_w, d_b, d_state, dw_r, db_r, dw_i, db_i, dlam, dh0, dbranch) = (_bwd or _core_bwd)(
        dy, dh_last, x_in, conv_w, conv_b, conv_state, w_r, w_i, lam, h0, tok, u_r, u_i, ws, branch, ctx.c,
        ctx.want_dh0, ctx.want_state)
    brdt, bidt = ctx.bias_dtypes
    return (dx_in, d_w, None if conv_b is None else d_b, d_state if ctx.want_state else None,
            dw_r, db_r.to(brdt), dw_i, db_i.to(bidt), dlam, (dh0 if ctx.want_dh0 else None), None, None,
            (dbranch if branch is not None else None), None)


_core_fwd.register_autograd(_core_backward, setup_context=_core_setup)
_CoreNode = _eager_node("RecurrentCore", _core_fwd_impl, _core_setup, _core_backward, _core_bwd_impl)


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
    save = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (x_in, conv_w, conv_b, conv_state, w_r, b_r, w_i, b_i, lam, h0, branch))
    y, h_last, new_state, _, _, _ = (_core_fwd if _library_ops_active() else _CoreNode.apply)(
        x_in.contiguous(), conv_w.to(torch.float32).contiguous(),
        None if conv_b is None else conv_b.to(torch.float32).contiguous(),
        None if conv_state is None else conv_state.to(x_in.dtype).contiguous(), w_r, b_r, w_i, b_i,
        lam.to(torch.float32).contiguous(), None if h0 is None else h0.to(torch.float32).contiguous(),
        None if tok is None else tok.contiguous(), float(c),
        None if branch is None else branch.to(x_in.dtype).contiguous(), save)
    return y, h_last, new_state


# ----------------------------------------------------------------------------- linear layers around the recurrence
def column_sums(m: Tensor) -> Tensor:
    """fp32 column sums of a dense [rows, cols] CUDA matrix (``rglru_column_sums``): fixed summation order, one
    streaming pass.  The bias gradient of a linear layer from the gradient of its output."""
    if m.dim() != 2:
        raise ValueError("column_sums takes a [rows, cols] matrix")
    _require_cuda(m)
    lib = _lib.load()
    dt = _io_dtype(m, "column sums")
    m = m.contiguous()
    rows, cols = m.shape
    out = torch.empty(cols, device=m.device, dtype=torch.float32)
    if rows == 0:
        return out.zero_()
    nbytes = lib.rglru_column_sums_workspace_bytes(rows, cols)
    ws = torch.empty(nbytes, device=m.device, dtype=torch.uint8)
    with _on(m, "rglru_column_sums"):
        rc = lib.rglru_column_sums(_ptr(m), _ptr(out), _ptr(ws), nbytes, rows, cols, dt, _stream(m))
    _lib.check(rc, "rglru_column_sums")
    return out


class _BiasGradTap(torch.autograd.Function):
    """Identity on the output of a linear layer that was computed with its bias detached; the backward hands the
    gradient through untouched and supplies the bias gradient from :func:`column_sums`.  The GEMMs and their
    backward stay autograd's own; only the generic reduction it would launch for the bias (a fifth of streaming
    bandwidth on [32768, 1024] bf16) is replaced."""

    @staticmethod
    def forward(ctx, y, bias):
        ctx.bias_dtype = bias.dtype
        return y.view_as(y)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        db = None
        if ctx.needs_input_grad[1]:
            db = column_sums(dy.reshape(-1, dy.shape[-1])).to(ctx.bias_dtype)
        return dy, db


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> Tensor:
    """``F.linear`` for the block's three projections (linear_x / linear_y / linear_out, griffin/griffin.py:379-389).
    Where a bias gradient is wanted on CUDA tensors of a kernel dtype, outside tracing, the bias gradient comes
    from :func:`column_sums`; everything else is ``F.linear`` itself."""
    tap = (bias is not None and bias.requires_grad and torch.is_grad_enabled() and x.is_cuda and x.numel() > 0
           and not _library_ops_active())
    if tap:
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        tap = out_dtype in _DTYPES
    if not tap:
        return torch.nn.functional.linear(x, weight, bias)
    y = torch.nn.functional.linear(x, weight, bias.detach())
    return _BiasGradTap.apply(y, bias)


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
