"""The differentiable operators as ``torch.library`` custom ops: shape inference without a device (CPU), and on
the GPU ``torch.library.opcheck``, ``torch.compile(fullgraph=True)`` and agreement with the eager
``torch.autograd.Function`` route that ordinary calls take."""

from __future__ import annotations

import pytest
import torch

from oracle.rglru_oracle import rel_l2


@pytest.mark.parametrize("kw", [{}, {"fold_merge": True}, {"fold_conv": True}, {"fold_conv": True, "fold_merge": True}])
def test_block_traces_with_fake_cuda_tensors_on_a_box_without_a_gpu(kw):
    """Every operator the block reaches has a fake implementation with the real output shapes and dtypes, so the
    forward runs on fake CUDA tensors (no device, no library call): what a tracing compiler relies on."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from griffin_b200 import RecurrentBlock, ops
    with FakeTensorMode():
        with torch.device("cuda"):
            blk = RecurrentBlock(32, 128, gate_blocks=2, **kw)
            x = torch.randn(2, 70, 32, requires_grad=True)
        with ops.library_ops():
            out, cache = blk(x, return_cache=True)
    assert out.shape == (2, 70, 32) and out.dtype == torch.float32 and out.grad_fn is not None
    assert cache.rnn_state.shape == (2, 128) and cache.rnn_state.dtype == torch.float32
    assert cache.conv_state.shape == (2, 3, 128) and cache.conv_state.dtype == torch.float32


def test_backward_ops_infer_shapes_without_a_gpu():
    from torch._subclasses.fake_tensor import FakeTensorMode

    from griffin_b200 import ops
    B, T, D, G = 2, 70, 128, 2
    with FakeTensorMode():
        with torch.device("cuda"):
            x, u = torch.randn(B, T, D), torch.randn(B, T, 2 * D)
            w, b, lam = torch.randn(G, 64, 64), torch.randn(G, 64), torch.randn(D)
            ws = torch.empty(ops.workspace_bytes(B, T, D), dtype=torch.uint8)
            h0 = torch.randn(B, D)
            wcat, bcat = torch.randn(G, 128, 64), torch.randn(2 * D)
            got = ops._grouped_bwd(x, None, x, u, wcat, bcat, x, lam, h0, None, ws, 8.0, True)
            assert [tuple(t.shape) for t in got] == [(B, T, D), (G, 128, 64), (G, 128), (D,), (B, D), (B, T, D)]
            got = ops._core_bwd(x, None, x, torch.randn(D, 4), torch.randn(D), torch.randn(B, 3, D), w, w, lam, None, None,
                                x, x, ws, None, 8.0, False, True)
            assert [tuple(t.shape) for t in got] == [(B, T, D), (D, 4), (D,), (B, 3, D), (G, 64, 64), (G, 64), (G, 64, 64),
                                                     (G, 64), (D,), (0,), (0,)]
            y, h_last, ws2 = ops._rglru_fwd(x, x, x, lam, None, None, 8.0, True)
            assert ws2.numel() == ops.workspace_bytes(B, T, D) and h_last.shape == (B, D)
            assert ops._rglru_fwd(x, x, x, lam, None, None, 8.0, False)[2].numel() == 0


@pytest.mark.gpu
def test_opcheck_on_the_registered_operators():
    from griffin_b200 import ops
    from griffin_b200.modules import token_flags
    torch.manual_seed(0)
    B, T, D = 2, 70, 128
    dev = "cuda"
    x, u_r, u_i = (torch.randn(B, T, D, device=dev, requires_grad=True) for _ in range(3))
    lam = torch.randn(D, device=dev, requires_grad=True)
    h0 = torch.randn(B, D, device=dev, requires_grad=True)
    tok = token_flags(B, T, dev, reset=torch.zeros(B, T, dtype=torch.bool, device=dev))
    tests = ("test_schema", "test_faketensor", "test_autograd_registration")
    torch.library.opcheck(ops._rglru_fwd, (x, u_r, u_i, lam, h0, tok, 8.0, True), test_utils=tests)
    w = torch.randn(D, 4, device=dev, requires_grad=True)
    bias = torch.randn(D, device=dev, requires_grad=True)
    torch.library.opcheck(ops._conv_fwd, (x, w, bias, None, tok, True), test_utils=tests)
    decay = torch.rand(B, T, D, device=dev, requires_grad=True)
    torch.library.opcheck(ops._scan_fwd, (decay, x, h0), test_utils=tests)
    branch = torch.randn(B, T, D, device=dev, requires_grad=True)
    torch.library.opcheck(ops._merged_fwd, (x, u_r, u_i, branch, lam, h0, tok, 8.0, True), test_utils=tests)
    gw = torch.randn(2, 64, 64, device=dev, requires_grad=True)
    gb = torch.randn(2, 64, device=dev, requires_grad=True)
    torch.library.opcheck(ops._grouped_fwd, (x, gw, gb, gw, gb, lam, h0, tok, 8.0, branch, True), test_utils=tests)
    torch.library.opcheck(ops._core_fwd, (x, w, bias, None, gw, gb, gw, gb, lam, h0, tok, 8.0, branch, True),
                          test_utils=tests)


@pytest.mark.gpu
@pytest.mark.parametrize("kw", [{}, {"fold_merge": True}, {"fold_conv": True, "fold_merge": True}])
def test_compiled_block_matches_eager(kw):
    """torch.compile(fullgraph=True) traces the block through the custom ops without a graph break and gives the
    values and gradients of the eager route (the autograd.Function twins over the same kernels)."""
    from griffin_b200 import RecurrentBlock
    torch.manual_seed(3)
    blk = RecurrentBlock(32, 128, gate_blocks=2, **kw).cuda()
    x = torch.randn(2, 70, 32, device="cuda")
    dout = torch.randn(2, 70, 32, device="cuda")

    def run(fn):
        blk.zero_grad(set_to_none=True)
        xi = x.clone().requires_grad_(True)
        out = fn(xi)
        (out * dout).sum().backward()
        return [out.detach(), xi.grad] + [p.grad.clone() for p in blk.parameters()]

    eager = run(blk)
    compiled = run(torch.compile(blk, fullgraph=True, backend="aot_eager"))
    for a, b in zip(compiled, eager):
        assert rel_l2(a, b) <= 1e-6


@pytest.mark.gpu
def test_block_called_first_under_inference_mode_then_trained():
    """The token flags shared between calls of one shape must not be an inference tensor (it is saved for
    backward by later training calls) and must be valid on whatever stream the later calls run."""
    from griffin_b200 import RecurrentBlock
    from griffin_b200 import modules
    modules._PLAIN_FLAGS.clear()
    torch.manual_seed(4)
    blk = RecurrentBlock(16, 64, gate_blocks=1).cuda()
    x = torch.randn(3, 21, 16, device="cuda")
    with torch.inference_mode():
        first = blk(x)
    xi = x.clone().requires_grad_(True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        out = blk(xi)
        out.sum().backward()
    torch.cuda.current_stream().wait_stream(side)
    assert rel_l2(out, first) <= 1e-6 and torch.isfinite(xi.grad).all()
    assert not any(t.is_inference() for t in modules._PLAIN_FLAGS.values())


def test_linear_is_functional_linear_off_the_gpu_and_under_tracing():
    """ops.linear only taps the bias gradient for CUDA tensors outside tracing; everywhere else it is F.linear."""
    from griffin_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(3, 5, 8, requires_grad=True)
    w = torch.randn(4, 8, requires_grad=True)
    b = torch.randn(4, requires_grad=True)
    out = ops.linear(x, w, b)
    assert "BiasGradTap" not in type(out.grad_fn).__name__
    ref = torch.nn.functional.linear(x, w, b)
    assert torch.equal(out, ref)
    got = torch.autograd.grad(out.sum(), (x, w, b))
    want = torch.autograd.grad(ref.sum(), (x, w, b))
    for a, r in zip(got, want):
        assert torch.equal(a, r)
    with ops.library_ops():
        assert "BiasGradTap" not in type(ops.linear(x, w, b).grad_fn).__name__
    with pytest.raises(RuntimeError):
        ops.column_sums(torch.zeros(4, 4))           # the kernel has no CPU path
    with pytest.raises(ValueError):
        ops.column_sums(torch.zeros(4))
