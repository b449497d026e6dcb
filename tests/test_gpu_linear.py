"""The column-sum kernel (rglru_column_sums) and the linear layer that takes its bias gradient from it, against
plain torch: the three projections of the recurrent block, griffin/griffin.py:379-389."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("rows,cols,dtype", [
    (32768, 768, torch.bfloat16),     # the block's output gradient at B=16 T=2048
    (32768, 1024, torch.bfloat16),
    (4096, 1024, torch.float32),
    (1000, 130, torch.float32),       # 520-byte rows: the scalar-column path
    (777, 72, torch.bfloat16),        # 144-byte rows, ragged row blocks
    (5, 64, torch.bfloat16),          # fewer rows than row lanes
    (1, 8, torch.float32),
    (70000, 8, torch.bfloat16),       # one column vector, many row blocks
])
def test_column_sums_match_a_float64_sum(rows, cols, dtype):
    from griffin_b200 import check_device, ops
    g = torch.Generator(device=DEV).manual_seed(rows + cols)
    m = (torch.randn(rows, cols, device=DEV, generator=g) + 0.25).to(dtype)
    got = ops.column_sums(m)
    want = m.double().sum(dim=0)
    assert got.dtype == torch.float32 and got.shape == (cols,)
    scale = m.double().abs().sum(dim=0).clamp_min(1.0)
    assert float(((got.double() - want).abs() / scale).max()) < 2e-6      # fp32 accumulation of exact inputs
    assert torch.equal(got, ops.column_sums(m))                            # fixed summation order
    check_device()


def test_column_sums_entry_point_stays_inside_its_tensors():
    from griffin_b200 import _lib
    lib = _lib.load()
    rows, cols, guard = 777, 72, 4096
    m = torch.randn(rows, cols, device=DEV).to(torch.bfloat16)
    need = lib.rglru_column_sums_workspace_bytes(rows, cols)
    out = torch.full((cols + 2 * guard,), 1024.0, device=DEV)
    ws = torch.full((need // 4 + 2 * guard,), 1024.0, device=DEV)
    rc = lib.rglru_column_sums(m.data_ptr(), out[guard:].data_ptr(), ws[guard:].data_ptr(), need, rows, cols, _lib.BF16,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert bool((out[:guard] == 1024.0).all()) and bool((out[guard + cols:] == 1024.0).all())
    assert bool((ws[:guard] == 1024.0).all()) and bool((ws[guard + need // 4:] == 1024.0).all())
    assert torch.allclose(out[guard:guard + cols], m.float().sum(dim=0), rtol=1e-4, atol=1e-2)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_linear_node_matches_functional_linear(dtype, tol):
    from griffin_b200 import ops
    torch.manual_seed(3)
    x = torch.randn(4, 300, 96, device=DEV).to(dtype).requires_grad_(True)
    w = (torch.randn(160, 96, device=DEV) / 10).to(dtype).requires_grad_(True)
    b = torch.randn(160, device=DEV).to(dtype).requires_grad_(True)
    dy = torch.randn(4, 300, 160, device=DEV).to(dtype)
    out = ops.linear(x, w, b)
    assert type(out.grad_fn).__name__ == "_BiasGradTapBackward"
    got = torch.autograd.grad(out, (x, w, b), dy)
    ref_out = F.linear(x, w, b)
    want = torch.autograd.grad(ref_out, (x, w, b), dy)
    assert torch.equal(out, ref_out)
    for a, r in zip(got, want):
        assert a.dtype == r.dtype and a.shape == r.shape
        assert float((a.float() - r.float()).norm() / r.float().norm().clamp_min(1e-12)) < tol
    # the bias gradient against a float64 sum: fp32 accumulation, then one rounding to the parameter's dtype
    exact = dy.double().sum(dim=(0, 1))
    scale = dy.double().abs().sum(dim=(0, 1))
    assert float(((got[2].double() - exact).abs() / scale).max()) < (2e-6 if dtype == torch.float32 else 4e-3)


def test_linear_node_under_autocast_returns_parameter_dtypes():
    from griffin_b200 import ops
    torch.manual_seed(4)
    x = torch.randn(2, 128, 64, device=DEV, requires_grad=True)
    w = (torch.randn(96, 64, device=DEV) / 8).requires_grad_(True)
    b = torch.randn(96, device=DEV, requires_grad=True)
    dy = torch.randn(2, 128, 96, device=DEV).to(torch.bfloat16)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = ops.linear(x, w, b)
        ref = F.linear(x, w, b)
    assert out.dtype == torch.bfloat16 and torch.equal(out, ref)
    got = torch.autograd.grad(out, (x, w, b), dy)
    want = torch.autograd.grad(ref, (x, w, b), dy)
    for a, r in zip(got, want):
        assert a.dtype == torch.float32
        assert float((a - r).norm() / r.norm()) < 1e-2


def test_linear_falls_back_to_functional_linear_where_the_node_does_not_apply():
    from griffin_b200 import ops
    x = torch.randn(2, 8, 16, device=DEV, requires_grad=True)
    w = torch.randn(4, 16, device=DEV, requires_grad=True)
    assert type(ops.linear(x, w, None).grad_fn).__name__ != "_BiasGradTapBackward"         # no bias
    with torch.no_grad():
        assert ops.linear(x, w, torch.zeros(4, device=DEV)).grad_fn is None
    xh = x.detach().half().requires_grad_(True)                                             # not a kernel dtype
    out = ops.linear(xh, w.detach().half().requires_grad_(True), torch.zeros(4, device=DEV).half().requires_grad_(True))
    assert type(out.grad_fn).__name__ != "_BiasGradTapBackward"


def test_block_with_a_replaced_projection_calls_the_replacement():
    from griffin_b200 import RecurrentBlock

    class Doubling(torch.nn.Linear):
        def forward(self, x):
            return 2.0 * super().forward(x)

    torch.manual_seed(5)
    blk = RecurrentBlock(32, 64, gate_blocks=1).to(DEV)
    x = torch.randn(2, 20, 32, device=DEV)
    base = blk(x)
    swapped = Doubling(64, 32).to(DEV)
    swapped.load_state_dict(blk.linear_out.state_dict())
    blk.linear_out = swapped
    assert torch.allclose(blk(x), 2.0 * base, rtol=1e-5, atol=1e-6)
    seen = []
    blk.linear_x.register_forward_hook(lambda m, i, o: seen.append(o.shape))
    blk(x)
    assert seen == [torch.Size([2, 20, 64])]
