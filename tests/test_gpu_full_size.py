"""Parity and size-independent properties at the benchmark's full sizes.

The reference's own backward is O(T^2) on CPU, so at these sizes the oracle's O(T) closed-form backward
(validated against the reference's autograd on the golden cases) is the checker; channels and batch rows
are independent recurrences, so a channel slab of a large problem can be checked on its own.
"""

from __future__ import annotations

import pytest
import torch

from oracle import rglru_oracle as orc
from oracle.rglru_oracle import rel_l2 as rel_l2_

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16_REL = 2e-2
FP32_REL = 1e-5


def _inputs(B, T, D, dtype, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    mk = lambda: torch.randn(B, T, D, device=DEV, generator=gen).to(dtype)
    cpu_gen = torch.Generator().manual_seed(seed)
    lam = orc.init_lambda(D, 8.0, cpu_gen).to(DEV)
    return mk(), mk(), mk(), mk(), lam


def _run(x, u_r, u_i, dy, lam, h0=None, dh=None):
    from griffin_b200 import ops
    xs = [t.detach().clone().requires_grad_(True) for t in (x, u_r, u_i)]
    lam = lam.detach().clone().requires_grad_(True)
    y, h_last = ops.rglru(xs[0], xs[1], xs[2], lam, h0)
    loss = (y.float() * dy.float()).sum()
    if dh is not None:
        loss = loss + (h_last * dh).sum()
    loss.backward()
    return {"y": y.detach(), "h_last": h_last.detach(), "dx": xs[0].grad, "du_r": xs[1].grad, "du_i": xs[2].grad,
            "dLambda": lam.grad}


def _oracle_slab(x, u_r, u_i, dy, lam, sl, rows):
    cut = lambda t: t[rows, :, sl].double().cpu()
    return orc.rglru_backward_linear(cut(x), cut(u_r), cut(u_i), lam[sl].double().cpu(), cut(dy))


def test_layer_full_shape_bf16_against_oracle():
    """bf16 I/O, B=8, T=2048, D=1024 (the benchmark's headline shape) -- every output and gradient, all channels."""
    x, u_r, u_i, dy, lam = _inputs(8, 2048, 1024, torch.bfloat16, 1)
    got = _run(x, u_r, u_i, dy, lam)
    want = _oracle_slab(x, u_r, u_i, dy, lam, slice(None), slice(None))
    for key in ("y", "h_last", "dx", "du_r", "du_i", "dLambda"):
        err = orc.rel_l2(got[key], want[key])
        assert err <= BF16_REL, (key, err)


def test_layer_full_shape_fp32_against_oracle():
    """The same shape with fp32 I/O (what the RG-LRU sees inside the 100M model): 1e-5 on everything,
    including dLambda, a 16384-term reduction per channel."""
    x, u_r, u_i, dy, lam = _inputs(8, 2048, 1024, torch.float32, 2)
    got = _run(x, u_r, u_i, dy, lam)
    want = _oracle_slab(x, u_r, u_i, dy, lam, slice(None), slice(None))
    for key in ("y", "h_last", "dx", "du_r", "du_i", "dLambda"):
        err = orc.rel_l2(got[key], want[key])
        assert err <= FP32_REL, (key, err)


@pytest.mark.parametrize("fold_merge", [False, True])
def test_recurrent_block_full_shape_bf16_against_oracle(fold_merge):
    """The whole recurrent block at B=16, T=2048, 768 -> 1024 -> 768 in bf16 (conv weights ~ N(0, 1/4), input
    ~ N(0, 1)), with and without the GeLU-branch product folded into the scan kernels: output, input gradient and
    every parameter gradient of all 16 rows against the oracle block (griffin/griffin.py:439-529 of the
    reference) evaluated in fp32 on the bf16-rounded parameters.  The oracle differentiates the scan with its
    O(T) closed form, which tests/test_oracle_golden.py holds to the reference's autograd."""
    from griffin_b200 import RecurrentBlock
    torch.manual_seed(5)
    B, T, DM, DR = 16, 2048, 768, 1024
    blk = RecurrentBlock(DM, DR, gate_blocks=16, scan_mode="cuda", fold_merge=fold_merge)
    with torch.no_grad():
        blk.temporal_conv.weight.normal_(0.0, 0.5)
    blk = blk.to(torch.bfloat16)
    params = {k: v.detach().float().clone().requires_grad_(True) for k, v in blk.state_dict().items()}
    x = torch.randn(B, T, DM).to(torch.bfloat16)
    dout = torch.randn(B, T, DM).to(torch.bfloat16)
    xr = x.float().requires_grad_(True)
    ref, ref_cache = orc.recurrent_block(xr, params, linear_backward=True)
    (ref * dout.float()).sum().backward()

    blk = blk.to(DEV)
    xg = x.to(DEV).requires_grad_(True)
    out, cache = blk(xg, return_cache=True)
    (out.float() * dout.to(DEV).float()).sum().backward()
    errs = {"out": orc.rel_l2(out, ref), "dx": orc.rel_l2(xg.grad, xr.grad),
            "rnn_state": orc.rel_l2(cache.rnn_state, ref_cache.rnn_state),
            "conv_state": orc.rel_l2(cache.conv_state, ref_cache.conv_state)}
    for key, p in blk.named_parameters():
        errs["g." + key] = orc.rel_l2(p.grad, params[key].grad)
    bad = {k: v for k, v in errs.items() if not v <= BF16_REL}
    assert not bad, (bad, errs)
    assert torch.equal(cache.segment_position.cpu(), ref_cache.segment_position)


def test_long_wide_slab_and_properties():
    """Long and wide geometry (T=8192, D=5632, bf16) at B=2: a 256-channel slab against the oracle, plus
    properties that need no oracle: time-chunked == whole, backward is linear in the upstream gradient,
    rows are independent, repeated runs are bit-identical."""
    from griffin_b200 import ops
    B, T, D = 2, 8192, 5632
    x, u_r, u_i, dy, lam = _inputs(B, T, D, torch.bfloat16, 3)
    got = _run(x, u_r, u_i, dy, lam)
    sl = slice(2048, 2304)
    want = _oracle_slab(x, u_r, u_i, dy, lam, sl, slice(0, 1))
    for key in ("y", "dx", "du_r", "du_i"):
        err = orc.rel_l2(got[key][0:1, :, sl], want[key])
        assert err <= BF16_REL, (key, err)
    assert orc.rel_l2(got["h_last"][0:1, sl], want["h_last"]) <= BF16_REL

    with torch.no_grad():
        # whole == two time chunks with the fp32 state carried across
        cutp = 3000
        ya, ha = ops.rglru(x[:, :cutp].contiguous(), u_r[:, :cutp].contiguous(), u_i[:, :cutp].contiguous(), lam)
        yb, hb = ops.rglru(x[:, cutp:].contiguous(), u_r[:, cutp:].contiguous(), u_i[:, cutp:].contiguous(), lam, ha)
        assert orc.rel_l2(torch.cat([ya, yb], 1), got["y"]) <= 4e-3      # bf16 outputs, fp32 state
        assert orc.rel_l2(hb, got["h_last"]) <= 1e-5
        # batch rows are independent: with the two rows swapped, each row's results are the same bits
        ys, hs = ops.rglru(x.flip(0).contiguous(), u_r.flip(0).contiguous(), u_i.flip(0).contiguous(), lam)
        assert torch.equal(ys.flip(0), got["y"]) and torch.equal(hs.flip(0), got["h_last"])
        # and a row on its own (which may run a different kernel shape) agrees to rounding
        y1, h1 = ops.rglru(x[1:2].contiguous(), u_r[1:2].contiguous(), u_i[1:2].contiguous(), lam)
        assert rel_l2_(y1, got["y"][1:2]) <= 2e-3 and rel_l2_(h1, got["h_last"][1:2]) <= 1e-5
    # determinism and linearity of the backward in dy
    again = _run(x, u_r, u_i, dy, lam)
    for key in got:
        assert torch.equal(again[key], got[key]), key
    doubled = _run(x, u_r, u_i, (2 * dy.float()).to(torch.bfloat16), lam)
    for key in ("dx", "du_r", "du_i", "dLambda"):
        assert orc.rel_l2(doubled[key].float(), 2 * got[key].float()) <= 4e-3, key


def test_decode_steps_at_batch_512_against_sequence_kernel():
    """Decode geometry (B=512, D=5632, bf16, fp32 carried state): 16 single-token updates equal
    one 16-step sequence call, and the first step equals the oracle."""
    from griffin_b200 import ops
    B, D, S = 512, 5632, 16
    x, u_r, u_i, _, lam = _inputs(B, S, D, torch.bfloat16, 4)
    h = torch.zeros(B, D, device=DEV)
    ys = []
    for t in range(S):
        ys.append(ops.decode_step(x[:, t].contiguous(), u_r[:, t].contiguous(), u_i[:, t].contiguous(), lam, h))
    with torch.no_grad():
        y_seq, h_seq = ops.rglru(x, u_r, u_i, lam)
    assert orc.rel_l2(torch.stack(ys, 1), y_seq) <= 4e-3
    assert orc.rel_l2(h, h_seq) <= 2e-3      # decode gates use ex2/rcp, the sequence kernel the tanh unit
    rows = slice(0, 4)
    y_ref, h_ref = orc.rglru_core(x[rows, :1].float().cpu(), u_r[rows, :1].float().cpu(), u_i[rows, :1].float().cpu(),
                                  lam.cpu())
    assert orc.rel_l2(ys[0][rows], y_ref[:, 0]) <= BF16_REL
