"""GPU parity of the conv, the cached recurrent block and single-token decode against the
reference's stored results (tests/golden, written by the unmodified reference) and the CPU oracle."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, params_of
from oracle import rglru_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP32_REL = 1e-5
BF16_REL = 2e-2


def _block(case, input_dim, width, blocks=16, dtype=torch.float32):
    from griffin_b200 import RecurrentBlock
    blk = RecurrentBlock(input_dim, width, gate_blocks=blocks, scan_mode="cuda")
    blk.load_state_dict(params_of(case))
    return blk.to(DEV, dtype).eval()


def _cache_to(cache):
    return cache


def test_chunked_prefill_matches_full_and_reference():
    """tests/test_recurrentblock.py:33-50 of the reference: chunks 3/4/2 carry conv history and RNN state."""
    case = load_golden("block_chunked")
    blk = _block(case, 8, 12)
    x = case["x"].to(DEV)
    with torch.no_grad():
        full = blk(x)
        a, c1 = blk(x[:, :3], return_cache=True)
        b, c2 = blk(x[:, 3:7], c1, return_cache=True)
        c, c3 = blk(x[:, 7:], c2, return_cache=True)
    torch.testing.assert_close(full.cpu(), case["full"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(torch.cat([a, b, c], 1).cpu(), case["chunks"], atol=2e-6, rtol=2e-5)
    for tag, cache in (("c1", c1), ("c2", c2), ("c3", c3)):
        torch.testing.assert_close(cache.rnn_state.cpu(), case[f"{tag}.rnn"], atol=2e-6, rtol=2e-5)
        torch.testing.assert_close(cache.conv_state.cpu(), case[f"{tag}.conv"], atol=1e-6, rtol=1e-6)
        assert torch.equal(cache.segment_position.cpu(), case[f"{tag}.pos"])
        assert cache.rnn_state.dtype == torch.float32


def test_document_reset_inside_sequence():
    case = load_golden("block_reset")
    blk = _block(case, 8, 16, 4)
    with torch.no_grad():
        out, cache = blk(case["x"].to(DEV), segment_pos=case["segment_pos"].to(DEV), return_cache=True)
    torch.testing.assert_close(out.cpu(), case["full"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(cache.rnn_state.cpu(), case["rnn"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(cache.conv_state.cpu(), case["conv"], atol=1e-6, rtol=1e-6)
    assert torch.equal(cache.segment_position.cpu(), case["pos"])
    # cached continuation across the reset equals the full run
    seg = case["segment_pos"].to(DEV)
    x = case["x"].to(DEV)
    with torch.no_grad():
        first, c1 = blk(x[:, :6], segment_pos=seg[:, :6], return_cache=True)
        second, _ = blk(x[:, 6:], c1, seg[:, 6:], return_cache=True)
    torch.testing.assert_close(torch.cat([first, second], 1).cpu(), case["full"], atol=2e-6, rtol=2e-5)


def test_right_padded_prefill_then_decode():
    case = load_golden("block_padded")
    blk = _block(case, 8, 16, 4)
    with torch.no_grad():
        pre, c1 = blk(case["x"].to(DEV), active_mask=case["active"].to(DEV), return_cache=True)
        dec, c2 = blk(case["next"].to(DEV), c1, return_cache=True)
    torch.testing.assert_close(pre.cpu(), case["prefill"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(dec.cpu(), case["decode"], atol=2e-6, rtol=2e-5)
    for tag, cache in (("c1", c1), ("c2", c2)):
        torch.testing.assert_close(cache.rnn_state.cpu(), case[f"{tag}.rnn"], atol=2e-6, rtol=2e-5)
        torch.testing.assert_close(cache.conv_state.cpu(), case[f"{tag}.conv"], atol=1e-6, rtol=1e-6)
        assert torch.equal(cache.segment_position.cpu(), case[f"{tag}.pos"])


@pytest.mark.parametrize("fold", [False, True])
def test_padding_that_is_not_right_padding(fold):
    """Left padding and holes, two cached chunks, and the gradients of the first (griffin/griffin.py:488-510)."""
    case = load_golden("block_ragged")
    blk = _block(case, 8, 16, 4)
    blk.fold_conv = fold
    x = case["x"].to(DEV).requires_grad_(True)
    first, c1 = blk(x, active_mask=case["active"].to(DEV), return_cache=True)
    (first * case["dout"].to(DEV)).sum().backward()
    with torch.no_grad():
        second, c2 = blk(case["x2"].to(DEV), c1, active_mask=case["active2"].to(DEV), return_cache=True)
    torch.testing.assert_close(first.detach().cpu(), case["first"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(second.cpu(), case["second"], atol=2e-6, rtol=2e-5)
    assert orc.rel_l2(x.grad.cpu(), case["dx"]) <= 1e-5
    for tag, cache in (("c1", c1), ("c2", c2)):
        torch.testing.assert_close(cache.rnn_state.detach().cpu(), case[f"{tag}.rnn"], atol=2e-6, rtol=2e-5)
        torch.testing.assert_close(cache.conv_state.detach().cpu(), case[f"{tag}.conv"], atol=1e-6, rtol=1e-6)
        assert torch.equal(cache.segment_position.cpu(), case[f"{tag}.pos"])
    grads = dict(blk.named_parameters())
    for key in case:
        if key.startswith("g."):
            assert orc.rel_l2(grads[key[2:]].grad.cpu(), case[key]) <= 1e-5, key


def test_token_by_token_decode_matches_full():
    """tests/test_griffin_model.py:87-118 family at the block level, plus the dedicated decode kernels."""
    from griffin_b200 import ops
    case = load_golden("block_decode")
    blk = _block(case, 8, 16, 4)
    x = case["x"].to(DEV)
    cache = None
    outs = []
    with torch.no_grad():
        for t in range(x.shape[1]):
            o, cache = blk(x[:, t : t + 1], cache, return_cache=True)
            outs.append(o)
            torch.testing.assert_close(cache.rnn_state.cpu(), case["rnn"][t], atol=2e-6, rtol=2e-5)
            torch.testing.assert_close(cache.conv_state.cpu(), case["conv"][t], atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(torch.cat(outs, 1).cpu(), case["steps"], atol=2e-6, rtol=2e-5)

    # the in-place single-token kernels give the same trajectory
    B, T, _ = x.shape
    D = 16
    h = torch.zeros(B, D, device=DEV)
    conv_state = torch.zeros(B, 3, D, device=DEV)
    w = blk.temporal_conv.weight[:, 0, :].float().contiguous()
    bias = blk.temporal_conv.bias.float().contiguous()
    lam = blk.rg_lru.Lambda.float().contiguous()
    outs = []
    with torch.no_grad():
        for t in range(T):
            flag = torch.full((B,), (3 - min(t, 3)) | (4 if t == 0 else 0), device=DEV, dtype=torch.uint8)
            gate = torch.nn.functional.gelu(blk.linear_y(x[:, t]), approximate="tanh")
            xc = ops.decode_conv(blk.linear_x(x[:, t]), w, bias, conv_state, flag)
            y = ops.decode_step(xc, blk.rg_lru.recurrence_gate(xc), blk.rg_lru.input_gate(xc), lam, h, flag)
            outs.append(blk.linear_out(y * gate))
            torch.testing.assert_close(h.cpu(), case["rnn"][t], atol=2e-6, rtol=2e-5)
            torch.testing.assert_close(conv_state.cpu(), case["conv"][t], atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(torch.stack(outs, 1).cpu(), case["steps"], atol=2e-6, rtol=2e-5)


def test_block_forward_backward_all_gradients():
    """Whole block with conv weights ~ N(0, 1/4): output, dx and every parameter gradient."""
    case = load_golden("block_grads")
    blk = _block(case, 16, 32, 4).train()
    x = case["x"].to(DEV).requires_grad_(True)
    out = blk(x)
    (out * case["dout"].to(DEV)).sum().backward()
    assert orc.rel_l2(out, case["out"]) <= FP32_REL
    assert orc.rel_l2(x.grad, case["dx"]) <= FP32_REL
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad, case["g." + key]) <= FP32_REL, key


# the last two shapes have enough (row, channel tile) pairs for the TMA-staged conv kernels
@pytest.mark.parametrize("shape", [(2, 70, 64), (3, 37, 20), (1, 300, 136), (2, 5, 7), (10, 70, 960), (19, 133, 520)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv_forward_backward_against_oracle(shape, dtype):
    """Conv alone with a carried state, document boundaries, and gradients incl. the state's."""
    from griffin_b200 import ops
    from griffin_b200.modules import token_flags
    B, T, D = shape
    gen = torch.Generator().manual_seed(T + D)
    x_in = torch.randn(B, T, D, generator=gen).to(dtype)
    w = torch.randn(D, 4, generator=gen) * 0.5
    b = torch.randn(D, generator=gen) * 0.1
    state = torch.randn(B, 3, D, generator=gen).to(dtype)
    dout = torch.randn(B, T, D, generator=gen).to(dtype)
    seg = torch.arange(T)[None, :].repeat(B, 1) + 2     # continues a document: two earlier tokens exist
    if T > 8:
        seg[:, T // 2 :] = torch.arange(T - T // 2)      # a new document starts mid-sequence
    xr = x_in.double().requires_grad_(True)
    wr = w.double().requires_grad_(True)
    br = b.double().requires_grad_(True)
    sr = state.double().requires_grad_(True)
    ref, ref_state = orc.causal_conv_dense(xr, wr, br, sr, seg)
    (ref * dout.double()).sum().backward()

    xg = x_in.to(DEV).requires_grad_(True)
    wg = w.to(DEV).requires_grad_(True)
    bg = b.to(DEV).requires_grad_(True)
    sg = state.to(DEV).requires_grad_(True)
    flags = token_flags(B, T, DEV, segment_pos=seg.to(DEV))
    out, new_state = ops.causal_conv(xg, wg, bg, sg, flags)
    (out.float() * dout.to(DEV).float()).sum().backward()
    tol = FP32_REL if dtype == torch.float32 else BF16_REL
    assert orc.rel_l2(out, ref) <= tol
    assert orc.rel_l2(new_state, ref_state) <= tol
    assert orc.rel_l2(xg.grad, xr.grad) <= tol
    assert orc.rel_l2(wg.grad, wr.grad) <= tol
    assert orc.rel_l2(bg.grad, br.grad) <= tol
    assert orc.rel_l2(sg.grad, sr.grad) <= tol


def test_block_bf16_against_fp32_oracle():
    """Config-2 style block in bf16 (reduced size) against the oracle on bf16-rounded weights."""
    from griffin_b200 import RecurrentBlock
    torch.manual_seed(11)
    blk = RecurrentBlock(48, 128, gate_blocks=4, scan_mode="cuda")
    with torch.no_grad():
        blk.temporal_conv.weight.normal_(0.0, 0.5)
    blk = blk.to(torch.bfloat16)
    params = {k: v.detach().float().clone().requires_grad_(True) for k, v in blk.state_dict().items()}
    x = torch.randn(2, 150, 48).to(torch.bfloat16)
    dout = torch.randn(2, 150, 48).to(torch.bfloat16)
    xr = x.float().requires_grad_(True)
    ref, _ = orc.recurrent_block(xr, params)
    (ref * dout.float()).sum().backward()
    blk = blk.to(DEV)
    xg = x.to(DEV).requires_grad_(True)
    out = blk(xg)
    (out.float() * dout.to(DEV).float()).sum().backward()
    assert orc.rel_l2(out, ref) <= BF16_REL
    assert orc.rel_l2(xg.grad, xr.grad) <= BF16_REL
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad, params[key].grad) <= 3e-2, key


@pytest.mark.parametrize("fold_merge", [False, True])
def test_wide_batch_block_with_padding_and_cache_against_oracle(fold_merge):
    """A batch wide enough for the TMA-staged conv kernels: right padding, ragged padding in one row, a carried
    cache into a second chunk, and all gradients, against the oracle block (griffin/griffin.py:439-529)."""
    from griffin_b200 import RecurrentBlock
    torch.manual_seed(21)
    B, T, DM, DR = 20, 70, 32, 512
    blk = RecurrentBlock(DM, DR, gate_blocks=8, scan_mode="cuda", fold_merge=fold_merge)
    with torch.no_grad():
        blk.temporal_conv.weight.normal_(0.0, 0.5)
        blk.temporal_conv.bias.normal_(0.0, 0.1)
    params = {k: v.detach().clone().requires_grad_(True) for k, v in blk.state_dict().items()}
    x, x2 = torch.randn(B, T, DM), torch.randn(B, 9, DM)
    dout = torch.randn(B, T, DM)
    active = torch.ones(B, T, dtype=torch.bool)
    for r in range(B):
        active[r, T - 3 * r:] = False if r else True        # row r ends 3 r tokens early (row 0 is full)
    active[5, 10:14] = False                                  # a hole: not right padding
    active2 = torch.ones(B, 9, dtype=torch.bool)
    active2[3, 6:] = False
    xr = x.clone().requires_grad_(True)
    ref, c1 = orc.recurrent_block(xr, params, active=active)
    (ref * dout).sum().backward()
    with torch.no_grad():
        ref2, c2 = orc.recurrent_block(x2, params, c1, active=active2)

    blk = blk.to(DEV)
    xg = x.to(DEV).requires_grad_(True)
    out, g1 = blk(xg, active_mask=active.to(DEV), return_cache=True)
    (out * dout.to(DEV)).sum().backward()
    with torch.no_grad():
        out2, g2 = blk(x2.to(DEV), g1, active_mask=active2.to(DEV), return_cache=True)
    assert orc.rel_l2(out, ref) <= FP32_REL and orc.rel_l2(out2, ref2) <= FP32_REL
    assert orc.rel_l2(xg.grad, xr.grad) <= FP32_REL
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad, params[key].grad) <= 2e-5, key
    for got, want in ((g1, c1), (g2, c2)):
        assert orc.rel_l2(got.rnn_state, want.rnn_state) <= FP32_REL
        assert orc.rel_l2(got.conv_state, want.conv_state) <= FP32_REL
        assert torch.equal(got.segment_position.cpu(), want.segment_position)


# ---------------------------------------------------------------- conv folded into the scan's load stage
@pytest.mark.parametrize("shape", [(2, 150, 128), (3, 67, 64), (2, 70, 72), (1, 9, 20)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv_scan_kernels_against_oracle(shape, dtype):
    """rglru_conv_scan_fwd / _bwd through the C ABI: conv (with a carried state and a document boundary)
    fused into the scan, against the oracle's conv followed by its O(T) RG-LRU backward."""
    from griffin_b200 import ops
    from griffin_b200.modules import token_flags
    B, T, D = shape
    gen = torch.Generator().manual_seed(7 * T + D)
    x_in = torch.randn(B, T, D, generator=gen).to(dtype)
    u_r = torch.randn(B, T, D, generator=gen).to(dtype)
    u_i = torch.randn(B, T, D, generator=gen).to(dtype)
    dy = torch.randn(B, T, D, generator=gen).to(dtype)
    w = torch.randn(D, 4, generator=gen) * 0.5
    bias = torch.randn(D, generator=gen) * 0.1
    state = torch.randn(B, 3, D, generator=gen).to(dtype)
    lam = orc.init_lambda(D, 8.0, gen)
    h0 = torch.randn(B, D, generator=gen)
    dh = torch.randn(B, D, generator=gen)
    seg = torch.arange(T)[None, :].repeat(B, 1) + 2
    if T > 8:
        seg[:, T // 2:] = torch.arange(T - T // 2)
    reset = seg == 0
    xc_ref, _ = orc.causal_conv_dense(x_in.double(), w.double(), bias.double(), state.double(), seg)
    want = orc.rglru_backward_linear(xc_ref, u_r.double(), u_i.double(), lam.double(), dy.double(), h0=h0, dh_last=dh,
                                     reset=reset)
    flags = token_flags(B, T, DEV, reset=reset.to(DEV), segment_pos=seg.to(DEV))
    args = [t.to(DEV).contiguous() for t in (x_in, w, bias, state, u_r, u_i, lam, h0)]
    y, h_last, ws = ops.conv_scan_fwd(*args, flags, 8.0, True)
    dxc, du_r, du_i, dlam, dh0 = ops.conv_scan_bwd(dy.to(DEV), dh.to(DEV), *args, flags, ws, 8.0, True)
    tol = FP32_REL if dtype == torch.float32 else BF16_REL
    got = {"y": y, "h_last": h_last, "dx": dxc, "du_r": du_r, "du_i": du_i, "dLambda": dlam, "dh0": dh0}
    for key, val in got.items():
        err = orc.rel_l2(val, want[key])
        assert err <= tol, (key, err)


@pytest.mark.parametrize("conv", [False, True])
@pytest.mark.parametrize("shape", [(2, 150, 128), (3, 67, 64), (2, 70, 72), (1, 9, 20)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_merged_scan_kernels_against_oracle(shape, dtype, conv):
    """rglru_merge_fwd / _bwd through the C ABI: out = RG-LRU(...) * gelu_tanh(branch) formed in the store stage
    and differentiated in the backward load stage (griffin/griffin.py:464, 520), with and without the conv fold."""
    from griffin_b200 import ops
    from griffin_b200.modules import token_flags
    B, T, D = shape
    gen = torch.Generator().manual_seed(11 * T + D + int(conv))
    x_in = torch.randn(B, T, D, generator=gen).to(dtype)
    u_r = torch.randn(B, T, D, generator=gen).to(dtype)
    u_i = torch.randn(B, T, D, generator=gen).to(dtype)
    branch = (torch.randn(B, T, D, generator=gen) * 1.5).to(dtype)
    dout = torch.randn(B, T, D, generator=gen).to(dtype)
    w = torch.randn(D, 4, generator=gen) * 0.5
    bias = torch.randn(D, generator=gen) * 0.1
    state = torch.randn(B, 3, D, generator=gen).to(dtype)
    lam = orc.init_lambda(D, 8.0, gen)
    h0 = torch.randn(B, D, generator=gen)
    dh = torch.randn(B, D, generator=gen)
    seg = torch.arange(T)[None, :].repeat(B, 1) + 2
    if T > 8:
        seg[:, T // 2:] = torch.arange(T - T // 2)
    reset = seg == 0
    bd = branch.double().requires_grad_(True)
    gelu = torch.nn.functional.gelu(bd, approximate="tanh")
    (slope,) = torch.autograd.grad(gelu.sum(), bd)
    gelu = gelu.detach()
    x_ref = orc.causal_conv_dense(x_in.double(), w.double(), bias.double(), state.double(), seg)[0] if conv else x_in.double()
    want = orc.rglru_backward_linear(x_ref, u_r.double(), u_i.double(), lam.double(), dout.double() * gelu, h0=h0,
                                     dh_last=dh, reset=reset)
    want["out"] = want["y"] * gelu
    want["dbranch"] = dout.double() * want["y"] * slope
    flags = token_flags(B, T, DEV, reset=reset.to(DEV), segment_pos=seg.to(DEV))
    dev = lambda t: t.to(DEV).contiguous()
    conv_args = [dev(w), dev(bias), dev(state)] if conv else [None, None, None]
    args = [dev(x_in), *conv_args, dev(u_r), dev(u_i), dev(branch), dev(lam), dev(h0)]
    out, h_last, ws = ops.merge_scan_fwd(*args, flags, 8.0, True)
    dx, du_r, du_i, dbranch, dlam, dh0 = ops.merge_scan_bwd(dev(dout), dev(dh), *args, flags, ws, 8.0, True)
    tol = FP32_REL if dtype == torch.float32 else BF16_REL
    got = {"out": out, "h_last": h_last, "dx": dx, "du_r": du_r, "du_i": du_i, "dbranch": dbranch, "dLambda": dlam,
           "dh0": dh0}
    for key, val in got.items():
        err = orc.rel_l2(val, want[key])
        assert err <= tol, (key, err)
    from griffin_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("fold_conv", [False, True])
def test_merge_folded_block_matches_reference_gradients_and_cache(fold_conv):
    """RecurrentBlock(fold_merge=True): same outputs, gradients and caches as the reference's stored results."""
    from griffin_b200 import RecurrentBlock as _Block
    RecurrentBlock = lambda *a, **k: _Block(*a, fold_conv=fold_conv, **k)
    case = load_golden("block_grads")
    blk = RecurrentBlock(16, 32, gate_blocks=4, scan_mode="cuda", fold_merge=True)
    blk.load_state_dict(params_of(case))
    blk = blk.to(DEV)
    x = case["x"].to(DEV).requires_grad_(True)
    out = blk(x)
    (out * case["dout"].to(DEV)).sum().backward()
    assert orc.rel_l2(out, case["out"]) <= FP32_REL
    assert orc.rel_l2(x.grad, case["dx"]) <= FP32_REL
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad, case["g." + key]) <= FP32_REL, key

    case = load_golden("block_chunked")
    blk = RecurrentBlock(8, 12, scan_mode="cuda", fold_merge=True)
    blk.load_state_dict(params_of(case))
    blk = blk.to(DEV).eval()
    x = case["x"].to(DEV)
    with torch.no_grad():
        a, c1 = blk(x[:, :3], return_cache=True)
        b, c2 = blk(x[:, 3:7], c1, return_cache=True)
        c, c3 = blk(x[:, 7:], c2, return_cache=True)
    torch.testing.assert_close(torch.cat([a, b, c], 1).cpu(), case["chunks"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(c3.rnn_state.cpu(), case["c3.rnn"], atol=2e-6, rtol=2e-5)

    case = load_golden("block_ragged")
    blk = RecurrentBlock(8, 16, gate_blocks=4, scan_mode="cuda", fold_merge=True)
    blk.load_state_dict(params_of(case))
    blk = blk.to(DEV)
    x = case["x"].to(DEV).requires_grad_(True)
    first, c1 = blk(x, active_mask=case["active"].to(DEV), return_cache=True)
    (first * case["dout"].to(DEV)).sum().backward()
    torch.testing.assert_close(first.detach().cpu(), case["first"], atol=2e-6, rtol=2e-5)
    assert orc.rel_l2(x.grad.cpu(), case["dx"]) <= FP32_REL
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad.cpu(), case["g." + key]) <= FP32_REL, key


@pytest.mark.parametrize("merge", [False, True])
@pytest.mark.parametrize("shape", [(2, 150, 128, 2), (1, 70, 256, 2), (3, 33, 192, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grouped_gate_layout_against_oracle(shape, dtype, merge):
    """ops.rglru_grouped (rglru_grouped_fwd / _bwd): both block-diagonal gates from one grouped GEMM, biases
    added in the kernel, against the oracle's RG_LRU.forward (griffin/griffin.py:129-154, 237-286) and autograd."""
    from griffin_b200 import ops, _lib
    from griffin_b200.modules import token_flags
    B, T, D, G = shape
    bw = D // G
    gen = torch.Generator().manual_seed(13 * T + D + int(merge))
    rnd = lambda *sz: torch.randn(*sz, generator=gen)
    x = rnd(B, T, D).to(dtype)
    branch = (rnd(B, T, D) * 1.5).to(dtype)
    dout = rnd(B, T, D).to(dtype)
    params = {"recurrence_gate.weight": rnd(G, bw, bw) / bw ** 0.5, "recurrence_gate.bias": rnd(G, bw) * 0.3,
              "input_gate.weight": rnd(G, bw, bw) / bw ** 0.5, "input_gate.bias": rnd(G, bw) * 0.3,
              "Lambda": orc.init_lambda(D, 8.0, gen)}
    if dtype == torch.bfloat16:   # the GEMM sees bf16 weights; give the oracle the same rounded values
        for k in ("recurrence_gate.weight", "input_gate.weight"):
            params[k] = params[k].to(dtype).float()
    h0, dh = rnd(B, D), rnd(B, D)
    reset = torch.zeros(B, T, dtype=torch.bool)
    reset[:, T // 2] = True
    ref_p = {k: v.double().requires_grad_(True) for k, v in params.items()}
    xd = x.double().requires_grad_(True)
    bd = branch.double().requires_grad_(True)
    h0d = h0.double().requires_grad_(True)
    y_ref, hl_ref = orc.rglru_layer(xd, ref_p, h0d, reset=reset)
    out_ref = y_ref * torch.nn.functional.gelu(bd, approximate="tanh") if merge else y_ref
    ((out_ref * dout.double()).sum() + (hl_ref * dh.double()).sum()).backward()

    dev_p = {k: v.to(DEV).requires_grad_(True) for k, v in params.items()}
    xg = x.to(DEV).requires_grad_(True)
    bg = branch.to(DEV).requires_grad_(True)
    h0g = h0.to(DEV).requires_grad_(True)
    flags = token_flags(B, T, DEV, reset=reset.to(DEV))
    out, h_last = ops.rglru_grouped(xg, dev_p["recurrence_gate.weight"], dev_p["recurrence_gate.bias"],
                                    dev_p["input_gate.weight"], dev_p["input_gate.bias"], dev_p["Lambda"], h0g, flags, 8.0,
                                    bg if merge else None)
    ((out.float() * dout.to(DEV).float()).sum() + (h_last * dh.to(DEV)).sum()).backward()
    tol = FP32_REL if dtype == torch.float32 else BF16_REL
    pairs = {"out": (out, out_ref), "h_last": (h_last, hl_ref), "dx": (xg.grad, xd.grad), "dh0": (h0g.grad, h0d.grad)}
    if merge:
        pairs["dbranch"] = (bg.grad, bd.grad)
    for k in params:
        pairs["d" + k] = (dev_p[k].grad, ref_p[k].grad)
    for key, (got, want) in pairs.items():
        err = orc.rel_l2(got, want)
        assert err <= tol, (key, err)
    assert _lib.device_status() == 0


def test_folded_block_matches_reference_gradients_and_cache():
    """RecurrentBlock(fold_conv=True): same outputs, gradients and caches as the reference's stored results."""
    from griffin_b200 import RecurrentBlock
    case = load_golden("block_grads")
    blk = RecurrentBlock(16, 32, gate_blocks=4, scan_mode="cuda", fold_conv=True)
    blk.load_state_dict(params_of(case))
    blk = blk.to(DEV)
    x = case["x"].to(DEV).requires_grad_(True)
    out = blk(x)
    (out * case["dout"].to(DEV)).sum().backward()
    assert orc.rel_l2(out, case["out"]) <= FP32_REL
    assert orc.rel_l2(x.grad, case["dx"]) <= FP32_REL
    for key, p in blk.named_parameters():
        assert orc.rel_l2(p.grad, case["g." + key]) <= FP32_REL, key

    case = load_golden("block_chunked")
    blk = RecurrentBlock(8, 12, scan_mode="cuda", fold_conv=True)
    blk.load_state_dict(params_of(case))
    blk = blk.to(DEV).eval()
    x = case["x"].to(DEV)
    with torch.no_grad():
        a, c1 = blk(x[:, :3], return_cache=True)
        b, c2 = blk(x[:, 3:7], c1, return_cache=True)
        c, c3 = blk(x[:, 7:], c2, return_cache=True)
    torch.testing.assert_close(torch.cat([a, b, c], 1).cpu(), case["chunks"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(c3.rnn_state.cpu(), case["c3.rnn"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(c3.conv_state.cpu(), case["c3.conv"], atol=1e-6, rtol=1e-6)

    case = load_golden("block_reset")
    blk = RecurrentBlock(8, 16, gate_blocks=4, scan_mode="cuda", fold_conv=True)
    blk.load_state_dict(params_of(case))
    blk = blk.to(DEV).eval()
    with torch.no_grad():
        out = blk(case["x"].to(DEV), segment_pos=case["segment_pos"].to(DEV))
    torch.testing.assert_close(out.cpu(), case["full"], atol=2e-6, rtol=2e-5)


def test_blocks_that_share_mask_tensors_agree_with_blocks_given_their_own_copies():
    """A model hands one segment_pos / active_mask tensor to all its blocks; what the first block derives from them
    is reused by the others.  Results must equal those of calls given fresh copies (nothing to reuse), also after
    the mask has been changed in place, and with padding that is not right padding."""
    from griffin_b200 import RecurrentBlock
    torch.manual_seed(21)
    B, T = 3, 70
    blocks = [RecurrentBlock(32, 64, gate_blocks=1).to(DEV) for _ in range(2)]
    x = torch.randn(B, T, 32, device=DEV)
    pos = (torch.arange(T, device=DEV) % 23).expand(B, T).contiguous()
    mask = torch.ones(B, T, dtype=torch.bool, device=DEV)
    mask[1, 50:] = False                                   # right padding
    mask[2, :7] = False                                    # left padding: rows are partitioned

    def run(p, m):
        h = x
        for blk in blocks:
            h = blk(h, segment_pos=p() if callable(p) else p, active_mask=m() if callable(m) else m)
        return h

    shared = run(pos, mask)
    fresh = run(lambda: pos.clone(), lambda: mask.clone())
    assert torch.equal(shared, fresh)
    mask[0, 60:] = False                                   # same object, new version
    assert torch.equal(run(pos, mask), run(lambda: pos.clone(), lambda: mask.clone()))
    assert not torch.equal(run(pos, mask), shared)
    g = torch.autograd.grad(run(pos, mask).square().sum(), blocks[0].linear_x.weight)[0]
    g2 = torch.autograd.grad(run(lambda: pos.clone(), lambda: mask.clone()).square().sum(), blocks[0].linear_x.weight)[0]
    assert torch.equal(g, g2)
