"""The CPU oracle must reproduce the reference's stored outputs and gradients.

Every golden file was written by the unmodified reference (see
tests/golden/make_golden.py).  Tolerances: the oracle uses the same torch
primitives in the same order, so fp32 agreement is expected to ~1e-6.
"""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, params_of
from oracle import rglru_oracle as orc

TIGHT = dict(atol=2e-6, rtol=2e-6)


def _run_layer(case, dtype=torch.float32):
    params = {k: v.to(dtype).clone().requires_grad_(True) for k, v in params_of(case).items()}
    x = case["x"].to(dtype).clone().requires_grad_(True)
    h0 = case["h0"].clone().requires_grad_(True) if "h0" in case else None
    reset = case.get("reset")
    active = case.get("active")
    u_r = orc.block_diagonal_linear(x, params["recurrence_gate.weight"], params["recurrence_gate.bias"])
    u_i = orc.block_diagonal_linear(x, params["input_gate.weight"], params["input_gate.bias"])
    u_r.retain_grad()
    u_i.retain_grad()
    y, h_last = orc.rglru_core(x, u_r, u_i, params["Lambda"], h0, reset, active)
    loss = (y.float() * case["dy"].float()).sum()
    if "dh_last" in case:
        loss = loss + (h_last * case["dh_last"]).sum()
    loss.backward()
    return x, h0, params, u_r, u_i, y, h_last


@pytest.mark.parametrize("name", ["rglru_masks_f32", "rglru_state_f32", "rglru_plain_f32"])
def test_layer_matches_reference_fp32(name):
    case = load_golden(name)
    x, h0, params, u_r, u_i, y, h_last = _run_layer(case)
    torch.testing.assert_close(y, case["y"], **TIGHT)
    torch.testing.assert_close(h_last, case["h_last"], **TIGHT)
    torch.testing.assert_close(x.grad, case["dx"], **TIGHT)
    torch.testing.assert_close(u_r.grad, case["du_r"], **TIGHT)
    torch.testing.assert_close(u_i.grad, case["du_i"], **TIGHT)
    for key, p in params.items():
        torch.testing.assert_close(p.grad, case["g." + key], **TIGHT)
    if h0 is not None:
        torch.testing.assert_close(h0.grad, case["dh0"], **TIGHT)


@pytest.mark.parametrize("name", ["rglru_masks_f32", "rglru_state_f32", "rglru_plain_f32"])
def test_linear_time_backward_matches_reference(name):
    """The hand-derived O(T) reverse pass agrees with the reference's autograd."""
    case = load_golden(name)
    got = orc.rglru_backward_linear(
        case["x"].double(), case["u_r"].double(), case["u_i"].double(), case["p.Lambda"].double(), case["dy"].double(),
        h0=case.get("h0"), dh_last=case.get("dh_last"), reset=case.get("reset"), active=case.get("active"),
    )
    loose = dict(atol=5e-6, rtol=5e-5)  # golden values are fp32 results
    torch.testing.assert_close(got["y"].float(), case["y"], **loose)
    torch.testing.assert_close(got["du_r"].float(), case["du_r"], **loose)
    torch.testing.assert_close(got["du_i"].float(), case["du_i"], **loose)
    torch.testing.assert_close(got["dLambda"].float(), case["g.Lambda"], atol=2e-5, rtol=2e-4)
    if "dh0" in case:
        torch.testing.assert_close(got["dh0"].float(), case["dh0"], **loose)
    # total dx = direct part + both gate paths
    params = params_of(case)
    def back(du, w):
        g, bo, bi = w.shape
        return torch.einsum("...go,goi->...gi", du.reshape(*du.shape[:-1], g, bo), w.double()).reshape(du.shape)
    dx = got["dx"] + back(got["du_r"], params["recurrence_gate.weight"]) + back(got["du_i"], params["input_gate.weight"])
    torch.testing.assert_close(dx.float(), case["dx"], **loose)


def test_bf16_extreme_case_is_finite_and_close():
    case = load_golden("rglru_extreme_bf16")
    x, h0, params, u_r, u_i, y, h_last = _run_layer(case, torch.bfloat16)
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    assert torch.isfinite(params["Lambda"].grad.float()).all()
    torch.testing.assert_close(y.float(), case["y"], atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(x.grad.float(), case["dx"], atol=2e-2, rtol=2e-2)


def test_config0_full_shape():
    case = load_golden("rglru_config0_f32")
    inp = orc.make_rglru_case(2, 256, 256, 4, seed=0)
    chk = torch.tensor([inp["x"].double().sum(), inp["dy"].double().sum(), inp["Lambda"].double().sum()])
    torch.testing.assert_close(chk, case["input_checksum"], atol=1e-9, rtol=1e-12)
    params = {k: inp[k].clone().requires_grad_(True) for k in
              ("Lambda", "recurrence_gate.weight", "recurrence_gate.bias", "input_gate.weight", "input_gate.bias")}
    x = inp["x"].clone().requires_grad_(True)
    y, h_last = orc.rglru_layer(x, params)
    (y * inp["dy"]).sum().backward()
    ts = int(case["subsample"][0])
    torch.testing.assert_close(y[:, ts // 2 :: ts], case["y"], **TIGHT)
    torch.testing.assert_close(x.grad[:, ts // 2 :: ts], case["dx"], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(h_last, case["h_last"], **TIGHT)
    for key, p in params.items():
        assert orc.rel_l2(p.grad, case["g." + key]) < 1e-6


def test_bf16_pair_both_references():
    case = load_golden("rglru_bf16_pair")
    params = params_of(case)
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        p = {k: v.to(dtype).detach().requires_grad_(True) for k, v in params.items()}
        x = case["x"].to(dtype).detach().requires_grad_(True)
        y, h_last = orc.rglru_layer(x, p)
        (y.float() * case["dy"].float()).sum().backward()
        # same primitives in the same order: agreement is at rounding level
        assert orc.rel_l2(y, case[f"{tag}.y"]) <= 1e-6
        assert orc.rel_l2(x.grad, case[f"{tag}.dx"]) <= 1e-5
        assert orc.rel_l2(p["Lambda"].grad, case[f"{tag}.g.Lambda"]) <= 1e-5


def test_raw_scan_selftest_and_random():
    vec = orc.selftest_vectors()
    gold = load_golden("scan_selftest")
    leaves = [vec[k].clone().requires_grad_(True) for k in ("decay", "drive", "h0")]
    out = orc.linear_scan(*leaves)
    grads = torch.autograd.grad(out, leaves, vec["upstream"])
    torch.testing.assert_close(out, gold["out"], **TIGHT)
    for g, key in zip(grads, ("d_decay", "d_drive", "d_h0")):
        torch.testing.assert_close(g, gold[key], **TIGHT)
    rnd = load_golden("scan_random")
    leaves = [rnd[k].clone().requires_grad_(True) for k in ("decay", "drive", "h0")]
    out = orc.linear_scan(*leaves)
    grads = torch.autograd.grad(out, leaves, rnd["upstream"])
    torch.testing.assert_close(out, rnd["out"], **TIGHT)
    for g, key in zip(grads, ("d_decay", "d_drive", "d_h0")):
        torch.testing.assert_close(g, rnd[key], **TIGHT)


def test_block_chunked_reset_padded_decode():
    case = load_golden("block_chunked")
    p = params_of(case)
    x = case["x"]
    full, _ = orc.recurrent_block(x, p)
    torch.testing.assert_close(full, case["full"], **TIGHT)
    a, c1 = orc.recurrent_block(x[:, :3], p)
    b, c2 = orc.recurrent_block(x[:, 3:7], p, c1)
    c, c3 = orc.recurrent_block(x[:, 7:], p, c2)
    torch.testing.assert_close(torch.cat([a, b, c], 1), case["chunks"], **TIGHT)
    for tag, cache in (("c1", c1), ("c2", c2), ("c3", c3)):
        torch.testing.assert_close(cache.rnn_state, case[f"{tag}.rnn"], **TIGHT)
        torch.testing.assert_close(cache.conv_state, case[f"{tag}.conv"], **TIGHT)
        assert torch.equal(cache.segment_position, case[f"{tag}.pos"])

    case = load_golden("block_reset")
    out, cache = orc.recurrent_block(case["x"], params_of(case), segment_pos=case["segment_pos"])
    torch.testing.assert_close(out, case["full"], **TIGHT)
    torch.testing.assert_close(cache.rnn_state, case["rnn"], **TIGHT)
    torch.testing.assert_close(cache.conv_state, case["conv"], **TIGHT)
    assert torch.equal(cache.segment_position, case["pos"])

    case = load_golden("block_padded")
    p = params_of(case)
    pre, c1 = orc.recurrent_block(case["x"], p, active=case["active"])
    dec, c2 = orc.recurrent_block(case["next"], p, c1)
    torch.testing.assert_close(pre, case["prefill"], **TIGHT)
    torch.testing.assert_close(dec, case["decode"], **TIGHT)
    torch.testing.assert_close(c1.conv_state, case["c1.conv"], **TIGHT)
    torch.testing.assert_close(c2.rnn_state, case["c2.rnn"], **TIGHT)
    assert torch.equal(c2.segment_position, case["c2.pos"])

    case = load_golden("block_decode")
    p = params_of(case)
    cache = None
    outs = []
    for t in range(case["x"].shape[1]):
        o, cache = orc.recurrent_block(case["x"][:, t : t + 1], p, cache)
        outs.append(o)
        torch.testing.assert_close(cache.rnn_state, case["rnn"][t], **TIGHT)
        torch.testing.assert_close(cache.conv_state, case["conv"][t], **TIGHT)
    torch.testing.assert_close(torch.cat(outs, 1), case["steps"], **TIGHT)


def test_block_with_padding_that_is_not_right_padding():
    """Left padding and holes: padding must neither enter the conv history nor move the state (griffin/griffin.py:488-510)."""
    case = load_golden("block_ragged")
    p = {k: v.clone().requires_grad_(True) for k, v in params_of(case).items()}
    x = case["x"].clone().requires_grad_(True)
    first, c1 = orc.recurrent_block(x, p, active=case["active"])
    (first * case["dout"]).sum().backward()
    with torch.no_grad():
        second, c2 = orc.recurrent_block(case["x2"], p, c1, active=case["active2"])
    torch.testing.assert_close(first.detach(), case["first"], **TIGHT)
    torch.testing.assert_close(second, case["second"], **TIGHT)
    torch.testing.assert_close(x.grad, case["dx"], **TIGHT)
    for tag, cache in (("c1", c1), ("c2", c2)):
        torch.testing.assert_close(cache.rnn_state.detach(), case[f"{tag}.rnn"], **TIGHT)
        torch.testing.assert_close(cache.conv_state.detach(), case[f"{tag}.conv"], **TIGHT)
        assert torch.equal(cache.segment_position, case[f"{tag}.pos"])
    for key in case:
        if key.startswith("g."):
            torch.testing.assert_close(p[key[2:]].grad, case[key], **TIGHT)


def test_ragged_block_gradients_through_the_linear_backward():
    """The O(T) backward with padding that is not right padding and a carried cache (stored reference gradients)."""
    case = load_golden("block_ragged")
    p = {k: v.clone().requires_grad_(True) for k, v in params_of(case).items()}
    x = case["x"].clone().requires_grad_(True)
    first, _ = orc.recurrent_block(x, p, active=case["active"], linear_backward=True)
    (first * case["dout"]).sum().backward()
    torch.testing.assert_close(first.detach(), case["first"], **TIGHT)
    torch.testing.assert_close(x.grad, case["dx"], **TIGHT)
    for key in case:
        if key.startswith("g."):
            torch.testing.assert_close(p[key[2:]].grad, case[key], **TIGHT)


@pytest.mark.parametrize("linear_backward", [False, True])
def test_block_gradients(linear_backward):
    """The reference's stored block gradients, through autograd over the sequential loop and through the
    oracle's O(T) closed-form backward of the scan (the route the full-size GPU tests check against)."""
    case = load_golden("block_grads")
    p = {k: v.clone().requires_grad_(True) for k, v in params_of(case).items()}
    x = case["x"].clone().requires_grad_(True)
    out, _ = orc.recurrent_block(x, p, linear_backward=linear_backward)
    (out * case["dout"]).sum().backward()
    torch.testing.assert_close(out, case["out"], **TIGHT)
    torch.testing.assert_close(x.grad, case["dx"], atol=1e-5, rtol=1e-5)
    for key, v in p.items():
        assert orc.rel_l2(v.grad, case["g." + key]) < 1e-5, key
