"""Generate the golden vectors under tests/golden/ from the unmodified reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/Griffin

It imports the reference package (CPU, ``scan_mode="sequential"``), runs small
seeded cases through ``RG_LRU`` / ``RecurrentBlock`` / the raw scan, and writes
one ``.npz`` per case with inputs, parameters, outputs and gradients.  The
tests never import the reference; they only read these files.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import rglru_oracle as orc  # noqa: E402  (seeded input builders only)


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach()
    if t.dtype == torch.bfloat16:
        t = t.float()
    return t.cpu().numpy()


def _save(name: str, payload: dict[str, torch.Tensor | np.ndarray]) -> None:
    arrays = {k: (v if isinstance(v, np.ndarray) else _np(v)) for k, v in payload.items()}
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB, {len(arrays)} arrays")


def _hook_gates(module, store):
    def keep(tag):
        def fn(_mod, _inp, out):
            if out.requires_grad:
                out.retain_grad()
            store[tag] = out

        return fn

    return [
        module.recurrence_gate.register_forward_hook(keep("u_r")),
        module.input_gate.register_forward_hook(keep("u_i")),
    ]


def _rglru_case(G, name, batch, steps, width, blocks, *, dtype=torch.float32, seed=0,
                use_h0=False, use_dh=False, reset_at=None, inactive_tail=0,
                extreme=False, subsample=None):
    torch.manual_seed(seed)
    module = G.RG_LRU(width, gate_blocks=blocks, scan_mode="sequential")
    if extreme:
        with torch.no_grad():
            module.Lambda[: max(1, width // 6)] = 20.0
            module.recurrence_gate.bias[0, :2] = -100.0
    module = module.to(dtype)
    x = torch.randn(batch, steps, width).to(dtype).requires_grad_(True)
    dy = torch.randn(batch, steps, width).to(dtype)
    h0 = torch.randn(batch, width) if use_h0 else None
    if h0 is not None:
        h0.requires_grad_(True)
    dh = torch.randn(batch, width) if use_dh else None
    reset = None
    if reset_at is not None:
        reset = torch.zeros(batch, steps, dtype=torch.bool)
        for row, t in reset_at:
            reset[row, t] = True
    active = None
    if inactive_tail:
        active = torch.ones(batch, steps, dtype=torch.bool)
        active[-1, -inactive_tail:] = False
    store = {}
    hooks = _hook_gates(module, store)
    y, h_last = module(x, h0, reset_mask=reset, active_mask=active, return_state=True)
    loss = (y.float() * dy.float()).sum()
    if dh is not None:
        loss = loss + (h_last * dh).sum()
    loss.backward()
    for h in hooks:
        h.remove()
    out = {
        "x": x, "dy": dy, "y": y, "h_last": h_last, "dx": x.grad,
        "u_r": store["u_r"], "u_i": store["u_i"],
        "du_r": store["u_r"].grad, "du_i": store["u_i"].grad,
    }
    for key, p in module.state_dict().items():
        out["p." + key] = p
    for key, p in module.named_parameters():
        out["g." + key] = p.grad
    if h0 is not None:
        out["h0"] = h0
        out["dh0"] = h0.grad
    if dh is not None:
        out["dh_last"] = dh
    if reset is not None:
        out["reset"] = reset.numpy()
    if active is not None:
        out["active"] = active.numpy()
    if subsample is not None:
        ts, ds = subsample
        for key in ("y", "dx", "du_r", "du_i", "u_r", "u_i"):
            out[key] = out[key][:, ts // 2 :: ts, ::ds]
        out["subsample"] = np.array([ts, ds])
        del out["x"], out["dy"]  # regenerated from the seed by the test
    _save(name, out)


def _config0(G):
    """B=2, T=256, D=256, 4 gate heads, fp32 at full shape; inputs come from oracle.make_rglru_case(seed=0)."""
    case = orc.make_rglru_case(2, 256, 256, 4, seed=0)
    module = G.RG_LRU(256, gate_blocks=4, scan_mode="sequential")
    with torch.no_grad():
        module.Lambda.copy_(case["Lambda"])
        module.recurrence_gate.weight.copy_(case["recurrence_gate.weight"])
        module.recurrence_gate.bias.copy_(case["recurrence_gate.bias"])
        module.input_gate.weight.copy_(case["input_gate.weight"])
        module.input_gate.bias.copy_(case["input_gate.bias"])
    x = case["x"].clone().requires_grad_(True)
    store = {}
    hooks = _hook_gates(module, store)
    y, h_last = module(x, return_state=True)
    (y * case["dy"]).sum().backward()
    for h in hooks:
        h.remove()
    ts, ds = 16, 1
    out = {
        "input_checksum": np.array([case["x"].double().sum().item(), case["dy"].double().sum().item(),
                                    case["Lambda"].double().sum().item()]),
        "subsample": np.array([ts, ds]),
        "y": y[:, ts // 2 :: ts], "dx": x.grad[:, ts // 2 :: ts],
        "du_r": store["u_r"].grad[:, ts // 2 :: ts], "du_i": store["u_i"].grad[:, ts // 2 :: ts],
        "h_last": h_last,
        "y_norm": np.array([y.double().norm().item()]),
        "dx_norm": np.array([x.grad.double().norm().item()]),
    }
    for key, p in module.named_parameters():
        out["g." + key] = p.grad
    _save("rglru_config0_f32", out)


def _bf16_pair(G):
    """bf16 I/O slice: the literal bf16 reference and the fp32 reference on bf16-rounded data."""
    torch.manual_seed(3)
    batch, steps, width, blocks = 2, 160, 64, 2
    ref32 = G.RG_LRU(width, gate_blocks=blocks, scan_mode="sequential")
    with torch.no_grad():
        for p in ref32.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    x = torch.randn(batch, steps, width).to(torch.bfloat16)
    dy = torch.randn(batch, steps, width).to(torch.bfloat16)
    out = {"x": x, "dy": dy}
    for key, p in ref32.state_dict().items():
        out["p." + key] = p
    for tag, module, xin in (
        ("f32", ref32, x.float()),
        ("bf16", G.RG_LRU(width, gate_blocks=blocks, scan_mode="sequential"), x),
    ):
        if tag == "bf16":
            module.load_state_dict(ref32.state_dict())
            module = module.to(torch.bfloat16)
        xin = xin.clone().requires_grad_(True)
        store = {}
        hooks = _hook_gates(module, store)
        y, h_last = module(xin, return_state=True)
        (y.float() * dy.float()).sum().backward()
        for h in hooks:
            h.remove()
        out[f"{tag}.y"] = y
        out[f"{tag}.h_last"] = h_last
        out[f"{tag}.dx"] = xin.grad
        out[f"{tag}.u_r"] = store["u_r"]
        out[f"{tag}.u_i"] = store["u_i"]
        out[f"{tag}.du_r"] = store["u_r"].grad
        out[f"{tag}.du_i"] = store["u_i"].grad
        for key, p in module.named_parameters():
            out[f"{tag}.g.{key}"] = p.grad
    _save("rglru_bf16_pair", out)


def _scan_selftest(TS):
    vec = orc.selftest_vectors()
    leaves = [vec[k].clone().requires_grad_(True) for k in ("decay", "drive", "h0")]
    out = TS._reference_scan(*leaves)
    grads = torch.autograd.grad(out, leaves, vec["upstream"])
    _save("scan_selftest", {"out": out, "d_decay": grads[0], "d_drive": grads[1], "d_h0": grads[2]})

    torch.manual_seed(0)
    decay = torch.sigmoid(torch.randn(2, 37, 65)).requires_grad_(True)
    drive = torch.randn(2, 37, 65, requires_grad=True)
    h0 = torch.randn(2, 65, requires_grad=True)
    up = torch.randn(2, 37, 65)
    out = TS._reference_scan(decay, drive, h0)
    grads = torch.autograd.grad(out, (decay, drive, h0), up)
    _save("scan_random", {"decay": decay, "drive": drive, "h0": h0, "upstream": up, "out": out,
                          "d_decay": grads[0], "d_drive": grads[1], "d_h0": grads[2]})


def _block_cases(G):
    # chunked prefill == full (tests/test_recurrentblock.py:33-50 shape family)
    torch.manual_seed(0)
    block = G.RecurrentBlock(input_dim=8, rnn_width=12, scan_mode="sequential").eval()
    x = torch.randn(2, 9, 8)
    with torch.no_grad():
        full = block(x)
        first, cache1 = block(x[:, :3], return_cache=True)
        second, cache2 = block(x[:, 3:7], cache1, return_cache=True)
        third, cache3 = block(x[:, 7:], cache2, return_cache=True)
    out = {"x": x, "full": full, "chunks": torch.cat([first, second, third], dim=1)}
    for n, cache in (("c1", cache1), ("c2", cache2), ("c3", cache3)):
        out[f"{n}.rnn"] = cache.rnn_state
        out[f"{n}.conv"] = cache.conv_state
        out[f"{n}.pos"] = cache.segment_position
    for key, p in block.state_dict().items():
        out["p." + key] = p
    _save("block_chunked", out)

    # document reset in the middle, explicit segment positions
    torch.manual_seed(1)
    block = G.RecurrentBlock(input_dim=8, rnn_width=16, gate_blocks=4, scan_mode="sequential").eval()
    with torch.no_grad():
        block.temporal_conv.weight.normal_(0.0, 0.5)
        block.temporal_conv.bias.normal_(0.0, 0.1)
    x = torch.randn(2, 11, 8)
    seg = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 3, 4, 5, 6], [0, 1, 0, 1, 2, 3, 4, 0, 1, 2, 3]])
    with torch.no_grad():
        full, cache = block(x, segment_pos=seg, return_cache=True)
    out = {"x": x, "segment_pos": seg, "full": full, "rnn": cache.rnn_state, "conv": cache.conv_state,
           "pos": cache.segment_position}
    for key, p in block.state_dict().items():
        out["p." + key] = p
    _save("block_reset", out)

    # right-padded prefill followed by one decode token
    torch.manual_seed(2)
    block = G.RecurrentBlock(input_dim=8, rnn_width=16, gate_blocks=4, scan_mode="sequential").eval()
    with torch.no_grad():
        block.temporal_conv.weight.normal_(0.0, 0.5)
    x = torch.randn(2, 5, 8)
    mask = torch.tensor([[True, True, True, True, True], [True, True, True, False, False]])
    nxt = torch.randn(2, 1, 8)
    with torch.no_grad():
        pre, cache = block(x, active_mask=mask, return_cache=True)
        dec, cache2 = block(nxt, cache, return_cache=True)
    out = {"x": x, "active": mask.numpy(), "next": nxt, "prefill": pre, "decode": dec,
           "c1.rnn": cache.rnn_state, "c1.conv": cache.conv_state, "c1.pos": cache.segment_position,
           "c2.rnn": cache2.rnn_state, "c2.conv": cache2.conv_state, "c2.pos": cache2.segment_position}
    for key, p in block.state_dict().items():
        out["p." + key] = p
    _save("block_padded", out)

    # padding that is not right padding (left padding, holes), two cached chunks, gradients of the first
    torch.manual_seed(6)
    block = G.RecurrentBlock(input_dim=8, rnn_width=16, gate_blocks=4, scan_mode="sequential")
    with torch.no_grad():
        block.temporal_conv.weight.normal_(0.0, 0.5)
        block.temporal_conv.bias.normal_(0.0, 0.1)
    x = torch.randn(3, 10, 8, requires_grad=True)
    mask = torch.tensor([[0, 0, 0, 1, 1, 1, 1, 1, 1, 1],
                         [1, 1, 0, 1, 0, 0, 1, 1, 0, 1],
                         [0, 1, 1, 1, 1, 0, 0, 0, 0, 0]], dtype=torch.bool)
    x2 = torch.randn(3, 6, 8)
    mask2 = torch.tensor([[1, 0, 1, 1, 0, 1], [0, 0, 1, 1, 1, 1], [0, 0, 0, 0, 0, 0]], dtype=torch.bool)
    dout = torch.randn(3, 10, 8)
    first, cache = block(x, active_mask=mask, return_cache=True)
    (first * dout).sum().backward()
    with torch.no_grad():
        second, cache2 = block(x2, cache, active_mask=mask2, return_cache=True)
    out = {"x": x, "active": mask.numpy(), "x2": x2, "active2": mask2.numpy(), "dout": dout, "first": first,
           "second": second, "dx": x.grad,
           "c1.rnn": cache.rnn_state, "c1.conv": cache.conv_state, "c1.pos": cache.segment_position,
           "c2.rnn": cache2.rnn_state, "c2.conv": cache2.conv_state, "c2.pos": cache2.segment_position}
    for key, p in block.state_dict().items():
        out["p." + key] = p
    for key, p in block.named_parameters():
        out["g." + key] = p.grad
    _save("block_ragged", out)

    # forward + backward through the whole block, conv weights ~ N(0, 1/4)
    torch.manual_seed(4)
    block = G.RecurrentBlock(input_dim=16, rnn_width=32, gate_blocks=4, scan_mode="sequential")
    with torch.no_grad():
        block.temporal_conv.weight.normal_(0.0, 0.5)
        block.temporal_conv.bias.normal_(0.0, 0.1)
    x = torch.randn(2, 33, 16, requires_grad=True)
    dout = torch.randn(2, 33, 16)
    out_t = block(x)
    (out_t * dout).sum().backward()
    out = {"x": x, "dout": dout, "out": out_t, "dx": x.grad}
    for key, p in block.state_dict().items():
        out["p." + key] = p
    for key, p in block.named_parameters():
        out["g." + key] = p.grad
    _save("block_grads", out)

    # token-by-token decode with the cache (tests/test_griffin_model.py:87-118 family)
    torch.manual_seed(5)
    block = G.RecurrentBlock(input_dim=8, rnn_width=16, gate_blocks=4, scan_mode="sequential").eval()
    with torch.no_grad():
        block.temporal_conv.weight.normal_(0.0, 0.5)
    x = torch.randn(3, 7, 8)
    outs, rnn, conv = [], [], []
    cache = None
    with torch.no_grad():
        full = block(x)
        for t in range(x.size(1)):
            o, cache = block(x[:, t : t + 1], cache, return_cache=True)
            outs.append(o)
            rnn.append(cache.rnn_state)
            conv.append(cache.conv_state)
    out = {"x": x, "full": full, "steps": torch.cat(outs, dim=1), "rnn": torch.stack(rnn), "conv": torch.stack(conv)}
    for key, p in block.state_dict().items():
        out["p." + key] = p
    _save("block_decode", out)


def _model_cases(G):
    """Tiny hybrid LM (reference tests/test_griffin_model.py shapes): logits, CE loss and a few gradients,
    with default positions and with a document reset; plus the local attention block alone."""
    torch.manual_seed(7)
    model = G.GriffinModel(vocab_size=23, input_dim=8, mlp_expansion_factor=2, rnn_width=12, depth=3,
                           attention_heads=2, attention_window_size=4, scan_mode="sequential")
    with torch.no_grad():
        for layer in model.layers:
            if layer.temporal_block_type == "recurrent":
                layer.recurrent.temporal_conv.weight.normal_(0.0, 0.5)
    tokens = torch.randint(0, 23, (2, 9))
    targets = torch.randint(0, 23, (2, 9))
    seg = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 3, 4], [0, 1, 2, 3, 4, 5, 6, 0, 1]])
    out = {"tokens": tokens, "targets": targets, "segment_pos": seg}
    for key, p_ in model.state_dict().items():
        out["p." + key] = p_
    for tag, kwargs in (("plain", {}), ("seg", {"segment_pos": seg})):
        model.zero_grad()
        logits = model(tokens, **kwargs)
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 23), targets.reshape(-1))
        loss.backward()
        out[f"{tag}.logits"] = logits
        out[f"{tag}.loss"] = loss.detach().reshape(1)
        for name in ("embd.weight", "layers.0.recurrent.rg_lru.Lambda", "layers.0.recurrent.temporal_conv.weight",
                     "layers.1.recurrent.rg_lru.input_gate.weight", "layers.2.attention.query.weight",
                     "layers.2.mlp.linear3.weight", "final_norm.g"):
            out[f"{tag}.g.{name}"] = dict(model.named_parameters())[name].grad
    _save("model_tiny", out)

    torch.manual_seed(8)
    attn = G.LocalMQAAttention(input_dim=16, num_heads=2, window_size=5, chunk_size=3)
    x = torch.randn(2, 11, 16)
    seg = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 0, 1, 2, 3], [3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13]])
    with torch.no_grad():
        out = {"x": x, "segment_pos": seg, "plain": attn(x), "seg": attn(x, segment_pos=seg)}
    for key, p_ in attn.state_dict().items():
        out["p." + key] = p_
    _save("attention_block", out)


def _model_autocast_case(G):
    """A small hybrid LM run the way the reference trains (train.py:254-267): bf16 autocast around the model,
    cross-entropy on the logits, fp32 parameters and gradients.  Gate heads are 64 wide like the 100M model's, the
    vocabulary is odd, and the sequence spans more than one 64-step chunk."""
    torch.manual_seed(9)
    vocab = 131
    model = G.GriffinModel(vocab_size=vocab, input_dim=16, mlp_expansion_factor=2, rnn_width=128, depth=3,
                           attention_heads=2, attention_window_size=16, gate_blocks=2, scan_mode="sequential")
    tokens = torch.randint(0, vocab, (2, 97))
    out = {"tokens": tokens}
    for key, p_ in model.state_dict().items():
        out["p." + key] = p_
    with torch.autocast("cpu", dtype=torch.bfloat16):
        logits = model(tokens[:, :-1])
    loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, vocab), tokens[:, 1:].reshape(-1))
    loss.backward()
    out["logits"] = logits.float()
    out["loss"] = loss.detach().reshape(1)
    keep = ("embd.weight", "final_norm.g", "layers.2.attention.query.weight", "layers.2.mlp.linear3.weight")
    for name, p_ in model.named_parameters():
        if name.startswith("layers.0.recurrent.") or name.startswith("layers.1.recurrent.rg_lru.") or name in keep:
            out["g." + name] = p_.grad
    _save("model_autocast_bf16", out)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("GRIFFIN_REFERENCE"),
                    help="checkout of the unmodified reference project (or set GRIFFIN_REFERENCE)")
    ap.add_argument("--only", default=None, help="write just this case (e.g. model_autocast_bf16)")
    args = ap.parse_args()
    if not args.reference or not os.path.isdir(args.reference):
        ap.error("pass --reference <checkout of the reference project>")
    sys.path.insert(0, args.reference)
    import griffin as G  # the unmodified reference
    from griffin import triton_scan as TS

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    if args.only == "model_autocast_bf16":
        _model_autocast_case(G)
        return
    _rglru_case(G, "rglru_masks_f32", 2, 29, 32, 4, seed=0, reset_at=[(0, 17), (1, 17)], inactive_tail=4)
    _rglru_case(G, "rglru_state_f32", 3, 19, 24, 4, seed=1, use_h0=True, use_dh=True,
                reset_at=[(1, 7)], inactive_tail=5, extreme=True)
    _rglru_case(G, "rglru_plain_f32", 2, 150, 40, 4, seed=2, use_h0=True)
    _rglru_case(G, "rglru_extreme_bf16", 2, 8, 16, 4, dtype=torch.bfloat16, seed=6, extreme=True)
    _config0(G)
    _bf16_pair(G)
    _scan_selftest(TS)
    _block_cases(G)
    _model_cases(G)
    _model_autocast_case(G)


if __name__ == "__main__":
    main()
