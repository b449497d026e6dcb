"""The whole-model harness (plain-torch blocks around the CUDA recurrent block) against the reference's
stored results: the local attention block on CPU, the tiny hybrid LM on the GPU."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, params_of
from oracle.rglru_oracle import rel_l2


def test_local_attention_matches_reference_cpu():
    from griffin_b200.lm import LocalMQAAttention
    case = load_golden("attention_block")
    attn = LocalMQAAttention(16, 2, window_size=5, chunk_size=3)
    attn.load_state_dict(params_of(case))
    with torch.no_grad():
        plain = attn(case["x"])
        seg = attn(case["x"], segment_pos=case["segment_pos"])
    torch.testing.assert_close(plain, case["plain"], atol=2e-6, rtol=2e-5)
    torch.testing.assert_close(seg, case["seg"], atol=2e-6, rtol=2e-5)


def test_model_state_dict_is_the_reference_layout():
    from griffin_b200.lm import GriffinModel
    case = load_golden("model_tiny")
    model = GriffinModel(23, 8, 2, 12, 3, attention_heads=2, attention_window_size=4)
    model.load_state_dict(params_of(case), strict=True)
    assert model.block_types == ("recurrent", "recurrent", "attention")
    assert model.lm_head.weight is model.embd.weight


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["plain", "seg"])
def test_tiny_model_logits_loss_and_gradients_gpu(tag):
    from griffin_b200.lm import GriffinModel
    case = load_golden("model_tiny")
    model = GriffinModel(23, 8, 2, 12, 3, attention_heads=2, attention_window_size=4)
    model.load_state_dict(params_of(case), strict=True)
    model = model.cuda()
    tokens, targets = case["tokens"].cuda(), case["targets"].cuda()
    seg = case["segment_pos"].cuda() if tag == "seg" else None
    logits = model(tokens, segment_pos=seg)
    loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 23), targets.reshape(-1))
    loss.backward()
    torch.testing.assert_close(logits.cpu(), case[f"{tag}.logits"], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(loss.detach().cpu().reshape(1), case[f"{tag}.loss"], atol=1e-5, rtol=1e-5)
    grads = dict(model.named_parameters())
    for key in case:
        if key.startswith(f"{tag}.g."):
            name = key[len(tag) + 3:]
            assert rel_l2(grads[name].grad, case[key]) <= 1e-5, name


@pytest.mark.gpu
def test_padded_vocabulary_head_matches_plain_linear_gpu():
    """Under autocast the head pads an odd vocabulary for the GEMM; values and the weight gradient must not change."""
    from griffin_b200.lm import GriffinModel
    torch.manual_seed(5)
    model = GriffinModel(1003, 64, 2, 64, 1, attention_heads=2, block_types=("attention",)).cuda()
    h = torch.randn(4, 48, 64, device="cuda")
    dlogits = torch.randn(4, 48, 1003, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        padded = model._logits(h)
        plain = torch.nn.functional.linear(h, model.lm_head.weight)
    assert padded.shape == plain.shape == (4, 48, 1003) and padded.dtype == torch.bfloat16
    assert rel_l2(padded.float(), plain.float()) <= 4e-3
    (g_padded,) = torch.autograd.grad((padded.float() * dlogits).sum(), model.lm_head.weight)
    (g_plain,) = torch.autograd.grad((plain.float() * dlogits).sum(), model.lm_head.weight)
    assert g_padded.shape == model.lm_head.weight.shape
    assert rel_l2(g_padded, g_plain) <= 4e-3
    # padded form: same loss and the same weight gradient as the sliced form
    targets = torch.randint(0, 1003, (4 * 48,), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        wide = model._logits(h, keep_padding=True)
        padded = model._logits(h)
    assert wide.shape == (4, 48, 1008) and torch.isinf(wide[..., 1003:]).all()
    ce = torch.nn.functional.cross_entropy
    loss_wide, loss_plain = ce(wide.float().reshape(-1, 1008), targets), ce(padded.float().reshape(-1, 1003), targets)
    torch.testing.assert_close(loss_wide, loss_plain, atol=1e-6, rtol=1e-6)
    (gw,) = torch.autograd.grad(loss_wide, model.lm_head.weight)
    (gp,) = torch.autograd.grad(loss_plain, model.lm_head.weight)
    assert torch.isfinite(gw).all() and rel_l2(gw, gp) <= 1e-5
    exact = model._logits(h)                       # no autocast: the plain fp32 path
    assert exact.dtype == torch.float32 and rel_l2(padded.float(), exact) <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("fold_merge", [False, True])
def test_autocast_model_against_reference_autocast_gpu(fold_merge):
    """The harness the way the training benchmark runs it -- CUDA bf16 autocast, the GeLU-branch product folded
    into the scan kernels, the vocabulary padded for the head -- against the reference's own autocast step
    (train.py:254-267 of the reference, run on CPU by tests/golden/make_golden.py): logits, loss and gradients.
    Both sides round to bf16 at different points of the graph, so the comparison is norm-wise at 2e-2
    (the loss, a mean over 192 tokens, at 2e-3)."""
    from griffin_b200.lm import GriffinModel
    case = load_golden("model_autocast_bf16")
    vocab = 131
    model = GriffinModel(vocab, 16, 2, 128, 3, attention_heads=2, attention_window_size=16, gate_blocks=2)
    model.load_state_dict(params_of(case), strict=True)
    for layer in model.layers:
        if hasattr(layer, "recurrent"):
            layer.recurrent.fold_merge = fold_merge
    model = model.cuda()
    tokens = case["tokens"].cuda()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        logits = model(tokens[:, :-1], pad_vocab=True)
    assert logits.shape[-1] == 136 and torch.isinf(logits[..., vocab:]).all()
    loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.size(-1)), tokens[:, 1:].reshape(-1))
    loss.backward()
    assert rel_l2(logits[..., :vocab].float(), case["logits"]) <= 2e-2
    torch.testing.assert_close(loss.detach().cpu().reshape(1), case["loss"], atol=0.0, rtol=2e-3)
    grads = dict(model.named_parameters())
    worst = {}
    for key in case:
        if key.startswith("g."):
            err = rel_l2(grads[key[2:]].grad, case[key])
            if not err <= 2e-2:
                worst[key] = err
    assert not worst, worst
