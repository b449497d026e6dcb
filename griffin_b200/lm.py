"""Whole-model harness for the Griffin language model around the CUDA recurrent block.

Only the recurrent temporal-mixing block is this package's product.  The blocks below -- RMSNorm,
gated MLP, local multi-query attention, the residual wrapper and the LM -- are plain torch and exist
so that the whole-model configurations (Griffin-100M training step, data-parallel over the GPUs of
one box) can be measured and so that checkpoints of the reference load unchanged: module and
parameter names follow the reference (griffin/griffin.py:68-116, 557-729, 732-961), including its
``temporal`` alias of the mixing block.  Training/prefill only: the attention block keeps no KV cache.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .modules import RecurrentBlock


class RMSNorm(nn.Module):
    """x / rms(x) * (1 + g)   (griffin/griffin.py:68-80)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.g = nn.Parameter(torch.zeros(dim))

    def forward(self, x: Tensor) -> Tensor:
        return F.rms_norm(x, (x.size(-1),), weight=(1.0 + self.g).to(x.dtype), eps=self.eps)


class GatedMLPBlock(nn.Module):
    """linear3(gelu_tanh(linear1 x) * linear2 x)   (griffin/griffin.py:83-116)."""

    def __init__(self, input_dim: int, hidden_dim: int, final_w_init_variance_scale: float = 1.0):
        super().__init__()
        self.linear1 = nn.Linear(input_dim, hidden_dim)
        self.linear2 = nn.Linear(input_dim, hidden_dim)
        self.linear3 = nn.Linear(hidden_dim, input_dim)
        nn.init.normal_(self.linear1.weight, std=math.sqrt(1.0 / input_dim))
        nn.init.normal_(self.linear2.weight, std=math.sqrt(1.0 / input_dim))
        nn.init.normal_(self.linear3.weight, std=math.sqrt(final_w_init_variance_scale / hidden_dim))
        for lin in (self.linear1, self.linear2, self.linear3):
            nn.init.zeros_(lin.bias)

    def forward(self, x: Tensor) -> Tensor:
        return self.linear3(F.gelu(self.linear1(x), approximate="tanh") * self.linear2(x))


def _rope(x: Tensor, positions: Tensor) -> Tensor:
    """Rotary embedding on [B, T, H, d] with the half-split pairing of griffin/griffin.py:532-554."""
    d = x.size(-1)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.to(torch.float32)[..., None] * inv_freq          # [B, T, d/2]
    ang = torch.cat([ang, ang], dim=-1).to(x.dtype)[:, :, None, :]   # [B, T, 1, d]
    lo, hi = x.chunk(2, dim=-1)
    return x * ang.cos() + torch.cat([-hi, lo], dim=-1) * ang.sin()


class LocalMQAAttention(nn.Module):
    """Causal sliding-window multi-query attention with RoPE (griffin/griffin.py:557-729), without a cache.

    A query at position p of its document sees keys no further back than min(p, window) tokens.
    """

    def __init__(self, input_dim: int, num_heads: int, window_size: int = 1024,
                 final_w_init_variance_scale: float = 1.0, chunk_size: int = 128):
        super().__init__()
        if input_dim % num_heads or (input_dim // num_heads) % 2:
            raise ValueError("input_dim must split into heads of even dimension")
        self.input_dim, self.num_heads, self.head_dim = input_dim, num_heads, input_dim // num_heads
        self.window_size = window_size
        self.chunk_size = chunk_size
        self.query = nn.Linear(input_dim, input_dim, bias=False)
        self.key = nn.Linear(input_dim, self.head_dim, bias=False)
        self.value = nn.Linear(input_dim, self.head_dim, bias=False)
        self.output = nn.Linear(input_dim, input_dim)
        std = math.sqrt(1.0 / input_dim)
        for lin in (self.query, self.key, self.value):
            nn.init.normal_(lin.weight, std=std)
        nn.init.normal_(self.output.weight, std=math.sqrt(final_w_init_variance_scale / input_dim))
        nn.init.zeros_(self.output.bias)

    def forward(self, x: Tensor, cache=None, segment_pos: Optional[Tensor] = None, *,
                active_mask: Optional[Tensor] = None, return_cache: bool = False) -> Tensor:
        if cache is not None or return_cache:
            raise NotImplementedError("the harness attention block keeps no KV cache (training / prefill only)")
        B, T, _ = x.shape
        if segment_pos is None:
            pos = torch.arange(T, device=x.device)[None, :].expand(B, T)
        else:
            pos = segment_pos.to(x.device)
        q = _rope(self.query(x).view(B, T, self.num_heads, self.head_dim), pos)
        k = _rope(self.key(x).view(B, T, 1, self.head_dim), pos)
        v = self.value(x).view(B, T, 1, self.head_dim)
        idx = torch.arange(T, device=x.device)
        back = pos.clamp(max=self.window_size)                                    # [B, T]
        allowed = (idx[None, None, :] <= idx[None, :, None]) & (idx[None, None, :] >= (idx[None, :] - back)[..., None])
        if active_mask is not None:
            allowed = allowed & active_mask[:, None, :] & active_mask[:, :, None]
        if segment_pos is None and active_mask is None:
            allowed = allowed[:1]
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                             attn_mask=allowed[:, None], enable_gqa=True)
        out = torch.nan_to_num(out).transpose(1, 2).reshape(B, T, self.input_dim)
        out = self.output(out)
        if active_mask is not None:
            out = torch.where(active_mask[..., None], out, torch.zeros_like(out))
        return out


def _autocast_once(h: Tensor) -> Tensor:
    """Under CUDA autocast every projection that consumes ``h`` would cast it to the autocast dtype on its own
    (autocast caches casts of parameters, not of activations); doing the same cast once here gives identical
    values and saves the repeated passes."""
    if h.is_cuda and h.dtype == torch.float32 and torch.is_autocast_enabled("cuda"):
        return h.to(torch.get_autocast_dtype("cuda"))
    return h


class ResidualBlock(nn.Module):
    """Pre-norm temporal mixing + gated MLP (griffin/griffin.py:732-809)."""

    def __init__(self, input_dim: int, expansion_factor: int, rnn_width: int, *, temporal_block_type: str = "recurrent",
                 attention_heads: int = 1, attention_window_size: int = 1024, gate_blocks: int = 16,
                 final_w_init_variance_scale: float = 1.0, scan_mode: str = "cuda", attention_chunk_size: int = 128):
        super().__init__()
        self.temporal_block_type = temporal_block_type
        self.norm1 = RMSNorm(input_dim)
        if temporal_block_type == "recurrent":
            self.recurrent = RecurrentBlock(input_dim, rnn_width, gate_blocks=gate_blocks,
                                            final_w_init_variance_scale=final_w_init_variance_scale, scan_mode=scan_mode)
            self.temporal = self.recurrent
        elif temporal_block_type == "attention":
            self.attention = LocalMQAAttention(input_dim, attention_heads, attention_window_size,
                                               final_w_init_variance_scale, attention_chunk_size)
            self.temporal = self.attention
        else:
            raise ValueError(f"Unknown temporal block type: {temporal_block_type}")
        self.norm2 = RMSNorm(input_dim)
        self.mlp = GatedMLPBlock(input_dim, input_dim * expansion_factor, final_w_init_variance_scale)

    def forward(self, x: Tensor, segment_pos: Optional[Tensor] = None, *, active_mask: Optional[Tensor] = None) -> Tensor:
        x = x + self.temporal(_autocast_once(self.norm1(x)), None, segment_pos, active_mask=active_mask)
        x = x + self.mlp(_autocast_once(self.norm2(x)))
        if active_mask is not None:
            x = torch.where(active_mask[..., None], x, torch.zeros_like(x))
        return x


class GriffinModel(nn.Module):
    """Griffin LM returning logits (griffin/griffin.py:827-961); blocks repeat recurrent, recurrent, attention."""

    def __init__(self, vocab_size: int, input_dim: int = 1024, mlp_expansion_factor: int = 3, rnn_width: int = 1536,
                 depth: int = 12, *, attention_heads: Optional[int] = None, attention_window_size: int = 1024,
                 block_types: Optional[Sequence[str]] = None, gate_blocks: int = 16, tie_embeddings: bool = True,
                 scan_mode: str = "cuda", attention_chunk_size: int = 128):
        super().__init__()
        if depth <= 0:
            raise ValueError("depth must be positive")
        pattern = ("recurrent", "recurrent", "attention")
        self.block_types = tuple(block_types) if block_types is not None else tuple(pattern[i % 3] for i in range(depth))
        if len(self.block_types) != depth:
            raise ValueError("block_types must contain exactly depth entries")
        if attention_heads is None:
            attention_heads = max(1, input_dim // 128)
            while input_dim % attention_heads or (input_dim // attention_heads) % 2:
                attention_heads -= 1
        self.vocab_size, self.input_dim = vocab_size, input_dim
        self.embd = nn.Embedding(vocab_size, input_dim)
        nn.init.normal_(self.embd.weight, std=math.sqrt(1.0 / input_dim))
        self.embedding_scale = math.sqrt(input_dim)
        self.layers = nn.ModuleList([
            ResidualBlock(input_dim, mlp_expansion_factor, rnn_width, temporal_block_type=kind,
                          attention_heads=attention_heads, attention_window_size=attention_window_size,
                          gate_blocks=gate_blocks, final_w_init_variance_scale=2.0 / depth, scan_mode=scan_mode,
                          attention_chunk_size=attention_chunk_size)
            for kind in self.block_types])
        self.final_norm = RMSNorm(input_dim)
        self.lm_head = nn.Linear(input_dim, vocab_size, bias=False)
        nn.init.normal_(self.lm_head.weight, std=math.sqrt(1.0 / input_dim))
        if tie_embeddings:
            self.lm_head.weight = self.embd.weight

    def forward(self, token_ids: Tensor, segment_pos: Optional[Tensor] = None, *, token_mask: Optional[Tensor] = None,
                pad_vocab: bool = False) -> Tensor:
        """Logits [B, T, vocab].  ``pad_vocab=True`` (not in the reference) returns them with the vocabulary axis
        padded to a multiple of 8 and -inf in the padding, which a cross-entropy treats as absent classes; a
        training loop that takes them this way skips the slice and its zero-filling backward."""
        if segment_pos is not None and segment_pos.shape != token_ids.shape:
            raise ValueError("segment_pos must have the same [batch, sequence] shape as token_ids")
        x = self.embd(token_ids) * self.embedding_scale
        if token_mask is not None:
            token_mask = token_mask.to(device=token_ids.device, dtype=torch.bool)
            x = torch.where(token_mask[..., None], x, torch.zeros_like(x))
        for layer in self.layers:
            x = layer(x, segment_pos, active_mask=token_mask)
        return self._logits(self.final_norm(x), pad_vocab)

    def _logits(self, h: Tensor, keep_padding: bool = False) -> Tensor:
        """lm_head(h). On CUDA with half-precision autocast and a vocabulary that is not a multiple of 8, the
        weight is zero-padded to the next multiple while it is cast, so the GEMMs (forward and both backward
        ones) take the aligned tensor-core kernels; the extra columns are sliced off (a view, same values)."""
        weight = self.lm_head.weight
        pad = -self.vocab_size % 8
        if pad and h.is_cuda and torch.is_autocast_enabled("cuda"):
            half = torch.get_autocast_dtype("cuda")
            wide = F.pad(weight.to(half), (0, 0, 0, pad))
            if keep_padding:   # -inf through the GEMM's own bias epilogue
                mask = torch.zeros(self.vocab_size + pad, device=h.device, dtype=half)
                mask[self.vocab_size:] = float("-inf")
                return F.linear(h.to(half), wide, mask)
            return F.linear(h.to(half), wide)[..., : self.vocab_size]
        logits = F.linear(h, weight)
        if keep_padding and pad:
            logits = F.pad(logits, (0, pad), value=float("-inf"))
        return logits
