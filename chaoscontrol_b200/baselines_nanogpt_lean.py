"""Lean modded-NanoGPT-style transformer baseline: RoPE (interleaved pairs), RMSNorm,
QK-norm, ReLU^2 MLP, SDPA, untied head (cf. src/chaoscontrol/baselines_nanogpt_lean.py:26-244).
Design defaults: d_model 256, 4 heads, 8 layers, ffn x4, ~10.5 M parameters at V = 8192."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from .baselines import _BaselineLM
from .models.core import RMSNorm

__all__ = ["relu_squared", "apply_rope", "NanoGPTLeanBlock", "NanoGPTLeanLM", "build_nanogpt_lean"]


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    return F.relu(x).square()


def _build_rope_cache(head_dim: int, seq_len: int, base: float = 10_000.0) -> torch.Tensor:
    """``[2, seq_len, head_dim]`` (cos, sin); each frequency occupies a channel pair (2i, 2i+1)."""
    inv = 1.0 / (base ** (2.0 * torch.arange(head_dim // 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32), inv).repeat_interleave(2, dim=-1)
    return torch.stack([ang.cos(), ang.sin()], 0)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotates channel pairs ``(2i, 2i+1)`` of ``x [..., seq, head_dim]``."""
    c, s = cos[..., 0::2].to(x.dtype), sin[..., 0::2].to(x.dtype)
    even, odd = x[..., 0::2], x[..., 1::2]
    return torch.stack([even * c - odd * s, odd * c + even * s], dim=-1).flatten(-2)


class NanoGPTLeanBlock(nn.Module):
    def __init__(self, d_model: int, n_head: int, ffn_mult: int) -> None:
        super().__init__()
        assert d_model % n_head == 0
        self.n_head, self.head_dim = n_head, d_model // n_head
        self.attn_norm = RMSNorm(d_model)
        self.qkv = nn.Linear(d_model, 3 * d_model, bias=False)
        self.q_norm, self.k_norm = RMSNorm(self.head_dim), RMSNorm(self.head_dim)
        self.out_proj = nn.Linear(d_model, d_model, bias=False)
        self.mlp_norm = RMSNorm(d_model)
        self.mlp_in = nn.Linear(d_model, ffn_mult * d_model, bias=False)
        self.mlp_out = nn.Linear(ffn_mult * d_model, d_model, bias=False)

    def forward(self, x: torch.Tensor, rope_cache: torch.Tensor) -> torch.Tensor:
        B, T, D = x.shape
        q, k, v = (t.view(B, T, self.n_head, self.head_dim).transpose(1, 2)
                   for t in self.qkv(self.attn_norm(x)).chunk(3, dim=-1))
        q = self.q_norm(apply_rope(q, rope_cache[0], rope_cache[1]))
        k = self.k_norm(apply_rope(k, rope_cache[0], rope_cache[1]))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D)
        x = x + self.out_proj(a)
        return x + self.mlp_out(relu_squared(self.mlp_in(self.mlp_norm(x))))


class NanoGPTLeanLM(_BaselineLM):
    def __init__(self, vocab_size: int, d_model: int = 256, n_head: int = 4, n_layer: int = 8, ffn_mult: int = 4,
                 max_seq_len: int = 2048, activation_checkpoint: bool = False) -> None:
        super().__init__(vocab_size, d_model)
        self.activation_checkpoint = activation_checkpoint
        self.blocks = nn.ModuleList(NanoGPTLeanBlock(d_model, n_head, ffn_mult) for _ in range(n_layer))
        self.register_buffer("rope_cache", _build_rope_cache(d_model // n_head, max_seq_len), persistent=False)

    def encode(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Pre-final-norm hidden state; identical to ``forward()["hidden"]``."""
        T = input_ids.shape[1]
        if T > self.rope_cache.shape[1]:
            self.rope_cache = _build_rope_cache(self.rope_cache.shape[-1], T).to(self.rope_cache.device)
        rope = self.rope_cache[:, :T]
        h = self.embed(input_ids)
        for block in self.blocks:
            if self.activation_checkpoint and self.training:
                h = _checkpoint(block, h, rope, use_reentrant=False)
            else:
                h = block(h, rope)
        return h


def build_nanogpt_lean(vocab_size: int = 8192, d_model: int = 256, n_head: int = 4, n_layer: int = 8,
                       ffn_mult: int = 4, max_seq_len: int = 2048, activation_checkpoint: bool = False) -> NanoGPTLeanLM:
    return NanoGPTLeanLM(vocab_size=vocab_size, d_model=d_model, n_head=n_head, n_layer=n_layer, ffn_mult=ffn_mult,
                         max_seq_len=max_seq_len, activation_checkpoint=activation_checkpoint)
