"""Baseline language models that share the train / eval path with
``CareStudentLM`` (same ``{"logits", "hidden"}`` forward contract, same
duck-typed ``outer_model`` / ``wernicke`` / ``semantic_tier`` attributes):

``SimpleTransformerLM``  minimal pre-norm causal transformer
``Mamba2LM``             Mamba-2 stack: the ``mamba_ssm`` package's block when it is
                         installed, else (``impl="torch"``) an in-tree selective diagonal
                         SSM block with the same interface
(cf. src/chaoscontrol/baselines.py:9-136).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .models.core import FeedForward, RMSNorm

__all__ = ["SimpleTransformerLM", "TransformerBlock", "CausalSelfAttention", "Mamba2LM", "SelectiveSSMBlock"]


def _no_stats() -> dict[str, torch.Tensor]:
    return {"lambda_max": torch.tensor(0.0), "sv_log_var": torch.tensor(0.0)}


class _BaselineLM(nn.Module):
    """Embedding, final norm, untied head and the duck-typed attributes."""

    def __init__(self, vocab_size: int, dim: int) -> None:
        super().__init__()
        self.vocab_size, self.dim = vocab_size, dim
        self.embed = nn.Embedding(vocab_size, dim)
        self.final_norm = RMSNorm(dim)
        self.lm_head = nn.Linear(dim, vocab_size, bias=False)
        self.outer_model = self.wernicke = self.semantic_tier = None
        self.wernicke_balance_weight = 0.0

    def artifact_bytes(self) -> int:
        return int(sum(p.numel() for p in self.parameters()) * 2)

    def encode(self, input_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, input_ids: torch.Tensor, *, return_jacobian_stats: bool = False):
        hidden = self.encode(input_ids)
        out = {"logits": self.lm_head(self.final_norm(hidden)), "hidden": hidden}
        if return_jacobian_stats:
            out["jacobian_stats"] = _no_stats()
        return out


class CausalSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int) -> None:
        super().__init__()
        assert dim % num_heads == 0
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.qkv = nn.Linear(dim, dim * 3, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.shape
        q, k, v = (t.transpose(1, 2) for t in self.qkv(x).view(B, T, 3, self.num_heads, self.head_dim).unbind(2))
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.out_proj(out.transpose(1, 2).reshape(B, T, C))


class TransformerBlock(nn.Module):
    def __init__(self, dim: int, num_heads: int, ff_mult: int = 2) -> None:
        super().__init__()
        self.attn_norm, self.ff_norm = RMSNorm(dim), RMSNorm(dim)
        self.attn = CausalSelfAttention(dim, num_heads)
        self.ff = FeedForward(dim, ff_mult)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.attn_norm(x))
        return x + self.ff(self.ff_norm(x))


class SimpleTransformerLM(_BaselineLM):
    def __init__(self, vocab_size: int = 256, dim: int = 128, num_layers: int = 4, num_heads: int = 4,
                 ff_mult: int = 2) -> None:
        super().__init__(vocab_size, dim)
        self.layers = nn.ModuleList(TransformerBlock(dim, num_heads, ff_mult) for _ in range(num_layers))

    def encode(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = self.embed(input_ids)
        for layer in self.layers:
            x = layer(x)
        return x


class SelectiveSSMBlock(nn.Module):
    """In-tree stand-in for a Mamba-2 mixer: expand, short causal depthwise conv, an
    input-dependent diagonal recurrence ``h <- exp(-softplus(dt) * a) h + dt * B x``
    per channel with a ``d_state``-wide state, read out by ``C``, gated and projected back."""

    def __init__(self, d_model: int, d_state: int = 64, d_conv: int = 4, expand: int = 2) -> None:
        super().__init__()
        self.d_inner, self.d_state = expand * d_model, d_state
        self.in_proj = nn.Linear(d_model, 2 * self.d_inner, bias=False)
        self.conv = nn.Conv1d(self.d_inner, self.d_inner, d_conv, groups=self.d_inner, padding=d_conv - 1)
        self.bc_dt = nn.Linear(self.d_inner, 2 * d_state + 1, bias=False)
        self.a_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32)))
        self.dt_bias = nn.Parameter(torch.zeros(1))
        self.norm = RMSNorm(self.d_inner)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, _ = x.shape
        u, z = self.in_proj(x).chunk(2, dim=-1)
        u = F.silu(self.conv(u.transpose(1, 2))[:, :, :T].transpose(1, 2))
        Bm, Cm, dt = self.bc_dt(u).split([self.d_state, self.d_state, 1], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias)                                  # [B, T, 1]
        decay = torch.exp(-dt * torch.exp(self.a_log))                              # [B, T, N]
        # log-space cumulative form of the diagonal recurrence (numerically safe for short T chunks)
        h = torch.zeros(B, self.d_inner, self.d_state, device=x.device, dtype=torch.float32)
        ys = []
        uf, Bf, Cf = u.float(), Bm.float(), Cm.float()
        for t in range(T):
            h = h * decay[:, t].unsqueeze(1) + (dt[:, t] * uf[:, t]).unsqueeze(-1) * Bf[:, t].unsqueeze(1)
            ys.append(torch.einsum("bdn,bn->bd", h, Cf[:, t]))
        y = torch.stack(ys, 1).to(x.dtype)
        return self.out_proj(self.norm(y) * F.silu(z))


class Mamba2LM(_BaselineLM):
    """Pre-norm + residual around each mixer (the package's block has neither)."""

    def __init__(self, vocab_size: int = 256, dim: int = 128, num_layers: int = 4, d_state: int = 64, d_conv: int = 4,
                 expand: int = 2, impl: str = "auto") -> None:
        super().__init__(vocab_size, dim)
        block = None
        if impl in ("auto", "mamba_ssm"):
            try:
                from mamba_ssm import Mamba2 as block           # type: ignore
            except ImportError:
                if impl == "mamba_ssm":
                    raise ImportError("Mamba-2 baseline requires the mamba-ssm package (>= 2.3.0); "
                                      "pass impl='torch' for the in-tree block")
        if block is None:
            if impl == "auto":
                raise ImportError("Mamba-2 baseline requires mamba-ssm package. Install mamba-ssm>=2.3.0, or pass "
                                  "impl='torch' for the in-tree selective-SSM block")
            block = SelectiveSSMBlock
        self.layers = nn.ModuleList(block(d_model=dim, d_state=d_state, d_conv=d_conv, expand=expand)
                                    for _ in range(num_layers))
        self.norms = nn.ModuleList(RMSNorm(dim) for _ in range(num_layers))

    def encode(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = self.embed(input_ids)
        for norm, layer in zip(self.norms, self.layers):
            x = x + layer(norm(x))
        return x
