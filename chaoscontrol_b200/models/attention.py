"""Attention components of the research path: the rolling KV window, the local
attention sidecar (sliding window / top-k / random-k), the SSM block with that
sidecar, and the pure-attention control block with RoPE
(cf. src/chaoscontrol/local_attn.py:9-217, model.py:143-570).  Parameter names
match the reference; the masked score path is one fused SDPA call."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .core import CareSSMCore, FeedForward, RMSNorm


class RollingKVCache:
    """The last ``window`` (key, value) pairs of a single-token decoding loop."""

    def __init__(self, window: int, dim: int) -> None:
        self.window, self.dim = window, dim
        self._keys: list[torch.Tensor] = []
        self._values: list[torch.Tensor] = []

    def write(self, k: torch.Tensor, v: torch.Tensor) -> None:
        self._keys.append(k.detach())
        self._values.append(v.detach())
        if len(self._keys) > self.window:
            del self._keys[0], self._values[0]

    def last(self, w: int):
        """``(keys [B,w,D], values [B,w,D], mask [B,w])`` left-aligned, zero padded."""
        n = len(self._keys)
        if n == 0:
            z = torch.zeros(1, w, self.dim)
            return z, z.clone(), torch.zeros(1, w, dtype=torch.bool)
        fill = min(n, w)
        ks = torch.stack(self._keys[n - fill:], dim=1)
        vs = torch.stack(self._values[n - fill:], dim=1)
        B = ks.shape[0]
        pad = ks.new_zeros(B, w - fill, self.dim)
        mask = torch.zeros(B, w, dtype=torch.bool, device=ks.device)
        mask[:, :fill] = True
        return torch.cat([ks, pad], 1), torch.cat([vs, pad], 1), mask

    def reset(self) -> None:
        self._keys.clear()
        self._values.clear()


class LocalAttention(nn.Module):
    def __init__(self, model_dim: int, attn_dim: int, num_heads: int = 1) -> None:
        super().__init__()
        self.num_heads, self.attn_dim, self.head_dim = num_heads, attn_dim, attn_dim // num_heads
        self.q_proj = nn.Linear(model_dim, attn_dim, bias=False)
        self.out_proj = nn.Linear(attn_dim, model_dim, bias=False)

    def _heads(self, t: torch.Tensor) -> torch.Tensor:
        B, S, _ = t.shape
        return t.view(B, S, self.num_heads, self.head_dim).transpose(1, 2)

    def forward(self, query, keys, values, mask):
        """One query ``[B, D]`` against a window of pre-projected keys / values."""
        q = self._heads(self.q_proj(query).unsqueeze(1))
        out = F.scaled_dot_product_attention(q, self._heads(keys), self._heads(values),
                                             attn_mask=mask[:, None, None, :])
        return self.out_proj(out.transpose(1, 2).reshape(query.shape[0], self.attn_dim))

    def forward_sequence(self, query_seq, keys_seq, values_seq, window: int, topk: int = 0,
                         topk_random: bool = False):
        """Strictly-causal attention over a whole sequence: sliding window of
        ``window`` previous positions, or ``topk`` previous positions chosen by
        score (or at random, as the control).  Position 0 has nothing to attend
        to and receives zeros."""
        B, S, _ = query_seq.shape
        if window <= 0 and topk <= 0:
            return torch.zeros_like(query_seq)
        dev = query_seq.device
        q, k, v = self._heads(self.q_proj(query_seq)), self._heads(keys_seq), self._heads(values_seq)
        pos = torch.arange(S, device=dev)
        causal = pos[None, :] < pos[:, None]
        if topk > 0:
            scores = (q @ k.transpose(-2, -1)) / self.head_dim ** 0.5
            if topk_random:
                scores = torch.rand_like(scores)
            scores = scores.masked_fill(~causal, float("-inf"))
            kk = min(topk, S)
            thresh = scores.topk(kk, dim=-1).values[..., -1:]
            mask = causal & (scores >= thresh)
        else:
            mask = (causal & (pos[:, None] - pos[None, :] <= window)).expand(B, self.num_heads, S, S)
        has_valid = mask.any(dim=-1, keepdim=True)
        safe = mask | ~has_valid                   # rows with no key: attend anywhere, zeroed below
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=safe)
        out = out * has_valid.to(out.dtype)
        return self.out_proj(out.transpose(1, 2).reshape(B, S, self.attn_dim))


def _bundle(y, stats, final_state, want_stats, want_final):
    if want_stats and want_final:
        return y, stats, final_state
    if want_stats:
        return y, stats
    if want_final:
        return y, final_state
    return y


class CareSSMHybridBlock(nn.Module):
    """SSM block plus a gated local-attention sidecar; the gate bias starts at -4
    so the block begins as a plain SSM block."""

    def __init__(self, dim: int, ff_mult: int = 2, *, a_mode: str = "diag", a_full_rank: int = 8,
                 a_full_gamma: float = 0.05, ssm_delta_rank: int = 0, local_attn_window: int = 64,
                 local_attn_heads: int = 1, local_attn_dim: int = 64, local_attn_topk: int = 0,
                 local_attn_topk_random: bool = False) -> None:
        super().__init__()
        self.input_norm, self.ff_norm = RMSNorm(dim), RMSNorm(dim)
        self.ff = FeedForward(dim, ff_mult)
        self.core = CareSSMCore(dim, a_mode=a_mode, a_full_rank=a_full_rank, a_full_gamma=a_full_gamma,
                                delta_rank=ssm_delta_rank)
        self.rich_b = None
        self.local_attn_window, self.local_attn_dim = local_attn_window, local_attn_dim
        self.local_attn_topk, self.local_attn_topk_random = local_attn_topk, local_attn_topk_random
        self.local_attn = LocalAttention(dim, local_attn_dim, local_attn_heads)
        self.k_proj = nn.Linear(dim, local_attn_dim, bias=False)
        self.v_proj = nn.Linear(dim, local_attn_dim, bias=False)
        self.gate_proj = nn.Linear(dim, 1, bias=False)
        self.gate_bias = nn.Parameter(torch.tensor(-4.0))

    def _init_kv_cache(self) -> RollingKVCache:
        return RollingKVCache(self.local_attn_window, self.local_attn_dim)

    def _gate(self, x):
        return torch.sigmoid(self.gate_proj(x) + self.gate_bias)

    def step(self, x, state, *, kv_cache: Optional[RollingKVCache] = None):
        y, new_state = self.core.step(self.input_norm(x), state)
        base = x + y
        out = base
        if kv_cache is not None:
            keys, values, mask = kv_cache.last(self.local_attn_window)
            if mask.any():
                out = base + self._gate(base) * self.local_attn(base, keys.to(base), values.to(base),
                                                                mask.to(base.device))
            kv_cache.write(self.k_proj(base), self.v_proj(base))
        return out + self.ff(self.ff_norm(out)), new_state

    def forward(self, x, *, return_jacobian_stats: bool = False, initial_state=None,
                return_final_state: bool = False):
        y, final_state = self.core(self.input_norm(x), initial_state=initial_state, return_final_state=True)
        h = x + y
        attn = self.local_attn.forward_sequence(h, self.k_proj(h), self.v_proj(h),
                                                window=self.local_attn_window, topk=self.local_attn_topk,
                                                topk_random=self.local_attn_topk_random)
        h = h + self._gate(h) * attn
        out = h + self.ff(self.ff_norm(h))
        stats = ({"lambda_max": torch.tensor(0.0), "sv_log_var": torch.tensor(0.0)}
                 if return_jacobian_stats else None)
        return _bundle(out, stats, final_state, return_jacobian_stats, return_final_state)


class AttentionControlBlock(nn.Module):
    """Causal multi-head attention with RoPE behind the SSM block's interface (the
    scientific control for "SSM stack vs attention stack").  Its "state" is a
    dummy tensor so callers can thread it like a recurrence state."""

    def __init__(self, dim: int, ff_mult: int = 2, *, num_heads: int = 8, attn_dropout: float = 0.0,
                 rope_base: float = 10000.0) -> None:
        super().__init__()
        if dim % num_heads:
            raise ValueError(f"dim ({dim}) must be divisible by num_heads ({num_heads})")
        if (dim // num_heads) % 2:
            raise ValueError(f"head_dim ({dim // num_heads}) must be even for RoPE; got dim={dim}, "
                             f"num_heads={num_heads}")
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.attn_dropout, self.rope_base = attn_dropout, rope_base
        self.input_norm, self.ff_norm = RMSNorm(dim), RMSNorm(dim)
        self.ff = FeedForward(dim, ff_mult)
        self.qkv_proj = nn.Linear(dim, 3 * dim, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)
        self.register_buffer("_rope_cos", torch.empty(0, self.head_dim), persistent=False)
        self.register_buffer("_rope_sin", torch.empty(0, self.head_dim), persistent=False)

    def _ensure_rope_cache(self, seq_len: int, device) -> None:
        if self._rope_cos.shape[0] >= seq_len and self._rope_cos.device == torch.device(device):
            return
        inv = 1.0 / (self.rope_base ** (torch.arange(0, self.head_dim, 2, device=device).float() / self.head_dim))
        ang = torch.outer(torch.arange(seq_len, device=device).float(), inv)
        ang = torch.cat([ang, ang], dim=-1)
        self._rope_cos, self._rope_sin = ang.cos(), ang.sin()

    def apply_rope(self, t: torch.Tensor, offset: int = 0) -> torch.Tensor:
        S = t.shape[-2]
        self._ensure_rope_cache(offset + S, t.device)
        cos = self._rope_cos[offset: offset + S].to(t.dtype)
        sin = self._rope_sin[offset: offset + S].to(t.dtype)
        half = t.shape[-1] // 2
        rot = torch.cat([-t[..., half:], t[..., :half]], dim=-1)
        return t * cos + rot * sin

    def _attn(self, x: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        q, k, v = (t.view(B, S, self.num_heads, self.head_dim).transpose(1, 2)
                   for t in self.qkv_proj(x).chunk(3, dim=-1))
        out = F.scaled_dot_product_attention(self.apply_rope(q), self.apply_rope(k), v, is_causal=True,
                                             dropout_p=self.attn_dropout if self.training else 0.0)
        return self.out_proj(out.transpose(1, 2).reshape(B, S, self.dim))

    def step(self, x, state):
        raise NotImplementedError("AttentionControlBlock has no single-token step (no KV cache); "
                                  "use forward() on full sequences")

    def forward(self, x, *, return_jacobian_stats: bool = False, initial_state=None,
                return_final_state: bool = False):
        x = x + self._attn(self.input_norm(x))
        x = x + self.ff(self.ff_norm(x))
        stats = ({"lambda_max": torch.tensor(0.0), "sv_log_var": torch.tensor(0.0)}
                 if return_jacobian_stats else None)
        final = x.new_zeros(x.shape[0], self.dim) if return_final_state else None
        return _bundle(x, stats, final, return_jacobian_stats, return_final_state)
