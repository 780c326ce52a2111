"""Typed compositional pre-processing ("Wernicke" layer): a causal convolution
composes neighbouring tokens, a router (VQ codebook or MoE gate) assigns each
position a bucket, and a per-bucket projection refines it
(cf. src/chaoscontrol/wernicke.py:11-219).  The per-bucket projections are
evaluated as one batched matmul over the stacked expert weights."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .core import RMSNorm


class WernickeLayer(nn.Module):
    def __init__(self, dim: int, k_max: int = 16, window: int = 8, router_type: str = "vq",
                 balance_weight: float = 0.01, expert_dim: Optional[int] = None) -> None:
        super().__init__()
        if router_type not in ("vq", "moe"):
            raise ValueError(f"unsupported router_type: {router_type}")
        self.expert_dim = expert_dim or dim
        self.compose_conv = nn.Conv1d(dim, dim, kernel_size=window, padding=window - 1, bias=False)
        self.compose_norm = RMSNorm(dim)
        self.router_type = router_type
        if router_type == "vq":
            self.codebook = nn.Parameter(torch.randn(k_max, dim) * 0.01)
        else:
            self.router = nn.Linear(dim, k_max, bias=False)
        if self.expert_dim == dim:
            self.bucket_projs = nn.ModuleList(nn.Linear(dim, dim, bias=False) for _ in range(k_max))
        else:
            self.bucket_projs = nn.ModuleList(
                nn.Sequential(nn.Linear(dim, self.expert_dim, bias=False),
                              nn.Linear(self.expert_dim, dim, bias=False)) for _ in range(k_max))
        self.k_max, self.window, self.balance_weight = k_max, window, balance_weight

    def _route(self, h: torch.Tensor):
        if self.router_type == "vq":
            scores = -torch.cdist(h, self.codebook.unsqueeze(0).expand(h.size(0), -1, -1))
        else:
            scores = self.router(h)
        ids = scores.argmax(dim=-1)
        hard = F.one_hot(ids, self.k_max).to(h.dtype)
        soft = F.softmax(scores, dim=-1)
        return ids, hard, hard + soft - soft.detach()      # straight-through routing weights

    def _experts(self, h: torch.Tensor) -> torch.Tensor:
        """``[k, batch, seq, dim]`` outputs of all bucket projections."""
        if self.expert_dim == h.size(-1):
            W = torch.stack([p.weight for p in self.bucket_projs], 0)            # [k, dim, dim]
            return torch.einsum("bsd,ked->kbse", h, W)
        W1 = torch.stack([p[0].weight for p in self.bucket_projs], 0)
        W2 = torch.stack([p[1].weight for p in self.bucket_projs], 0)
        return torch.einsum("kbsm,kem->kbse", torch.einsum("bsd,kmd->kbsm", h, W1), W2)

    def forward(self, x: torch.Tensor):
        """``(refined [B,T,D], bucket_ids [B,T], balance_loss)``."""
        seq = x.size(1)
        h = self.compose_conv(x.transpose(1, 2))[:, :, :seq].transpose(1, 2)
        h = self.compose_norm(h)
        ids, hard, weights = self._route(h)
        frac = hard.sum(dim=(0, 1))
        frac = frac / frac.sum().clamp_min(1e-8)
        balance = ((frac - 1.0 / self.k_max) ** 2).sum() * self.k_max
        refined = torch.einsum("kbse,bsk->bse", self._experts(h), weights)
        return refined, ids, balance

    @torch.no_grad()
    def compression_consequence_update(self, bucket_id: int, quality_delta: float, lr: float = 0.01) -> None:
        """Gradient-free feedback from memory compression: a merge that hurt quality
        makes the router more discriminating for that bucket."""
        if quality_delta >= 0:
            return
        step = lr * abs(quality_delta)
        if self.router_type == "moe":
            self.router.weight.data[bucket_id] *= 1.0 + step
            return
        d = torch.cdist(self.codebook.data, self.codebook.data)
        d[bucket_id, bucket_id] = float("inf")
        away = self.codebook.data[bucket_id] - self.codebook.data[d[bucket_id].argmin()]
        self.codebook.data[bucket_id] += step * away / (away.norm() + 1e-8)


class HierarchicalWernicke(nn.Module):
    """Coarse type then fine subtype; bucket id = ``coarse * k_fine + fine``."""

    def __init__(self, dim: int, k_coarse: int, k_fine: int, window: int = 8, router_type: str = "moe",
                 balance_weight: float = 0.01, expert_dim: Optional[int] = None) -> None:
        super().__init__()
        self.k_coarse, self.k_fine = k_coarse, k_fine
        self.total_buckets = k_coarse * k_fine
        self.balance_weight = balance_weight
        kw = dict(window=window, router_type=router_type, balance_weight=balance_weight, expert_dim=expert_dim)
        self.coarse = WernickeLayer(dim=dim, k_max=k_coarse, **kw)
        self.fine = WernickeLayer(dim=dim, k_max=k_fine, **kw)

    def forward(self, x: torch.Tensor):
        x, c, bc = self.coarse(x)
        x, f, bf = self.fine(x)
        return x, c * self.k_fine + f, bc + bf
