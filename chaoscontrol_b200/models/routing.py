"""Input-dependent update networks ("rich B") and straight-through vector
quantisation (cf. src/chaoscontrol/routing.py:10-124, vq.py:11-46).  Module
and parameter names are the reference's so checkpoints load unchanged."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .core import RMSNorm


class RichBNN(nn.Module):
    """``B(x, h)``: a two-layer bottleneck MLP over ``concat(x, h)``, tanh-bounded."""

    def __init__(self, dim: int, bottleneck: int = 32) -> None:
        super().__init__()
        self.net = nn.Sequential(nn.Linear(dim * 2, bottleneck, bias=False), nn.SiLU(),
                                 nn.Linear(bottleneck, dim, bias=False), nn.Tanh())

    def forward(self, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        return self.net(torch.cat([x, h], dim=-1))


def _mlp(d_in: int, d_mid: int, d_out: int) -> nn.Sequential:
    return nn.Sequential(nn.Linear(d_in, d_mid, bias=False), nn.SiLU(), nn.Linear(d_mid, d_out, bias=False))


class DistributedB(nn.Module):
    """K sub-networks, each seeing its own learned view of the state.

    ``hub``: a central MLP aggregates the partial signals; ``assembly``: the
    partials exchange lateral messages for ``settling_steps`` rounds and are
    averaged; ``hybrid``: message passing, then a hub that sees the partials
    before and after settling."""

    def __init__(self, dim: int, num_subnets: int = 4, bottleneck: int = 32, topology: str = "hub",
                 settling_steps: int = 2) -> None:
        super().__init__()
        if topology not in ("hub", "assembly", "hybrid"):
            raise ValueError(f"unsupported topology: {topology}")
        self.dim, self.num_subnets, self.topology, self.settling_steps = dim, num_subnets, topology, settling_steps
        sub = max(dim // num_subnets, 4)
        self.view_projs = nn.ModuleList(nn.Linear(dim, dim, bias=False) for _ in range(num_subnets))
        self.subnets = nn.ModuleList(_mlp(dim * 2, sub, dim) for _ in range(num_subnets))
        if topology in ("assembly", "hybrid"):
            self.lateral = nn.Linear(dim * num_subnets, dim, bias=False)
            self.settling_norm = RMSNorm(dim)
        if topology in ("hub", "hybrid"):
            self.hub = _mlp(dim * num_subnets * (2 if topology == "hybrid" else 1), bottleneck, dim)
        self.out_act = nn.Tanh()

    def _settle(self, parts: list[torch.Tensor]) -> list[torch.Tensor]:
        for _ in range(self.settling_steps):
            msg = self.settling_norm(self.lateral(torch.cat(parts, dim=-1)))
            parts = [p + msg for p in parts]
        return parts

    def forward(self, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        parts = [net(torch.cat([x, view(h)], dim=-1)) for net, view in zip(self.subnets, self.view_projs)]
        if self.topology == "hub":
            return self.out_act(self.hub(torch.cat(parts, dim=-1)))
        settled = self._settle(parts)
        if self.topology == "assembly":
            return self.out_act(torch.stack(settled, 0).mean(0))
        return self.out_act(self.hub(torch.cat(parts + settled, dim=-1)))


def vector_quantize(x: torch.Tensor, codebook: torch.Tensor, beta: float = 0.25):
    """Nearest-codeword quantisation with a straight-through gradient.
    Returns ``(quantized, indices, commitment_loss)``."""
    flat = x.reshape(-1, x.size(-1))
    idx = torch.cdist(flat, codebook).argmin(dim=-1)
    q = codebook[idx]
    loss = F.mse_loss(flat.detach(), q) + beta * F.mse_loss(flat, q.detach())
    return (flat + (q - flat).detach()).reshape(x.shape), idx.reshape(x.shape[:-1]), loss
