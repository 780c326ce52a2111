"""Offline behaviour-cloning pretrain of the simplex replay policy.

The online learner starts far better from a policy that already imitates the
heuristic ranking than from random weights (a uniform policy gives the
policy-gradient step no direction).  This module trains a PyTorch twin of the
native forward graph to pick the highest-utility vertex of synthetic
simplices and writes the result as a policy file the episodic runtime loads
through ``episodic_controller_weights_path``
(experiments/25_controller_pretrain/pretrain_controller.py:1-317; the export
of experiments/25_controller_pretrain/dump_to_cpp.py:69-140 is
``controller.save_simplex_policy``).

    vertex_h = gelu(V @ W_vp + b_vp)
    attn     = softmax_j(vertex_h vertex_h^T / sqrt(H) + alpha * E)
    mixed_h  = attn @ vertex_h + vertex_h
    logits   = mixed_h @ W_lh + b_lh
    p        = softmax((logits + feats @ W_sb) / T)

``python -m chaoscontrol_b200.episodic.pretrain --out simplex_policy_v1.pt``
"""
from __future__ import annotations

import argparse
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

__all__ = ["PretrainConfig", "SimplexPolicyModule", "synthetic_batch", "train", "to_native", "main"]


@dataclass
class PretrainConfig:
    n_vertices: int = 16
    k_v: int = 16
    k_s: int = 4
    h: int = 32
    temperature: float = 1.0
    learning_rate: float = 5e-3
    weight_decay: float = 1e-4
    batch_size: int = 64
    n_batches: int = 1000
    seed: int = 1337


class SimplexPolicyModule(nn.Module):
    """Same graph and parameter layout as the native policy, differentiable."""

    def __init__(self, cfg: PretrainConfig) -> None:
        super().__init__()
        self.cfg = cfg
        self.W_vp = nn.Parameter(torch.randn(cfg.k_v, cfg.h) / math.sqrt(cfg.k_v))
        self.b_vp = nn.Parameter(torch.zeros(cfg.h))
        self.W_lh = nn.Parameter(torch.randn(cfg.h) / math.sqrt(cfg.h))
        self.b_lh = nn.Parameter(torch.zeros(()))
        self.W_sb = nn.Parameter(torch.zeros(cfg.k_s))
        self.alpha = nn.Parameter(torch.zeros(()))
        self.register_buffer("temperature", torch.tensor(float(cfg.temperature)))

    def forward(self, V: torch.Tensor, E: torch.Tensor, feats: torch.Tensor) -> torch.Tensor:
        """``V [B, N, K_v]``, ``E [B, N, N]``, ``feats [B, K_s]`` -> tempered logits ``[B, N]``."""
        vh = F.gelu(V @ self.W_vp + self.b_vp)
        attn = torch.softmax(vh @ vh.transpose(-1, -2) / math.sqrt(self.cfg.h) + self.alpha * E, dim=-1)
        mixed = attn @ vh + vh
        logits = mixed @ self.W_lh + self.b_lh
        return (logits + (feats @ self.W_sb).unsqueeze(-1)) / self.temperature

    def flat(self) -> np.ndarray:
        """``[W_vp | b_vp | W_lh | b_lh | W_sb | alpha]``, the native flat layout."""
        parts = (self.W_vp, self.b_vp, self.W_lh, self.b_lh, self.W_sb, self.alpha)
        return torch.cat([p.detach().float().reshape(-1) for p in parts]).numpy()


def synthetic_batch(batch_size: int, cfg: PretrainConfig, generator: torch.Generator):
    """``(V, E, feats, target)``: column 0 of ``V`` plays the utility the heuristic ranks by and
    ``target`` is its argmax; ``E`` is the cosine between the remaining columns, so the edges say
    nothing about the label; ``feats`` are (top-1, mean, std, spread) of the utility column."""
    V = torch.randn(batch_size, cfg.n_vertices, cfg.k_v, generator=generator)
    rest = F.normalize(V[..., 1:], dim=-1, eps=1e-6)
    E = rest @ rest.transpose(-1, -2)
    u = V[..., 0]
    top1 = u.max(dim=-1).values
    feats = torch.stack([top1, u.mean(dim=-1), u.std(dim=-1), top1 - u.min(dim=-1).values], dim=-1)
    return V, E, feats[:, : cfg.k_s], u.argmax(dim=-1)


def train(cfg: Optional[PretrainConfig] = None) -> dict:
    """Cross-entropy against the heuristic's choice; accuracy is measured on held-out simplices."""
    cfg = cfg or PretrainConfig()
    torch.manual_seed(cfg.seed)
    model = SimplexPolicyModule(cfg)
    opt = torch.optim.AdamW(model.parameters(), lr=cfg.learning_rate, weight_decay=cfg.weight_decay)
    data = torch.Generator().manual_seed(cfg.seed + 1)          # sample stream independent of the init
    loss = torch.tensor(float("nan"))
    for _ in range(cfg.n_batches):
        V, E, feats, target = synthetic_batch(cfg.batch_size, cfg, data)
        loss = F.cross_entropy(model(V, E, feats), target)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
    with torch.no_grad():
        V, E, feats, target = synthetic_batch(512, cfg, torch.Generator().manual_seed(cfg.seed + 9999))
        logits = model(V, E, feats)
        acc = float((logits.argmax(dim=-1) == target).float().mean())
        max_p = float(torch.softmax(logits, dim=-1).max(dim=-1).values.mean())
    return {"final_policy_acc": acc, "final_loss": float(loss.detach()), "mean_max_p": max_p, "model": model, "config": cfg}


def to_native(model: SimplexPolicyModule):
    """The trained module as a native ``SimplexPolicy`` (forward on the CPU controller path)."""
    from . import native
    c = model.cfg
    pol = native.SimplexPolicy(N=c.n_vertices, K_v=c.k_v, K_s=c.k_s, H=c.h, temperature=float(model.temperature))
    pol.flat[:] = model.flat()
    return pol


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--n-batches", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--out", type=Path, default=Path("simplex_policy_v1.pt"),
                    help="*.pt (tensor dict) or any other suffix for the CSWG binary")
    ap.add_argument("--checkpoint", type=Path, default=None,
                    help="dump mode: a saved policy (*.pt or CSWG) to convert instead of training")
    ap.add_argument("--output", type=Path, default=None,
                    help="dump mode: target file (self-describing CSWG version 3 unless it ends in .pt)")
    a = ap.parse_args(argv)
    if a.checkpoint is not None or a.output is not None:
        if a.checkpoint is None or a.output is None:
            ap.error("dump mode needs both --checkpoint and --output")
        from .controller import load_simplex_policy, save_simplex_policy
        from .cswg import policy_to_cswg
        pol = load_simplex_policy(a.checkpoint)
        if str(a.output).endswith(".pt"):
            save_simplex_policy(a.output, pol)
            print(f"wrote {a.output} ({a.output.stat().st_size} bytes)")
        else:
            m = policy_to_cswg(pol, a.output)
            d = m["dims"]
            print(f"wrote {m['path']} version={m['version']} dims=(N={d['n_vertices']}, K_v={d['k_v']}, K_e={d['k_e']}, "
                  f"K_s={d['k_s']}, H={d['h']}, heads={d['n_heads']}) file_bytes={m['file_bytes']} "
                  f"fp16_drift={m['fp32_vs_fp16_max_abs_drift']:.3g}")
        return 0
    res = train(PretrainConfig(n_batches=a.n_batches, seed=a.seed, temperature=a.temperature))
    print(f"final_policy_acc={res['final_policy_acc']:.4f} final_loss={res['final_loss']:.4f} "
          f"mean_max_p={res['mean_max_p']:.4f}")
    from .controller import save_simplex_policy
    a.out.parent.mkdir(parents=True, exist_ok=True)
    save_simplex_policy(a.out, to_native(res["model"]))
    print(f"wrote {a.out} ({a.out.stat().st_size} bytes)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
