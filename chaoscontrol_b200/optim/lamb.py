"""LAMB: Adam moments with a per-tensor trust ratio ``clip(||w|| / ||update||)``.

Constructor and semantics follow src/chaoscontrol/optim/lamb.py:43-210: weight
decay folded into the update direction, optional bias correction, 0/1-D tensors
left un-adapted unless ``always_adapt``, ``trust_ratio_override`` for the
"LAMB with ratio 1 == Adam" parity test.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch.optim import Optimizer


class LAMB(Optimizer):
    def __init__(self, params, *, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-6, weight_decay: float = 0.0, trust_clip: float = 10.0,
                 bias_correction: bool = True, always_adapt: bool = False,
                 trust_ratio_override: Optional[float] = None) -> None:
        if lr < 0.0:
            raise ValueError(f"invalid lr: {lr}")
        if eps < 0.0:
            raise ValueError(f"invalid eps: {eps}")
        for i, b in enumerate(betas):
            if not 0.0 <= b < 1.0:
                raise ValueError(f"invalid beta{i + 1}: {b}")
        if weight_decay < 0.0:
            raise ValueError(f"invalid weight_decay: {weight_decay}")
        if trust_clip <= 0.0:
            raise ValueError(f"invalid trust_clip: {trust_clip}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      trust_clip=trust_clip, bias_correction=bias_correction,
                                      always_adapt=always_adapt,
                                      trust_ratio_override=trust_ratio_override))

    @staticmethod
    def _trust_ratio(w_norm: torch.Tensor, r_norm: torch.Tensor, *, trust_clip: float) -> torch.Tensor:
        """``min(||w|| / ||r||, clip)``; 1 when either norm is zero."""
        ratio = torch.clamp(w_norm / r_norm.clamp_min(1e-38), max=trust_clip)
        return torch.where((w_norm > 0) & (r_norm > 0), ratio, torch.ones_like(ratio))

    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], torch.Tensor]] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("LAMB does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                t = st["step"]
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(p.grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                if g["bias_correction"]:
                    upd = (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + g["eps"])
                else:
                    upd = m / (v.sqrt() + g["eps"])
                if g["weight_decay"] != 0.0:
                    upd = upd.add(p, alpha=g["weight_decay"])
                if g["trust_ratio_override"] is not None:
                    ratio = torch.full((), float(g["trust_ratio_override"]), dtype=upd.dtype,
                                       device=upd.device)
                elif not g["always_adapt"] and p.ndim <= 1:
                    ratio = torch.ones((), dtype=upd.dtype, device=upd.device)
                else:
                    ratio = self._trust_ratio(p.float().norm(), upd.float().norm(),
                                              trust_clip=g["trust_clip"]).to(upd.dtype)
                p.add_(upd * ratio, alpha=-g["lr"])
        return loss
