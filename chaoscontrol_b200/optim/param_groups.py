"""Parameter grouping for SSM-aware optimisation
(cf. src/chaoscontrol/optim/param_groups.py:74-194).

``classify_param`` is shape-first with a name override for spectral / dynamics
parameters; ``ssm_three_group_params`` gives dynamics a reduced learning rate
and no decay, 1-D gains no decay, matrices the full recipe.
"""
from __future__ import annotations

from typing import Any, Iterable

from torch import Tensor

SPECTRAL_SUFFIXES = frozenset({"log_a", "log_r", "theta", "skew_params", "log_gamma", "U", "V"})


def classify_param(name: str, param: Tensor) -> str:
    """``"dynamics"`` (spectral names), ``"no_decay"`` (<= 1-D), or ``"main"``."""
    if name.rsplit(".", 1)[-1] in SPECTRAL_SUFFIXES:
        return "dynamics"
    return "no_decay" if param.ndim <= 1 else "main"


def ssm_three_group_params(named_params: Iterable[tuple[str, Tensor]], *, base_lr: float,
                           weight_decay: float, dynamics_lr_mul: float = 0.1) -> list[dict[str, Any]]:
    buckets: dict[str, list[Tensor]] = {"dynamics": [], "no_decay": [], "main": []}
    for name, p in named_params:
        if p.requires_grad:
            buckets[classify_param(name, p)].append(p)
    recipe = {"dynamics": (float(base_lr) * float(dynamics_lr_mul), 0.0),
              "no_decay": (float(base_lr), 0.0),
              "main": (float(base_lr), float(weight_decay))}
    groups = []
    for name in ("dynamics", "no_decay", "main"):
        if buckets[name]:
            lr, wd = recipe[name]
            groups.append({"name": name, "params": buckets[name], "lr": lr, "adamw_lr": lr,
                           "weight_decay": wd, "adamw_weight_decay": wd})
    return groups


def build_optimizer_params(named_params: Iterable[tuple[str, Tensor]], *, grouping: str,
                           base_lr: float, weight_decay: float, dynamics_lr_mul: float = 0.1):
    """``"flat"`` -> list of trainable tensors; ``"ssm_three_group"`` -> param groups.
    Unknown modes raise (a config typo must fail before GPU time is spent)."""
    mode = str(grouping).strip().lower()
    if mode == "flat":
        return [p for _, p in named_params if p.requires_grad]
    if mode == "ssm_three_group":
        return ssm_three_group_params(named_params, base_lr=base_lr, weight_decay=weight_decay,
                                      dynamics_lr_mul=dynamics_lr_mul)
    raise ValueError(f"unknown optimizer_param_grouping {grouping!r}; expected 'flat' or 'ssm_three_group'")
