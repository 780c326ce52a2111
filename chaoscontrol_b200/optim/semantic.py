"""Muon whose momentum time constant follows each SSM channel's own time
constant (behaviour of src/chaoscontrol/optim/semantic.py:35-443).

A channel with slow recurrence (``sigmoid(log_a)`` near 1) integrates
gradients over a long horizon, a fast channel forgets quickly: the momentum
decay of the matrices listed in ``channel_map`` is a per-channel vector
``beta_i = beta_min + (beta_max - beta_min) * sigmoid(log_a_i)`` broadcast along
the named axis.  The orthogonalised read-out and its ``max(1, rows/cols)**0.5``
scale are Muon's: spatial geometry stays per matrix, only temporal geometry
becomes per channel.  Momentum buffers are fp32 whenever the coupling is active
(betas near 0.999 do not survive bf16).  ``log_a`` itself is 1-D and goes
through AdamW; listing it in ``channel_map`` is an error (self-coupling would
need its own damped rule).

Unlike the reference's one-matrix-at-a-time step, the per-channel momentum
update is elementwise, so matrices of one shape are stacked and orthogonalised
by ONE batched Newton-Schulz call.
"""
from __future__ import annotations

from typing import Any, Callable, Iterable, Optional

import torch
from torch import Tensor

from .muon import newton_schulz_orthogonalize

__all__ = ["SemanticOptimizer", "default_beta_from_log_a", "semantic_optimizer_config"]


def default_beta_from_log_a(log_a: Tensor, *, beta_min: float, beta_max: float) -> Tensor:
    """Detached fp32 ``beta_min + (beta_max - beta_min) * sigmoid(log_a)``."""
    return beta_min + (beta_max - beta_min) * torch.sigmoid(log_a.detach().float())


def semantic_optimizer_config(model: torch.nn.Module, layer_index: int) -> dict[str, Any]:
    """``a_param_name`` / ``channel_map`` for one block of a ``CareStudentLM``: projections whose
    output axis is the state (axis 0) and ``out_proj`` whose input axis is (axis 1)."""
    prefix = f"layers.{int(layer_index)}.core"
    names = {n for n, _ in model.named_parameters()}
    if f"{prefix}.log_a" not in names:
        raise ValueError(f"semantic optimizer requires {prefix + '.log_a'!r}")
    axes = {"in_proj.weight": 0, "select_proj.weight": 0, "gate_proj.weight": 0, "delta_proj.weight": 0,
            "out_proj.weight": 1}
    cmap = {f"{prefix}.{n}": a for n, a in axes.items() if f"{prefix}.{n}" in names}
    if not cmap:
        raise ValueError(f"semantic optimizer requires at least one channel-coupled matrix under {prefix!r}")
    return {"a_param_name": f"{prefix}.log_a", "channel_map": cmap}


class SemanticOptimizer(torch.optim.Optimizer):
    def __init__(self, params: Iterable[Tensor] | Iterable[dict[str, Any]], *, lr: float = 0.02,
                 momentum: float = 0.95, momentum_min: float = 0.5, nesterov: bool = True, ns_steps: int = 5,
                 weight_decay: float = 0.0, adamw_betas: tuple[float, float] = (0.9, 0.95), adamw_eps: float = 1e-8,
                 adamw_lr: Optional[float] = None, adamw_weight_decay: Optional[float] = None,
                 a_param_name: Optional[str] = None, channel_map: Optional[dict[str, int]] = None,
                 beta_from_a: Optional[Callable[[Tensor], Tensor]] = None,
                 matrix_param_names: Optional[set[str]] = None,
                 is_matrix: Optional[Callable[[Tensor, Optional[str]], bool]] = None,
                 compute_dtype: Optional[torch.dtype] = None) -> None:
        if lr <= 0.0 or ns_steps <= 0:
            raise ValueError(f"invalid hparams: lr={lr} ns_steps={ns_steps}")
        if not 0.0 <= momentum_min <= momentum < 1.0:
            raise ValueError(f"require 0 <= momentum_min ({momentum_min}) <= momentum ({momentum}) < 1")
        if a_param_name is not None and channel_map and a_param_name in channel_map:
            raise ValueError(f"A-parameter {a_param_name!r} cannot be in channel_map in v1: A is 1D and uses the "
                             f"AdamW fallback, which has no matrix momentum buffer for per-channel β to broadcast "
                             f"across.")
        super().__init__(params, dict(
            lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps, weight_decay=weight_decay,
            adamw_betas=adamw_betas, adamw_eps=adamw_eps, adamw_lr=lr if adamw_lr is None else adamw_lr,
            adamw_weight_decay=weight_decay if adamw_weight_decay is None else adamw_weight_decay))
        self._a_param_name = a_param_name
        self._channel_map = dict(channel_map or {})
        self._matrix_param_names = None if matrix_param_names is None else set(matrix_param_names)
        self._is_matrix_fn = is_matrix or (lambda p, _n: p.ndim == 2)
        self._momentum_max, self._momentum_min = float(momentum), float(momentum_min)
        self._beta_from_a = beta_from_a or (lambda a: default_beta_from_log_a(
            a, beta_min=self._momentum_min, beta_max=self._momentum_max))
        self._compute_dtype = compute_dtype
        self._param_name_by_id: dict[int, str] = {}
        self._a_param_ref: Optional[Tensor] = None

    # ------------------------------------------------------------------ wiring
    def bind_param_names(self, named_params: Iterable[tuple[str, Tensor]]) -> None:
        """Resolves ``a_param_name`` and ``channel_map`` by name; a name that is missing
        raises here instead of silently reducing the optimizer to plain Muon."""
        named = list(named_params)
        self._param_name_by_id = {id(p): n for n, p in named}
        bound = {n for n, _ in named}
        if self._a_param_name is not None:
            if self._a_param_name not in bound:
                raise ValueError(f"a_param_name {self._a_param_name!r} not found in bound named_params; cannot "
                                 f"compute per-channel β")
            mine = {id(p) for g in self.param_groups for p in g["params"]}
            self._a_param_ref = next((p for n, p in named if n == self._a_param_name and id(p) in mine), None)
            if self._a_param_ref is None:
                raise ValueError(f"a_param_name {self._a_param_name!r} is in bindings but not in any param_group — "
                                 f"did you forget to pass it to the optimizer?")
        missing = [n for n in self._channel_map if n not in bound]
        if missing:
            raise ValueError(f"channel_map names not in bound named_params: {missing}")

    def current_beta_vec(self) -> Optional[Tensor]:
        return None if self._a_param_ref is None else self._beta_from_a(self._a_param_ref).detach()

    def beta_trace(self) -> Optional[dict[str, Any]]:
        """Current betas and their time constants ``-1 / ln(beta)`` in steps (beta clipped at 0.999)."""
        beta = self.current_beta_vec()
        if beta is None:
            return None
        beta = beta.float().cpu()
        tau = -1.0 / torch.log(beta.clamp(max=0.999)).clamp(max=-1e-6)
        return {"beta_vec": beta, "tau_steps": tau, "beta_min": float(beta.min()), "beta_max": float(beta.max()),
                "beta_mean": float(beta.mean())}

    def _is_matrix_param(self, p: Tensor) -> bool:
        name = self._param_name_by_id.get(id(p))
        if self._matrix_param_names is not None and name is not None:
            return name in self._matrix_param_names
        return self._is_matrix_fn(p, name)

    @staticmethod
    def _broadcast_beta(beta_vec: Tensor, shape: torch.Size, axis: int) -> Tensor:
        if axis < 0:
            axis += len(shape)
        if not 0 <= axis < len(shape):
            raise ValueError(f"channel axis {axis} out of range for shape {tuple(shape)}")
        if beta_vec.numel() != shape[axis]:
            raise ValueError(f"β has {beta_vec.numel()} channels, param axis {axis} has {shape[axis]}")
        view = [1] * len(shape)
        view[axis] = beta_vec.numel()
        return beta_vec.view(view)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], Tensor]] = None) -> Optional[Tensor]:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._a_param_name is not None and self._a_param_ref is None:
            raise RuntimeError(f"a_param_name={self._a_param_name!r} is set but no A parameter resolved — call "
                               f"bind_param_names() before step()")
        beta_vec = None if self._a_param_ref is None else self._beta_from_a(self._a_param_ref)
        buf_dtype_fp32 = self._a_param_ref is not None
        for group in self.param_groups:
            lr, mu, nesterov, wd = group["lr"], group["momentum"], group["nesterov"], group["weight_decay"]
            b1, b2 = group["adamw_betas"]
            stacks: dict[tuple, list[tuple[Tensor, Tensor]]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not self._is_matrix_param(p):
                    self._adamw(p, st, b1, b2, group["adamw_eps"], group["adamw_lr"], group["adamw_weight_decay"])
                    continue
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p, memory_format=torch.preserve_format,
                                                             dtype=torch.float32 if buf_dtype_fp32 else p.dtype)
                buf = st["momentum_buffer"]
                name = self._param_name_by_id.get(id(p))
                beta: Tensor | float = mu
                if beta_vec is not None and name in self._channel_map:
                    beta = self._broadcast_beta(beta_vec.to(device=buf.device, dtype=buf.dtype), buf.shape,
                                                self._channel_map[name])
                g = p.grad.to(buf.dtype)
                buf.mul_(beta).add_(g)
                direction = (g + beta * buf) if nesterov else buf
                stacks.setdefault((tuple(p.shape), direction.dtype, p.device), []).append((p, direction))
            for (shape, _dt, _dev), items in stacks.items():
                upd = newton_schulz_orthogonalize(torch.stack([d for _, d in items], 0), steps=group["ns_steps"],
                                                  compute_dtype=self._compute_dtype)
                scale = max(1.0, shape[-2] / shape[-1]) ** 0.5
                for i, (p, _d) in enumerate(items):
                    if wd > 0.0:
                        p.data.mul_(1.0 - lr * wd)
                    p.data.add_(upd[i].to(p.dtype), alpha=-lr * scale)
        return loss

    def _adamw(self, p: Tensor, st: dict, b1: float, b2: float, eps: float, lr: float, wd: float) -> None:
        if "step" not in st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        st["step"] += 1
        t = st["step"]
        g = p.grad
        st["exp_avg"].mul_(b1).add_(g, alpha=1.0 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1.0 - b2)
        denom = (st["exp_avg_sq"].sqrt() / ((1.0 - b2 ** t) ** 0.5)).add_(eps)
        if wd > 0.0:
            p.data.mul_(1.0 - lr * wd)
        p.data.addcdiv_(st["exp_avg"], denom, value=-lr / (1.0 - b1 ** t))
