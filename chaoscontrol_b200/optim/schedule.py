"""Momentum warm-up, weight EMA and the ``optimizer.step`` wrapper that applies
both (cf. src/chaoscontrol/optim/momentum_warmup.py, weight_ema.py:26-132,
step_wrapper.py:54-66)."""
from __future__ import annotations

import contextlib
from typing import Callable, Iterable, Iterator, Optional, TypeVar

import torch

T = TypeVar("T")


def apply_momentum_warmup(optimizer: torch.optim.Optimizer, *, step: int, target: float, start: float,
                          steps: int) -> float:
    """Linear ramp of ``param_group["momentum"]`` from ``start`` to ``target`` over
    ``steps`` steps (``steps <= 0`` pins the target).  Returns the applied value."""
    frac = 1.0 if steps <= 0 else min(step / steps, 1.0)
    momentum = (1.0 - frac) * start + frac * target
    for g in optimizer.param_groups:
        g["momentum"] = momentum
    return momentum


@torch.no_grad()
def _fake_quant_per_tensor_(t: torch.Tensor, *, bits: int) -> None:
    if bits <= 0:
        return
    amax = t.abs().max()
    if float(amax) == 0.0:
        return
    scale = amax / (((1 << bits) - 1) // 2)
    t.div_(scale).round_().mul_(scale)


class WeightEMA:
    """fp32 shadow of the trainable parameters; ``applied(model)`` swaps it in
    temporarily for evaluation."""

    def __init__(self, model: torch.nn.Module, *, decay: float, exclude_prefixes: Iterable[str] = (),
                 fake_quant_bits: int = 0) -> None:
        if not 0.0 <= decay < 1.0:
            raise ValueError(f"decay must be in [0, 1), got {decay}")
        self.decay = float(decay)
        self.exclude_prefixes = tuple(exclude_prefixes)
        self.fake_quant_bits = int(fake_quant_bits)
        self.shadow: dict[str, torch.Tensor] = {
            n: p.detach().to(torch.float32).clone() for n, p in model.named_parameters()
            if p.requires_grad and not any(n.startswith(pre) for pre in self.exclude_prefixes)}

    @torch.no_grad()
    def update(self, model: torch.nn.Module) -> None:
        if self.decay == 0.0:
            return
        sd = model.state_dict()
        for name, sh in self.shadow.items():
            sh.mul_(self.decay).add_(sd[name].detach().to(torch.float32), alpha=1.0 - self.decay)
            if self.fake_quant_bits > 0:
                _fake_quant_per_tensor_(sh, bits=self.fake_quant_bits)

    @contextlib.contextmanager
    def applied(self, model: torch.nn.Module) -> Iterator[None]:
        sd = model.state_dict()
        saved = {}
        for name, sh in self.shadow.items():
            saved[name] = sd[name].detach().clone()
            sd[name].copy_(sh.to(sd[name].dtype))
        try:
            yield
        finally:
            for name, orig in saved.items():
                sd[name].copy_(orig)


def eval_with_ema(model: torch.nn.Module, ema: Optional[WeightEMA], eval_fn: Callable[[], T]) -> T:
    if ema is None:
        return eval_fn()
    with ema.applied(model):
        return eval_fn()


def wrap_optimizer_step(optimizer: torch.optim.Optimizer, *, model: torch.nn.Module,
                        target_momentum: float, warmup_start: float, warmup_steps: int,
                        weight_ema_decay: float, is_rank_zero: bool,
                        ema_exclude_prefixes: Iterable[str] = (),
                        weight_ema_fake_quant_bits: int = 0) -> None:
    """Replace ``optimizer.step`` by: momentum warm-up -> original step -> EMA
    update (EMA on rank 0 only; the warm-up runs on every rank)."""
    ema = (WeightEMA(model, decay=weight_ema_decay, exclude_prefixes=tuple(ema_exclude_prefixes),
                     fake_quant_bits=weight_ema_fake_quant_bits)
           if is_rank_zero and weight_ema_decay > 0.0 else None)
    optimizer._weight_ema = ema                   # type: ignore[attr-defined]
    optimizer._momentum_warmup_step = 0           # type: ignore[attr-defined]
    inner = optimizer.step

    def step(*a, **kw):
        apply_momentum_warmup(optimizer, step=optimizer._momentum_warmup_step, target=target_momentum,
                              start=warmup_start, steps=warmup_steps)
        out = inner(*a, **kw)
        optimizer._momentum_warmup_step += 1
        if ema is not None:
            ema.update(model)
        return out

    optimizer.step = step                         # type: ignore[assignment]
