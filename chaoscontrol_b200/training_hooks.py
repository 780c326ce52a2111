"""Training-time mechanisms that ride on the optimizer step: the fast/slow
weight consolidator, the spectral regulariser on ``sigmoid(log_a)``, the
predictive auxiliary loss and the embedding-gradient freeze
(public surface of experiments/23_fast_path/training_hooks.py:11-489).

When the model's parameters live in a flat arena, the slow copy is ONE flat
tensor (``slow_state`` entries are views into it): a consolidation is a single
``lerp_`` launch over all parameters and ``copy_slow_to_model`` a single copy.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Iterable, Optional

import torch

from .utils.arena import get_arena

__all__ = ["FastSlowDecision", "FastSlowConsolidator", "fast_slow_decision_to_dict", "fast_slow_decision_from_dict",
           "iter_log_a_params", "spectral_regularization_loss", "spectral_summary", "predictive_auxiliary_loss",
           "zero_embedding_grad_until"]


@dataclass(frozen=True)
class FastSlowDecision:
    mode: str                 # disabled | learned | interval | hold
    accepted: bool
    alpha: float
    gate: float
    effective_alpha: float
    step: int
    reason: str


def _clamp(v: float, lo: float, hi: float) -> float:
    v = float(v)
    return float(lo) if not math.isfinite(v) else max(float(lo), min(float(hi), v))


def _readiness(action_space: Any, head: str) -> float:
    fn = getattr(action_space, "readiness", None)
    if not callable(fn):
        return 0.0
    try:
        v = float(fn(str(head)))
    except Exception:
        return 0.0
    return v if math.isfinite(v) else 0.0


@dataclass
class FastSlowConsolidator:
    """Slow copy ``s <- lerp(s, fast, alpha)`` every ``interval`` steps, or when a
    learned controller's ``consolidation`` head says so (gate x ``ema_alpha`` head).
    Evaluation uses the slow copy once it has received at least one real sync.
    The loss improvement after an accepted learned decision is fed back to the
    controller as that decision's reward."""

    enabled: bool
    interval: int
    alpha: float
    slow_state: dict[str, torch.Tensor]
    sync_count: int = 0
    decision_count: int = 0
    learned_decision_count: int = 0
    learned_sync_count: int = 0
    last_sync_step: int = -1
    last_decision: Optional[FastSlowDecision] = None
    last_reward: float = 0.0
    reward_update_count: int = 0
    _last_loss_value: Optional[float] = None
    _last_credit_key: Optional[int] = None
    _flat_slow: Optional[torch.Tensor] = field(default=None, repr=False)
    _flat_fast: Optional[torch.Tensor] = field(default=None, repr=False)

    @classmethod
    def from_config(cls, model: torch.nn.Module, config: dict[str, object]) -> "FastSlowConsolidator":
        on = bool(config.get("fast_slow_enabled", False))
        arena = get_arena(model)
        flat_slow = flat_fast = None
        if arena is not None and arena.still_valid():
            flat_fast = arena.flat_param
            flat_slow = flat_fast.detach().clone()
            slow = {}
            for name, p in model.named_parameters():
                off, shp = arena.slots[name]
                slow[name] = flat_slow[off: off + p.numel()].view(shp)
        else:
            slow = {name: p.detach().clone() for name, p in model.named_parameters()}
        return cls(enabled=on, interval=int(config.get("fast_slow_interval", 0)) if on else 0,
                   alpha=float(config.get("fast_slow_alpha", 0.0)) if on else 0.0, slow_state=slow,
                   _flat_slow=flat_slow, _flat_fast=flat_fast)

    # ------------------------------------------------------------------ decisions
    def after_optimizer_step(self, model, *, step: int, action_space: Any | None = None,
                             reward_context: dict[str, Any] | None = None,
                             loss_value: float | None = None) -> FastSlowDecision:
        d = self.decide(step=step, action_space=action_space, reward_context=reward_context, loss_value=loss_value)
        self.apply_decision(model, d)
        return d

    def _record(self, d: FastSlowDecision) -> FastSlowDecision:
        self.decision_count += 1
        self.learned_decision_count += int(d.mode == "learned")
        self.last_decision = d
        return d

    def decide(self, *, step: int, action_space: Any | None = None, reward_context: dict[str, Any] | None = None,
               loss_value: float | None = None) -> FastSlowDecision:
        step = int(step)
        if not self.enabled:
            return self._record(FastSlowDecision("disabled", False, 0.0, 0.0, 0.0, step, "disabled"))
        ctx = dict(reward_context or {})
        ctx.setdefault("steps_since_slow_sync", float(self.steps_since_sync(step)))
        ctx.setdefault("fast_slow_sync_count", float(self.sync_count))
        ctx.setdefault("fast_slow_last_reward", float(self.last_reward))
        self._apply_loss_reward(action_space=action_space, step=step, loss_value=loss_value, reward_context=ctx)
        if action_space is not None and _readiness(action_space, "consolidation") > 0.0:
            gate = _clamp(action_space.scalar_value(head_name="consolidation", gpu_step=step, fallback=0.0,
                                                    reward_context=ctx), 0.0, 1.0)
            alpha_ready = _readiness(action_space, "ema_alpha") > 0.0
            alpha = _clamp(action_space.scalar_value(head_name="ema_alpha", gpu_step=step, fallback=float(self.alpha),
                                                     reward_context=ctx) if alpha_ready else self.alpha, 0.0, 1.0)
            eff = _clamp(gate * alpha, 0.0, 1.0)
            d = FastSlowDecision("learned", eff > 0.0, alpha, gate, eff, step, "controller_consolidation_head")
            if d.accepted:
                self._last_credit_key = step
                rec = getattr(action_space, "record_credit_assignment", None)
                if callable(rec):
                    rec(key=step, head_names=["consolidation"] + (["ema_alpha"] if alpha_ready else []),
                        gpu_step=step, reward_context=ctx)
            return self._record(d)
        if self.interval > 0 and step % self.interval == 0:
            a = float(self.alpha)
            return self._record(FastSlowDecision("interval", True, a, 1.0, a, step, "fixed_interval_fallback"))
        return self._record(FastSlowDecision("hold", False, float(self.alpha), 0.0, 0.0, step, "not_due"))

    def apply_decision(self, model: torch.nn.Module, decision: FastSlowDecision) -> None:
        self.last_decision = decision
        if not decision.accepted or decision.effective_alpha <= 0.0:
            return
        alpha = float(decision.effective_alpha)
        with torch.no_grad():
            arena = get_arena(model)
            if (self._flat_slow is not None and arena is not None and arena.still_valid()
                    and arena.flat_param is self._flat_fast):
                self._flat_slow.lerp_(self._flat_fast, alpha)                 # one launch for the whole model
            else:
                params = dict(model.named_parameters())
                slow_l, fast_l = [], []
                for name, s in self.slow_state.items():
                    p = params.get(name)
                    if p is None:
                        continue
                    f = p.detach()
                    if f.device != s.device or f.dtype != s.dtype:
                        s.lerp_(f.to(device=s.device, dtype=s.dtype), alpha)
                    else:
                        slow_l.append(s)
                        fast_l.append(f)
                if slow_l:
                    torch._foreach_lerp_(slow_l, fast_l, alpha)
        self.sync_count += 1
        self.last_sync_step = int(decision.step)
        self.learned_sync_count += int(decision.mode == "learned")

    # ------------------------------------------------------------------ rewards
    def _apply_reward(self, action_space, key: int, reward: float, step: int, ctx: dict) -> int:
        fn = getattr(action_space, "apply_reward", None)
        if not callable(fn):
            return 0
        n = int(fn(key=int(key), reward=float(reward), gpu_step=int(step), reward_context=ctx))
        if n > 0:
            self.reward_update_count += n
            self.last_reward = float(reward)
        return n

    def apply_external_reward(self, *, action_space: Any | None, key: int, reward: float, step: int,
                              reward_context: dict[str, Any] | None = None) -> int:
        if action_space is None or not math.isfinite(float(reward)):
            return 0
        return self._apply_reward(action_space, key, reward, step, dict(reward_context or {}))

    def _apply_loss_reward(self, *, action_space, step: int, loss_value, reward_context: dict[str, Any]) -> None:
        if action_space is None or loss_value is None or not math.isfinite(float(loss_value)):
            return
        loss = float(loss_value)
        reward_context["loss"] = loss
        if self._last_loss_value is not None and self._last_credit_key is not None:
            self._apply_reward(action_space, self._last_credit_key, self._last_loss_value - loss, step, reward_context)
        self._last_loss_value = loss
        self._last_credit_key = None

    # ------------------------------------------------------------------ eval copy / diagnostics
    def copy_slow_to_model(self, model: torch.nn.Module) -> None:
        with torch.no_grad():
            arena = get_arena(model)
            if (self._flat_slow is not None and arena is not None and arena.still_valid()
                    and arena.flat_param is self._flat_fast):
                self._flat_fast.copy_(self._flat_slow)
                return
            params = dict(model.named_parameters())
            for name, s in self.slow_state.items():
                p = params.get(name)
                if p is not None:
                    p.copy_(s.to(device=p.device, dtype=p.dtype))

    def should_copy_slow_to_model_for_eval(self) -> bool:
        return bool(self.enabled and self.sync_count > 0)

    def steps_since_sync(self, step: int | None) -> int:
        if self.last_sync_step < 0:
            return 0 if step is None else int(step)
        if step is None:
            if self.last_decision is None:
                return 0
            step = self.last_decision.step
        return max(0, int(step) - int(self.last_sync_step))

    def diagnostics(self, model: torch.nn.Module) -> dict[str, object]:
        params = dict(model.named_parameters())
        sq = 0.0
        for name, s in self.slow_state.items():
            p = params.get(name)
            if p is not None:
                sq += float((p.detach().float() - s.to(p.device).float()).pow(2).sum())
        return {"enabled": self.enabled, "interval": self.interval, "alpha": self.alpha,
                "sync_count": self.sync_count, "fast_slow_l2": math.sqrt(sq), "decision_count": self.decision_count,
                "learned_decision_count": self.learned_decision_count, "learned_sync_count": self.learned_sync_count,
                "last_sync_step": self.last_sync_step, "steps_since_sync": self.steps_since_sync(None),
                "eval_copy_ready": self.should_copy_slow_to_model_for_eval(), "last_reward": self.last_reward,
                "reward_update_count": self.reward_update_count,
                "last_decision": fast_slow_decision_to_dict(self.last_decision)}


def fast_slow_decision_to_dict(d: FastSlowDecision | None) -> dict[str, object] | None:
    if d is None:
        return None
    return {"mode": str(d.mode), "accepted": bool(d.accepted), "alpha": float(d.alpha), "gate": float(d.gate),
            "effective_alpha": float(d.effective_alpha), "step": int(d.step), "reason": str(d.reason)}


def fast_slow_decision_from_dict(payload: object) -> FastSlowDecision | None:
    if not isinstance(payload, dict):
        return None
    try:
        return FastSlowDecision(mode=str(payload.get("mode", "")), accepted=bool(payload.get("accepted", False)),
                                alpha=float(payload.get("alpha", 0.0)), gate=float(payload.get("gate", 0.0)),
                                effective_alpha=float(payload.get("effective_alpha", 0.0)),
                                step=int(payload.get("step", 0)), reason=str(payload.get("reason", "")))
    except Exception:
        return None


# ---------------------------------------------------------------------------
def iter_log_a_params(model: torch.nn.Module) -> Iterable[tuple[str, torch.Tensor]]:
    for name, p in model.named_parameters():
        if name.endswith(".log_a") and p.ndim == 1:
            yield name, p


def spectral_regularization_loss(model, lambda_dead: float, lambda_sticky: float, min_a: float,
                                 max_a: float) -> torch.Tensor | None:
    """Quadratic hinge on ``a = sigmoid(log_a)`` outside ``[min_a, max_a]``:
    channels that forget everything ("dead") or nothing ("sticky")."""
    terms = []
    for _, log_a in iter_log_a_params(model):
        a = torch.sigmoid(log_a.float())
        terms.append((torch.relu(min_a - a).pow(2) * lambda_dead + torch.relu(a - max_a).pow(2) * lambda_sticky).mean())
    return torch.stack(terms).mean() if terms else None


def spectral_summary(model: torch.nn.Module) -> dict[str, float | int]:
    vals = [torch.sigmoid(p.float()).reshape(-1) for _, p in iter_log_a_params(model)]
    if not vals:
        return {"log_a_param_count": 0}
    a = torch.cat(vals).detach()
    q = torch.quantile(a, torch.tensor([0.05, 0.50, 0.95], device=a.device)).tolist()
    return {"log_a_param_count": len(vals), "a_min": float(a.min()), "a_max": float(a.max()),
            "a_mean": float(a.mean()), "a_p05": q[0], "a_p50": q[1], "a_p95": q[2]}


def predictive_auxiliary_loss(hidden: torch.Tensor, *, projection: torch.nn.Module, horizon: int) -> torch.Tensor | None:
    """MSE between ``projection(h[t])`` and the (detached) ``h[t + horizon]``."""
    horizon = int(horizon)
    if horizon <= 0 or hidden.size(1) <= horizon:
        return None
    return torch.nn.functional.mse_loss(projection(hidden[:, :-horizon]).float(), hidden[:, horizon:].detach().float())


def zero_embedding_grad_until(model: torch.nn.Module, step: int, freeze_steps: int) -> None:
    if freeze_steps <= 0 or step >= freeze_steps:
        return
    w = getattr(getattr(model, "embed", None), "weight", None)
    if w is not None and w.grad is not None:
        w.grad.zero_()


# ---------------------------------------------------------------------------
# criticality distillation in the training loop
# ---------------------------------------------------------------------------
class CriticalityDistillHook:
    """Runs criticality distillation beside a training step
    (runner_fast_path.py:11127-11190, 12545-12812): captures every layer's
    recurrence states and the per-token CE / entropy in ONE extra no-grad pass,
    turns ``relu(CE - entropy)`` into event pressure, folds the device-side
    aggregates into the seat bookkeeping (host side, ``[L, D]`` sized), refreshes
    the seats on their interval, and back-propagates the ``log_a`` loss as its own
    pass (its gradients touch ``log_a`` only).  Single rank only: seats and the
    loss are rank-local."""

    def __init__(self, model: torch.nn.Module, *, num_layers: int, dim: int, budget_frac: float = 0.15,
                 critical_value: float = 0.95, trace_ttl_steps: int = 1024, trace_half_life_steps: float = 256.0,
                 seat_refresh_interval: int = 64, min_weighted_events_per_layer: float = 256.0,
                 horizon_H: int = 16, event_frac: float = 0.05, weight: float = 1e-3,
                 uniform_pressure: bool = False, score_permute_before_topk: bool = False,
                 fixed_random_seats: bool = False) -> None:
        from .optim.criticality import CriticalityDistillation
        self.cores = [m for m in model.modules() if callable(getattr(m, "capture_states", None))]
        if len(self.cores) != int(num_layers):
            raise ValueError(f"criticality_distill_num_layers mismatch: configured {int(num_layers)} but the model "
                             f"exposes {len(self.cores)} modules with capture_states()")
        self.cd = CriticalityDistillation(
            num_layers=int(num_layers), dim=int(dim), trace_ttl_steps=int(trace_ttl_steps),
            trace_half_life_steps=float(trace_half_life_steps), seat_refresh_interval=int(seat_refresh_interval),
            criticality_budget_frac=float(budget_frac), critical_value=float(critical_value),
            min_weighted_events_per_layer=float(min_weighted_events_per_layer),
            criticality_distill_weight=float(weight), score_permute_before_topk=bool(score_permute_before_topk),
            fixed_random_seats=bool(fixed_random_seats))
        self.horizon_H, self.event_frac, self.uniform = int(horizon_H), float(event_frac), bool(uniform_pressure)
        self.snapshots: list[dict] = []
        self.loss_trajectory: list[dict] = []
        self.ingests = self.seat_refreshes = 0

    @classmethod
    def from_config(cls, model: torch.nn.Module, config: dict) -> "Optional[CriticalityDistillHook]":
        if not bool(config.get("criticality_distill_enabled", False)):
            return None
        pre = "criticality_distill_"
        for need in ("num_layers", "dim"):
            if config.get(pre + need) is None:
                raise ValueError(f"criticality_distill_enabled=True requires {pre}{need}")
        kw = {k[len(pre):]: v for k, v in config.items() if k.startswith(pre) and k != pre + "enabled"}
        return cls(model, **kw)

    def _log_a(self) -> list[torch.Tensor]:
        return [c.log_a for c in self.cores]

    def after_backward(self, model: torch.nn.Module, inputs: torch.Tensor, targets: torch.Tensor, *, step: int,
                       lm_head_tile_size: int = 8192) -> Optional[torch.Tensor]:
        """Call between the step's backward and the gradient clip.  Returns the
        distillation loss (device scalar) when seats exist, else ``None``."""
        import contextlib

        from .kernels.lm_head_loss import fused_lm_head_forward_with_ce_entropy
        with contextlib.ExitStack() as stack, torch.no_grad():
            getters = [stack.enter_context(c.capture_states()) for c in self.cores]
            normed = model.final_norm(model.encode(inputs))
            states = [g() for g in getters]
            if any(s is None for s in states):
                raise RuntimeError("criticality distillation: a recurrence core did not record its states; "
                                   "state capture needs a_mode='diag'")
            B, T = inputs.shape
            if self.uniform:
                pressure = torch.ones(B, T, device=normed.device)
            else:
                _, _, ce, ent = fused_lm_head_forward_with_ce_entropy(normed, model.lm_head.weight, targets,
                                                                      tile_size=int(lm_head_tile_size))
                pressure = torch.relu(ce.reshape(B, T).float() - ent.reshape(B, T).float())
            prepared = self.cd.ingest_gpu(pressure=pressure, states_per_layer=states, horizon_H=self.horizon_H,
                                          event_frac=self.event_frac)
        host = {k: v.to("cpu") for k, v in prepared.items()}          # [L, D] aggregates and two counters
        self.cd.ingest_cpu_from_prepared(step=int(step), prepared=host)
        self.ingests += 1
        every = int(self.cd.seat_refresh_interval)
        if step > 0 and every > 0 and step % every == 0:
            self.cd.allocate_seats_from_accumulators(current_step=int(step))
            self.seat_refreshes += 1
            self.snapshots.append(self.cd.diagnostics_snapshot(log_a_per_layer=self._log_a(),
                                                               current_step=int(step)))
        if not bool(self.cd.seat_mask.any()):
            return None
        loss = self.cd.criticality_loss(self._log_a())
        if loss.requires_grad:
            loss.backward()
        self.loss_trajectory.append({"step": int(step), "cd_loss": float(loss.detach())})
        return loss.detach()

    def diagnostics(self) -> dict:
        return {"enabled": True, "ingests": self.ingests, "seat_refreshes": self.seat_refreshes,
                "seats": int(self.cd.seat_mask.sum()), "loss_trajectory": self.loss_trajectory[-64:],
                "snapshots": self.snapshots[-8:]}
