"""Bounded learned action space of the episodic controller (behaviour of
src/chaoscontrol/episodic/learned_action_space.py:66-707).

A learned head may only add a bounded residual to an action the heuristic
already made legal: ``effective = heuristic + tanh(raw) * max_delta * readiness``
for rankings, ``(1 - readiness) * fallback + readiness * spec.map(raw)`` for
scalar knobs.  Readiness 0 (or ``trace_only``) is the heuristic bit for bit, and
every intervention / clamp is reported to a trace sink.

All heads read one tiny recurrent state (``SharedEventSsm``): a stable full
transition matrix (rotation pairs + damping + a low-rank perturbation, rescaled so
its top log singular value is ``target_log_sv``) driven by ``tanh(W_in f)``.
State, input and head weights live in tensors; one ``observe`` is three small
mat-vecs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence

import torch
import torch.nn.functional as F

TraceSink = list

DEFAULT_EVENT_FEATURES: tuple[str, ...] = (
    "bias", "pressure", "ce", "score", "rank", "utility", "age", "bucket", "entropy", "reward",
    "finite_reward", "cache_fill", "wall_pressure", "steps_since_slow_sync", "fast_slow_sync_count",
    "fast_slow_last_reward", "loss")
DEFAULT_HEADS: tuple[str, ...] = (
    "write_admission", "eviction", "replay_timing", "replay_budget", "write_budget", "temperature",
    "entropy_beta", "ema_alpha", "consolidation", "selection_rank")

__all__ = ["BoundedScalarSpec", "SharedEventSsm", "ActionSpaceTrace", "ConstrainedActionSpace",
           "coerce_action_space", "make_shared_event_ssm_from_config", "DEFAULT_EVENT_FEATURES", "DEFAULT_HEADS"]


def _clamp01(v: float) -> float:
    v = float(v)
    return min(1.0, max(0.0, v)) if math.isfinite(v) else 0.0


def _tanh_or_zero(v: float) -> float:
    v = float(v)
    return math.tanh(v) if math.isfinite(v) else 0.0


@dataclass(frozen=True)
class BoundedScalarSpec:
    """Maps an unconstrained scalar into ``[minimum, maximum]``."""
    name: str
    minimum: float
    maximum: float
    transform: str = "sigmoid"

    def __post_init__(self) -> None:
        for side in ("minimum", "maximum"):
            if not math.isfinite(float(getattr(self, side))):
                raise ValueError(f"{self.name}.{side} must be finite")
        if float(self.maximum) < float(self.minimum):
            raise ValueError(f"{self.name}.maximum must be >= minimum")
        if self.transform not in ("sigmoid", "tanh", "softplus"):
            raise ValueError("BoundedScalarSpec.transform must be 'sigmoid', 'tanh', or 'softplus'")

    def map(self, raw: float) -> float:
        x, lo, hi = float(raw), float(self.minimum), float(self.maximum)
        if not math.isfinite(x) or hi == lo:
            return lo
        if self.transform == "sigmoid":
            unit = 0.5 * (1.0 + math.tanh(0.5 * x))            # overflow-free logistic
        elif self.transform == "tanh":
            unit = 0.5 * (math.tanh(x) + 1.0)
        else:
            sp = x if x > 20.0 else math.log1p(math.exp(x))
            unit = sp / (1.0 + sp)
        return lo + unit * (hi - lo)


class SharedEventSsm:
    """Small full-matrix recurrent state shared by every action head."""

    def __init__(self, hidden_dim: int = 16, feature_names: Sequence[str] = DEFAULT_EVENT_FEATURES,
                 head_names: Sequence[str] = DEFAULT_HEADS, seed: int = 0, decay: float = 0.95,
                 input_scale: float = 0.05, head_scale: float = 0.05, rank: int = 4, gamma: float = 0.08,
                 perturbation_scale: float = 0.20, target_log_sv: float = -0.02,
                 max_state_norm: float = 8.0) -> None:
        if hidden_dim <= 0:
            raise ValueError("SharedEventSsm.hidden_dim must be positive")
        if not 0.0 <= float(decay) <= 1.0:
            raise ValueError("SharedEventSsm.decay must be in [0, 1]")
        self.hidden_dim, self.seed, self.decay = int(hidden_dim), int(seed), float(decay)
        self.input_scale, self.head_scale = float(input_scale), float(head_scale)
        self.rank = max(1, min(int(rank), self.hidden_dim))
        self.gamma = max(1e-4, float(gamma))
        self.perturbation_scale = max(0.0, float(perturbation_scale))
        self.target_log_sv = float(target_log_sv)
        self.max_state_norm = max(1e-4, float(max_state_norm))
        self.feature_names = tuple(str(x) for x in feature_names)
        self.head_names = tuple(str(x) for x in head_names)
        self._head_index = {h: i for i, h in enumerate(self.head_names)}
        gen = torch.Generator().manual_seed(self.seed)
        H, Fd, Nh = self.hidden_dim, len(self.feature_names), len(self.head_names)
        self.W_in = (torch.rand(Fd, H, generator=gen) * 2 - 1) * self.input_scale       # [F, H]
        self.W_head = (torch.rand(H, Nh, generator=gen) * 2 - 1) * self.head_scale      # [H, heads]
        self.b_head = torch.zeros(Nh)
        self.state = torch.zeros(H)
        self.A, self._top_log_sv = self._transition(gen)
        self._state_clamp_count = 0

    def _transition(self, gen: torch.Generator) -> tuple[torch.Tensor, float]:
        H = self.hidden_dim
        cont = -self.gamma * torch.eye(H)
        pairs = H // 2
        if pairs:
            om = torch.linspace(0.08, 0.55, pairs)
            a = torch.arange(pairs) * 2
            cont[a, a + 1] -= om
            cont[a + 1, a] += om
        U = F.normalize(torch.randn(H, self.rank, generator=gen), dim=0, eps=1e-8)
        V = F.normalize(torch.randn(H, self.rank, generator=gen), dim=0, eps=1e-8)
        low = U @ V.T
        cont = cont + low * (self.perturbation_scale / torch.linalg.matrix_norm(low, ord=2).clamp_min(1e-8))
        A = torch.matrix_exp(cont)
        top = float(torch.linalg.svdvals(A).clamp_min(1e-8).log().max())
        if top > self.target_log_sv:
            A = A * math.exp(self.target_log_sv - top)
            top = float(torch.linalg.svdvals(A).clamp_min(1e-8).log().max())
        return A.contiguous(), top

    # -- views kept for callers that think in lists -------------------------
    @property
    def hidden(self) -> list[float]:
        return self.state.tolist()

    @property
    def head_weights(self) -> dict[str, list[float]]:
        return {h: self.W_head[:, i].tolist() for h, i in self._head_index.items()}

    @property
    def head_bias(self) -> dict[str, float]:
        return {h: float(self.b_head[i]) for h, i in self._head_index.items()}

    def _features(self, features: Mapping[str, float]) -> torch.Tensor:
        vals = []
        for name in self.feature_names:
            v = 1.0 if name == "bias" else float(features.get(name, 0.0))
            vals.append(v if math.isfinite(v) else 0.0)
        return torch.tensor(vals, dtype=torch.float32)

    @torch.no_grad()
    def observe(self, features: Optional[Mapping[str, float]] = None) -> dict[str, float]:
        """``state <- decay * A state + tanh(W_in^T f)`` (non-finite states reset, norm capped), then all heads."""
        new = self.decay * (self.A @ self.state) + torch.tanh(self._features(features or {}) @ self.W_in)
        if not bool(torch.isfinite(new).all()):
            new = torch.zeros_like(new)
        norm = float(new.norm())
        if norm > self.max_state_norm:
            new = new * (self.max_state_norm / max(norm, 1e-8))
            self._state_clamp_count += 1
        self.state = new
        return self.head_outputs()

    @torch.no_grad()
    def head_outputs(self) -> dict[str, float]:
        return dict(zip(self.head_names, (self.state @ self.W_head + self.b_head).tolist()))

    def head_output(self, head_name: str) -> float:
        return float(self.head_outputs().get(str(head_name), 0.0))

    @torch.no_grad()
    def update_head_from_hidden(self, *, head_name: str, hidden: Sequence[float], reward: float,
                                learning_rate: float, reward_clip: float = 5.0, weight_clip: float = 1.0) -> None:
        """Reward-weighted Hebbian step on one head: ``w += lr * clip(reward) * hidden`` (weights and bias
        clipped to ``+-weight_clip``)."""
        idx = self._head_index.get(str(head_name))
        lr, r = float(learning_rate), float(reward)
        if idx is None or lr <= 0.0 or not math.isfinite(r):
            return
        clip, limit = abs(float(reward_clip)), abs(float(weight_clip))
        if clip > 0.0:
            r = max(-clip, min(clip, r))
        h = torch.as_tensor(list(hidden), dtype=torch.float32)[: self.hidden_dim]
        w = self.W_head[: h.numel(), idx] + lr * r * h
        b = self.b_head[idx] + lr * r
        if limit > 0.0:
            w, b = w.clamp(-limit, limit), b.clamp(-limit, limit)
        self.W_head[: h.numel(), idx] = w
        self.b_head[idx] = b

    def diagnostics(self) -> dict[str, Any]:
        H, Fd, Nh = self.hidden_dim, len(self.feature_names), len(self.head_names)
        return {"recurrence_mode": "full_a_event_ssm", "hidden_dim": H, "rank": self.rank, "feature_dim": Fd,
                "head_count": Nh, "top_log_sv": self._top_log_sv, "state_norm": float(self.state.norm()),
                "state_clamp_count": self._state_clamp_count, "controller_work_units": Fd * H + H * H + H * Nh}

    def work_ratio_vs_bare_ssm(self, *, batch: int = 1024, seq: int = 512, dim: int = 384, layers: int = 4) -> float:
        """Multiply-accumulates of one controller step over those of one recurrence pass of the trunk."""
        return float(self.diagnostics()["controller_work_units"]) / float(max(1, batch * seq * dim * layers))


@dataclass
class ActionSpaceTrace:
    rows: list = field(default_factory=list)

    def append(self, row: dict[str, Any]) -> None:
        self.rows.append(row)


def _default_specs() -> dict[str, BoundedScalarSpec]:
    table = (("temperature", 0.25, 4.0, "softplus"), ("entropy_beta", 0.0, 0.2, "sigmoid"),
             ("ema_alpha", 0.0, 0.5, "sigmoid"), ("replay_budget", 0.0, 16.0, "sigmoid"),
             ("write_budget", 0.0, 16.0, "sigmoid"), ("eviction", 0.0, 1.0, "sigmoid"),
             ("consolidation", 0.0, 1.0, "sigmoid"))
    return {n: BoundedScalarSpec(n, lo, hi, transform=t) for n, lo, hi, t in table}


@dataclass
class ConstrainedActionSpace:
    trace_only: bool = False
    selection_readiness: float = 0.0
    selection_max_delta: float = 0.0
    max_tags_per_query: Optional[int] = None
    head_readiness: dict = field(default_factory=dict)
    head_max_delta: dict = field(default_factory=dict)
    scalar_specs: dict = field(default_factory=dict)
    event_ssm: Optional[SharedEventSsm] = None
    trace_log: Any = None
    online_learning_rate: float = 0.0
    reward_clip: float = 5.0
    credit_history: dict = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.selection_readiness = _clamp01(self.selection_readiness)
        if not math.isfinite(float(self.selection_max_delta)):
            raise ValueError("selection_max_delta must be finite")
        if self.selection_max_delta < 0.0:
            raise ValueError("selection_max_delta must be non-negative")
        if self.max_tags_per_query is not None and self.max_tags_per_query < 0:
            raise ValueError("max_tags_per_query must be >= 0")
        self.head_readiness = {str(k): _clamp01(v) for k, v in self.head_readiness.items()}
        deltas = {}
        for k, v in self.head_max_delta.items():
            v = float(v)
            if not math.isfinite(v):
                raise ValueError(f"{k}.max_delta must be finite")
            if v < 0.0:
                raise ValueError(f"{k}.max_delta must be non-negative")
            deltas[str(k)] = v
        self.head_max_delta = deltas
        if not self.scalar_specs:
            self.scalar_specs = _default_specs()
        if self.online_learning_rate < 0.0:
            raise ValueError("online_learning_rate must be non-negative")

    # -- gates --------------------------------------------------------------
    def readiness(self, head_name: str) -> float:
        default = self.selection_readiness if str(head_name) == "selection_rank" else 0.0
        return float(self.head_readiness.get(str(head_name), default))

    def max_delta(self, head_name: str) -> float:
        default = self.selection_max_delta if str(head_name) == "selection_rank" else 0.0
        return float(self.head_max_delta.get(str(head_name), default))

    def active_head(self, head_name: str) -> bool:
        return not self.trace_only and self.readiness(head_name) > 0.0 and self.max_delta(head_name) > 0.0

    @property
    def active_selection(self) -> bool:
        return not self.trace_only and self.selection_readiness > 0.0 and self.selection_max_delta > 0.0

    def _record(self, gpu_step: int, event_type: str, head_name: str, raw: Any, bounded: Any, invariant: str,
                clamp: float, readiness: float, ctx: Optional[dict], accepted: bool) -> None:
        if self.trace_log is not None:
            self.trace_log.append({
                "gpu_step": int(gpu_step), "event_type": event_type, "head_name": head_name, "raw_action": raw,
                "bounded_action": bounded, "invariant_name": invariant, "clamp_amount": float(clamp),
                "readiness": float(readiness), "reward_context": dict(ctx or {}), "accepted": bool(accepted)})

    # -- actions ------------------------------------------------------------
    def effective_scores(self, *, heuristic_scores: Sequence[float], learned_scores: Optional[Sequence[float]],
                         gpu_step: int, head_name: str = "selection_rank",
                         reward_context: Optional[dict] = None) -> list[float]:
        base = [float(x) for x in heuristic_scores]
        head = str(head_name)
        if not base or not self.active_head(head):
            return base
        if learned_scores is None and self.event_ssm is not None:
            learned_scores = []
            for i, sc in enumerate(base):
                feats = {"score": sc, "rank": float(i)}
                feats.update({str(k): float(v) for k, v in (reward_context or {}).items()
                              if isinstance(v, (int, float))})
                learned_scores.append(self.event_ssm.observe(feats).get(head, 0.0))
        if learned_scores is None:
            return base
        raw = [float(x) for x in learned_scores]
        if len(raw) != len(base):
            raise ValueError("learned_scores must have the same length as heuristic_scores")
        ready = self.readiness(head)
        scale = self.max_delta(head) * ready
        deltas = [_tanh_or_zero(x) * scale for x in raw]
        self._record(gpu_step, "action_space_delta", head, raw, deltas, "bounded_residual", 0.0, ready,
                     reward_context, True)
        return [b + d for b, d in zip(base, deltas)]

    def selected_indices(self, *, effective_scores: Sequence[float], gpu_step: int, requested_budget: int,
                         head_name: str = "replay_budget", reward_context: Optional[dict] = None) -> list[int]:
        n = len(effective_scores)
        want = min(n, max(0, int(requested_budget)))
        budget = want if self.max_tags_per_query is None else min(want, int(self.max_tags_per_query))
        if budget < want:
            self._record(gpu_step, "action_space_clamp", str(head_name), int(max(0, int(requested_budget))),
                         int(budget), "max_tags_per_query", float(want - budget), self.readiness(head_name),
                         reward_context, budget > 0)
        if budget <= 0:
            return []
        return sorted(range(n), key=lambda i: (-float(effective_scores[i]), i))[:budget]

    def scalar_value(self, *, head_name: str, raw_value: Optional[float] = None, gpu_step: int, fallback: float,
                     reward_context: Optional[dict] = None) -> float:
        head = str(head_name)
        ready = self.readiness(head)
        if self.trace_only or ready <= 0.0:
            return float(fallback)
        raw = raw_value
        if raw is None and self.event_ssm is not None:
            raw = self.event_ssm.observe(reward_context or {}).get(head, 0.0)
        if raw is None:
            return float(fallback)
        spec = self.scalar_specs.get(head)
        if spec is None:
            raise KeyError(f"no scalar spec configured for head {head!r}")
        value = (1.0 - ready) * float(fallback) + ready * float(spec.map(float(raw)))
        self._record(gpu_step, "action_space_scalar", head, float(raw), float(value), f"{head}_range", 0.0, ready,
                     reward_context, True)
        return float(value)

    # -- delayed credit -----------------------------------------------------
    def record_credit_assignment(self, *, key: int, head_names: Sequence[str], gpu_step: int,
                                 reward_context: Optional[dict] = None) -> None:
        if self.event_ssm is None or self.online_learning_rate <= 0.0:
            return
        snap = self.event_ssm.hidden
        entries = [(str(h), list(snap)) for h in head_names if str(h) in self.event_ssm._head_index]
        if not entries:
            return
        self.credit_history[int(key)] = entries
        self._record(gpu_step, "action_space_credit_record", ",".join(h for h, _ in entries), int(key), len(entries),
                     "reward_key", 0.0, 1.0, reward_context, True)

    def apply_reward(self, *, key: int, reward: float, gpu_step: int, reward_context: Optional[dict] = None) -> int:
        if self.event_ssm is None or self.online_learning_rate <= 0.0:
            return 0
        entries = self.credit_history.pop(int(key), [])
        for head, hidden in entries:
            self.event_ssm.update_head_from_hidden(head_name=head, hidden=hidden, reward=float(reward),
                                                   learning_rate=float(self.online_learning_rate),
                                                   reward_clip=float(self.reward_clip))
        if entries:
            self._record(gpu_step, "action_space_reward_update", ",".join(h for h, _ in entries), float(reward),
                         len(entries), "clipped_reward_update", 0.0, 1.0, reward_context, True)
        return len(entries)


def coerce_action_space(value: Any) -> Optional[ConstrainedActionSpace]:
    if value is None or value is False:
        return None
    if isinstance(value, ConstrainedActionSpace):
        return value
    if isinstance(value, dict):
        return ConstrainedActionSpace(**value)
    raise TypeError("action_space must be None, False, a dict, or ConstrainedActionSpace")


ACTION_SPACE_HEADS = ("write_admission", "eviction", "replay_timing", "replay_budget", "write_budget", "temperature",
                      "entropy_beta", "ema_alpha", "consolidation", "selection_rank")


def _head_value(config: Mapping[str, Any], head: str, what: str, default: float) -> float:
    """``episodic_controller_head_<what>: {head: value}`` wins over ``episodic_controller_<head>_<what>``."""
    table = config.get(f"episodic_controller_head_{what}")
    if isinstance(table, Mapping) and head in table:
        return float(table[head])
    return float(config.get(f"episodic_controller_{head}_{what}", default))


def build_action_space_from_config(config: Mapping[str, Any], *, trace_log: Any = None) -> Optional["ConstrainedActionSpace"]:
    """The bounded action space of the episodic controller as the run config describes it, or None when
    ``episodic_controller_action_space_enabled`` is off (runner_fast_path.py:6790-6850 of the reference):
    per-head readiness and maximal deviation, the selection head's pair under its own two keys, an optional
    cap on tags per query, trace-only mode, the shared event recurrence (on unless switched off) and the
    online learning rate / reward clip of the heads."""
    if not bool(config.get("episodic_controller_action_space_enabled", False)):
        return None
    ready = {h: _head_value(config, h, "readiness", 0.0) for h in ACTION_SPACE_HEADS}
    delta = {h: _head_value(config, h, "max_delta", 0.0) for h in ACTION_SPACE_HEADS}
    ready["selection_rank"] = float(config.get("episodic_controller_selection_readiness", ready["selection_rank"]))
    delta["selection_rank"] = float(config.get("episodic_controller_selection_max_delta", delta["selection_rank"]))
    max_tags = config.get("episodic_controller_max_tags_per_query")
    return ConstrainedActionSpace(
        trace_only=bool(config.get("episodic_controller_action_space_trace_only", False)),
        selection_readiness=ready["selection_rank"], selection_max_delta=delta["selection_rank"],
        max_tags_per_query=None if max_tags is None else int(max_tags), head_readiness=ready, head_max_delta=delta,
        event_ssm=(make_shared_event_ssm_from_config(config)
                   if bool(config.get("episodic_controller_shared_event_ssm_enabled", True)) else None),
        trace_log=trace_log, online_learning_rate=float(config.get("episodic_controller_action_learning_rate", 0.0)),
        reward_clip=float(config.get("episodic_controller_action_reward_clip", 5.0)))


def make_shared_event_ssm_from_config(config: Mapping[str, Any]) -> SharedEventSsm:
    g = config.get
    return SharedEventSsm(hidden_dim=int(g("episodic_controller_ssm_hidden_dim", 16)),
                          seed=int(g("episodic_controller_ssm_seed", 0)),
                          decay=float(g("episodic_controller_ssm_decay", 0.95)),
                          input_scale=float(g("episodic_controller_ssm_input_scale", 0.05)),
                          head_scale=float(g("episodic_controller_ssm_head_scale", 0.05)))
