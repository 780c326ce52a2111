"""Parallel time-horizon heads at evaluation: the same checkpoint is scored under
several ``log_a`` shifts and the per-head next-token distributions are mixed in
probability space (behaviour of src/chaoscontrol/eval_stream/temporal_heads.py:17-607).

Three mixers: uniform, fixed pre-registered weights, and causal exponential
weights.  The exponential-weights mixer is a prefix sum here, not a token loop:
the weights that score position ``t`` are
``softmax(log w0 + eta * sum_{s<t} log p_head(target_s))`` (an exclusive
cumulative sum over the sequence), so one ``cumsum`` + one ``logsumexp`` give the
whole chunk and the carried weights for the next chunk.

``score_temporal_heads_chunk`` leaves the model untouched: every head runs
inside a ``DeltaModulator`` that restores ``log_a`` on exit.  With
``capture_half_lives=False`` no module hooks are installed, so a bare-SSM bf16
model keeps its hand-scheduled trunk for every head.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Literal, Optional, Sequence, Union

import torch
import torch.nn.functional as F

from ..models.core import CareSSMCore
from .state import DeltaModulator

HeadKey = Union[float, str]

_MIXERS = ("uniform_logprob", "base_prior_logprob", "online_exp_weights_logprob")

__all__ = ["HeadKey", "TemporalHeadConfig", "TemporalHeadChunkResult", "PreviousChunkPriorityGate",
           "uniform_logprob_mixture", "weighted_logprob_mixture", "online_exp_weighted_logprob_mixture",
           "update_online_exp_weighted_log_weights", "score_temporal_heads_chunk",
           "make_same_horizon_virtual_depth_config"]


# ---------------------------------------------------------------- mixtures
def _positive_normalised_log(weights: Sequence[float], n: int, ref: torch.Tensor, what: str,
                             label: str) -> torch.Tensor:
    if len(weights) != n:
        raise ValueError(f"{what} length {len(weights)} does not match log_probs length {n}")
    w = torch.tensor(tuple(float(x) for x in weights), device=ref.device, dtype=ref.dtype)
    if bool((w <= 0).any()):
        raise ValueError(f"all {label} must be positive")
    return (w / w.sum()).log()


def uniform_logprob_mixture(log_probs: list[torch.Tensor]) -> torch.Tensor:
    """``log(mean_h p_h)`` over heads."""
    if not log_probs:
        raise ValueError("uniform_logprob_mixture requires at least one tensor")
    if len(log_probs) == 1:
        return log_probs[0]
    return torch.logsumexp(torch.stack(log_probs, 0), dim=0) - math.log(len(log_probs))


def weighted_logprob_mixture(log_probs: list[torch.Tensor], *, weights: tuple[float, ...]) -> torch.Tensor:
    """``log(sum_h w_h p_h)`` with fixed positive weights (normalised here)."""
    if not log_probs:
        raise ValueError("weighted_logprob_mixture requires at least one tensor")
    lw = _positive_normalised_log(weights, len(log_probs), log_probs[0], "weights", "mixture weights")
    stacked = torch.stack(log_probs, 0)
    return torch.logsumexp(stacked + lw.view(-1, *([1] * log_probs[0].ndim)), dim=0)


def update_online_exp_weighted_log_weights(log_weights: torch.Tensor, head_log_probs: list[torch.Tensor],
                                           target: torch.Tensor, *, eta: float) -> torch.Tensor:
    """One exponential-weights step after ``target`` [B] has been scored:
    ``log w <- log_softmax(log w + eta * log p_head(target))``; ``log_weights`` is [B, H]."""
    if eta < 0.0:
        raise ValueError("eta must be non-negative")
    if not head_log_probs:
        raise ValueError("head_log_probs requires at least one tensor")
    batch, heads = log_weights.shape
    if heads != len(head_log_probs):
        raise ValueError(f"log_weights head count {heads} does not match head_log_probs length "
                         f"{len(head_log_probs)}")
    if tuple(target.shape) != (batch,):
        raise ValueError(f"target shape {tuple(target.shape)} does not match expected {(batch,)}")
    lp = torch.stack(head_log_probs, 1)                                        # [B, H, V]
    tok = lp.gather(-1, target.to(lp.device).view(batch, 1, 1).expand(batch, heads, 1)).squeeze(-1)
    return torch.log_softmax(log_weights + float(eta) * tok.to(log_weights.device), dim=1)


def _online_mixture(log_probs: list[torch.Tensor], targets: torch.Tensor, *, eta: float,
                    initial_weights: Optional[tuple[float, ...]] = None,
                    initial_log_weights: Optional[torch.Tensor] = None
                    ) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Mixed log-probs [B, T, V] and the weights after the last target [B, H] (``None`` for one head)."""
    if not log_probs:
        raise ValueError("online_exp_weighted_logprob_mixture requires at least one tensor")
    if len(log_probs) == 1:
        return log_probs[0], None
    if eta < 0.0:
        raise ValueError("eta must be non-negative")
    shape = log_probs[0].shape
    if len(shape) != 3:
        raise ValueError("log_probs tensors must have shape [batch, seq, vocab]")
    if any(lp.shape != shape for lp in log_probs):
        raise ValueError("all log_probs tensors must have the same shape")
    batch, seq, _ = shape
    heads = len(log_probs)
    if tuple(targets.shape) != (batch, seq - 1):
        raise ValueError(f"targets shape {tuple(targets.shape)} does not match expected {(batch, seq - 1)}")
    ref = log_probs[0]
    if initial_log_weights is not None:
        if tuple(initial_log_weights.shape) != (batch, heads):
            raise ValueError(f"initial_log_weights shape {tuple(initial_log_weights.shape)} does not match "
                             f"expected {(batch, heads)}")
        lw0 = initial_log_weights.to(device=ref.device, dtype=ref.dtype)
    else:
        lw0 = _positive_normalised_log(initial_weights or (1.0,) * heads, heads, ref, "initial_weights",
                                       "initial online weights")
        lw0 = lw0.unsqueeze(0).expand(batch, -1)
    stacked = torch.stack(log_probs, 1)                                        # [B, H, T, V]
    idx = targets.to(ref.device).view(batch, 1, seq - 1, 1).expand(batch, heads, seq - 1, 1)
    tok = stacked[:, :, :-1].gather(-1, idx).squeeze(-1)                       # [B, H, T-1]
    # evidence seen BEFORE position t: exclusive prefix sum, positions 0..T-1, plus the final state
    evidence = F.pad(torch.cumsum(tok, dim=-1), (1, 0)) * float(eta)           # [B, H, T]
    lw = torch.log_softmax(lw0.unsqueeze(-1) + evidence, dim=1)                # [B, H, T]
    mixed = torch.logsumexp(stacked + lw.unsqueeze(-1), dim=1)
    return mixed, lw[:, :, -1].contiguous()


def online_exp_weighted_logprob_mixture(log_probs: list[torch.Tensor], targets: torch.Tensor, *, eta: float,
                                        initial_weights: Optional[tuple[float, ...]] = None) -> torch.Tensor:
    """Causal token-level exponential-weights mixture: position ``t`` is scored
    with weights that saw only targets ``< t``."""
    return _online_mixture(log_probs, targets, eta=eta, initial_weights=initial_weights)[0]


# ---------------------------------------------------------------- config / result / gate
@dataclass(frozen=True)
class TemporalHeadConfig:
    horizon_shifts: tuple[float, ...] = (-0.5, 0.0, 0.5)
    head_ids: Optional[tuple[str, ...]] = None
    horizon_knob: Literal["log_a_shift"] = "log_a_shift"
    mixer: Literal["uniform_logprob", "base_prior_logprob", "online_exp_weights_logprob"] = "uniform_logprob"
    mixer_weights: Optional[tuple[float, ...]] = None
    online_eta: float = 1.0
    online_initial_weights: Optional[tuple[float, ...]] = None
    policy: Literal["always", "previous_chunk_priority"] = "always"
    threshold: Optional[float] = None


@dataclass
class TemporalHeadChunkResult:
    loss_nats: float
    tokens_scored: int
    mixed_log_probs: torch.Tensor
    final_states_by_shift: dict
    per_head_loss_nats: dict
    winner_counts_by_shift: dict
    half_life_stats_by_shift: dict
    state_divergence_by_shift: dict
    last_mixed_log_probs: Optional[torch.Tensor] = None
    last_log_probs_by_shift: Optional[dict] = None
    online_final_log_weights: Optional[torch.Tensor] = None


@dataclass
class PreviousChunkPriorityGate:
    """Decides from the PREVIOUS chunk's signals whether the extra heads run on the
    next one: priority = weighted entropy + loss spike + state-delta norm
    (+ optional EMA of head disagreement), run iff priority > threshold and the
    remaining slack covers the extra cost."""
    threshold: float
    entropy_weight: float = 1.0
    loss_spike_weight: float = 1.0
    state_delta_weight: float = 1.0
    use_disagreement_ema: bool = False
    disagreement_weight: float = 0.0
    disagreement_decay: float = 0.9

    def __post_init__(self) -> None:
        self._priority = 0.0
        self._disagreement_ema = 0.0

    def update_after_chunk(self, *, entropy: float, loss_spike: float, state_delta_norm: float,
                           head_disagreement: Optional[float] = None, temporal_heads_ran: bool = False) -> None:
        if not self.use_disagreement_ema:
            self._disagreement_ema = 0.0
        else:
            self._disagreement_ema *= self.disagreement_decay
            if temporal_heads_ran and head_disagreement is not None:
                self._disagreement_ema += (1.0 - self.disagreement_decay) * float(head_disagreement)
        self._priority = (self.entropy_weight * float(entropy) + self.loss_spike_weight * float(loss_spike) +
                          self.state_delta_weight * float(state_delta_norm) +
                          self.disagreement_weight * self._disagreement_ema)

    def should_run(self, *, extra_cost_seconds: float, slack_remaining_seconds: float) -> bool:
        return self._priority > self.threshold and float(slack_remaining_seconds) >= float(extra_cost_seconds)


# ---------------------------------------------------------------- helpers
def _head_keys(cfg: TemporalHeadConfig) -> tuple:
    shifts = cfg.horizon_shifts
    if cfg.head_ids is None:
        if len(set(shifts)) != len(shifts):
            raise ValueError("duplicate horizon_shifts require explicit head_ids")
        return tuple(shifts)
    if len(cfg.head_ids) != len(shifts):
        raise ValueError(f"head_ids length {len(cfg.head_ids)} does not match horizon_shifts length "
                         f"{len(shifts)}")
    if len(set(cfg.head_ids)) != len(cfg.head_ids):
        raise ValueError("head_ids must be unique")
    return tuple(cfg.head_ids)


def _default_base_prior_weights(shifts: tuple[float, ...]) -> tuple[float, ...]:
    if len(shifts) != 3 or 0.0 not in shifts:
        raise ValueError("base_prior_logprob default weights require exactly three heads including 0.0")
    return tuple(0.8 if s == 0.0 else 0.1 for s in shifts)


class _DeltaMeans:
    """Running per-channel mean of ``softplus(delta_proj(x))`` per core, fed by forward hooks."""

    def __init__(self, cores: list) -> None:
        self.sums: list[Optional[torch.Tensor]] = [None] * len(cores)
        self.rows = [0] * len(cores)
        self._handles = [c.delta_proj.register_forward_hook(self._hook(i)) for i, c in enumerate(cores)]

    def _hook(self, i: int):
        def fn(_m, _inp, out):
            d = F.softplus(out.detach()).clamp_min(1e-4).reshape(-1, out.shape[-1]).float()
            self.sums[i] = d.sum(0) if self.sums[i] is None else self.sums[i] + d.sum(0)
            self.rows[i] += d.shape[0]
        return fn

    def close(self) -> list[Optional[torch.Tensor]]:
        for h in self._handles:
            h.remove()
        return [None if s is None else s / max(n, 1) for s, n in zip(self.sums, self.rows)]


def _half_lives(cores: list, mean_deltas: list[Optional[torch.Tensor]], shift: float) -> list[Optional[torch.Tensor]]:
    """``ln 2 / (mean_delta * sigmoid(log_a + shift))`` per channel: tokens until a state halves."""
    out: list[Optional[torch.Tensor]] = []
    for core, md in zip(cores, mean_deltas):
        if md is None or not hasattr(core, "log_a"):
            out.append(None)
            continue
        a = torch.sigmoid(core.log_a.detach().to(md.device).float() + float(shift))
        if md.numel() == 1 and a.numel() > 1:
            md = md.expand_as(a)
        out.append(None if md.shape != a.shape else math.log(2.0) / (md * a).clamp_min(1e-8))
    return out


def _half_life_summary(raw: dict, base_key) -> dict:
    base = raw.get(base_key) if base_key is not None else None
    summary: dict = {}
    for key, layers in raw.items():
        rows = []
        for li, hl in enumerate(layers):
            if hl is None:
                rows.append({"layer": li, "p10": None, "median": None, "p90": None,
                             "separated_fraction_vs_base": None})
                continue
            q = torch.quantile(hl.reshape(-1).float().cpu(), torch.tensor([0.10, 0.50, 0.90]))
            sep = None
            if base is not None and li < len(base) and base[li] is not None and base[li].shape == hl.shape:
                octaves = torch.log2((hl.float() / base[li].float()).clamp_min(1e-8))
                sep = float((octaves.abs() >= 0.5).float().mean())
            rows.append({"layer": li, "p10": float(q[0]), "median": float(q[1]), "p90": float(q[2]),
                         "separated_fraction_vs_base": sep})
        summary[key] = rows
    return summary


def _state_divergence(finals: dict, base_key) -> dict:
    base = finals.get(base_key) if base_key is not None else None
    if not base:
        return {}
    out: dict = {}
    for key, states in finals.items():
        if key == base_key or len(states) != len(base):
            continue
        s = torch.stack([x.detach().float() for x in states], 0)               # [L, B, D]
        b = torch.stack([x.detach().float() for x in base], 0)
        l2 = (s - b).norm(dim=-1).mean(-1).tolist()
        cos = F.cosine_similarity(s, b, dim=-1).mean(-1).tolist()
        out[key] = [{"layer": li, "l2_vs_base": float(l2[li]), "cosine_vs_base": float(cos[li])}
                    for li in range(len(states))]
    return out


# ---------------------------------------------------------------- scoring
def score_temporal_heads_chunk(model, chunk: torch.Tensor, *, states_by_shift: dict, cfg: TemporalHeadConfig,
                               online_initial_log_weights: Optional[torch.Tensor] = None,
                               capture_half_lives: bool = True) -> TemporalHeadChunkResult:
    """Scores ``chunk`` [B, T] under every horizon shift and mixes the heads; no
    parameter or mixer state outside the returned result is changed."""
    if chunk.size(1) < 1:
        raise ValueError(f"score_temporal_heads_chunk needs chunk length >= 1; got {tuple(chunk.shape)}")
    if cfg.horizon_knob != "log_a_shift":
        raise ValueError(f"unsupported horizon_knob: {cfg.horizon_knob!r}")
    if cfg.mixer not in _MIXERS:
        raise ValueError(f"unsupported mixer: {cfg.mixer!r}")
    model.eval()
    targets = chunk[:, 1:]
    keys = _head_keys(cfg)
    base_key = next((k for k, s in zip(keys, cfg.horizon_shifts) if s == 0.0), None)
    cores = [m for m in model.modules() if isinstance(m, CareSSMCore)]
    log_probs: list[torch.Tensor] = []
    finals: dict = {}
    raw_half_lives: dict = {}
    with torch.no_grad():
        for key, shift in zip(keys, cfg.horizon_shifts):
            kwargs = {}
            if states_by_shift.get(key):
                kwargs["initial_states"] = states_by_shift[key]
            tap = _DeltaMeans(cores) if capture_half_lives else None
            try:
                with DeltaModulator(model, log_a_shift=shift):
                    out = model(chunk, **kwargs)
            finally:
                means = tap.close() if tap is not None else [None] * len(cores)
            raw_half_lives[key] = _half_lives(cores, means, shift)
            logits = out["logits"] if isinstance(out, dict) else out
            log_probs.append(F.log_softmax(logits.float(), dim=-1))
            finals[key] = ([s.detach().clone() for s in out["final_states"]]
                           if isinstance(out, dict) and "final_states" in out else [])
        final_lw = None
        if cfg.mixer == "uniform_logprob":
            mixed = uniform_logprob_mixture(log_probs)
        elif cfg.mixer == "base_prior_logprob":
            mixed = weighted_logprob_mixture(
                log_probs, weights=cfg.mixer_weights or _default_base_prior_weights(cfg.horizon_shifts))
        else:
            mixed, final_lw = _online_mixture(log_probs, targets, eta=cfg.online_eta,
                                              initial_weights=cfg.online_initial_weights,
                                              initial_log_weights=online_initial_log_weights)
        tidx = targets.unsqueeze(-1)
        head_nll = -torch.stack([lp[:, :-1].gather(-1, tidx).squeeze(-1) for lp in log_probs], 0)  # [H, B, T-1]
        winners = torch.bincount(head_nll.argmin(0).reshape(-1), minlength=len(keys)).tolist()
        per_head = head_nll.sum((1, 2)).tolist()
        loss = float(-mixed[:, :-1].gather(-1, tidx).sum())
    return TemporalHeadChunkResult(
        loss_nats=loss, tokens_scored=int(targets.numel()), mixed_log_probs=mixed, final_states_by_shift=finals,
        per_head_loss_nats={k: float(v) for k, v in zip(keys, per_head)},
        winner_counts_by_shift={k: int(v) for k, v in zip(keys, winners)},
        half_life_stats_by_shift=_half_life_summary(raw_half_lives, base_key),
        state_divergence_by_shift=_state_divergence(finals, base_key),
        last_mixed_log_probs=mixed[:, -1].detach().clone(),
        last_log_probs_by_shift={k: lp[:, -1].detach().clone() for k, lp in zip(keys, log_probs)},
        online_final_log_weights=None if final_lw is None else final_lw.detach().clone())


def make_same_horizon_virtual_depth_config(cfg: dict, *, depth_recurrence_count: int) -> dict:
    """Model config of the compute-matched control: instead of H heads with
    different horizons, the same layers are re-run ``depth_recurrence_count``
    times (all layers shared unless the config already names a shared subset)."""
    if depth_recurrence_count < 1:
        raise ValueError("depth_recurrence_count must be >= 1")
    out = dict(cfg)
    out["depth_recurrence_shared_layers"] = (list(out.get("depth_recurrence_shared_layers") or []) or
                                             list(range(int(out["num_layers"]))))
    out["depth_recurrence_count"] = int(depth_recurrence_count)
    return out
