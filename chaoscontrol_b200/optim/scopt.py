"""Scarcity-aware optimizer ("ScOpt"): Muon plus rare-event state
(behaviour of src/chaoscontrol/optim/scopt.py:27-1042).

* event pressure: ``rarity(token) * max(CE - baseline, 0)``, detached, with an
  optional robust upper clamp;
* a rare-gradient EMA per parameter, whose component ORTHOGONAL to Muon's own
  Nesterov direction is added back (capped at ``rare_macro_c`` times the common
  norm), so rare events steer the update without fighting the common gradient;
* row scarcity for token-indexed matrices and two-sided (output x input)
  channel scarcity for projection matrices, applied BEFORE the orthogonalisation
  as ``1 + tanh(pressure / tau)`` factors;
* a recurrence-timescale-weighted factor on 1-D parameters such as ``log_a``.

With no scarcity state supplied (or during ``warmup_steps``) the update is
exactly Muon for matrices and AdamW for the rest.  The training loop owns the
autograd work and feeds state through ``update_rare_grad_ema`` /
``update_row_pressure_ema`` / ``set_channel_pressure``.

Telemetry scalars stay on the device until ``scarcity_trace()`` reads them.
"""
from __future__ import annotations

from collections import defaultdict
from collections.abc import Iterable, Mapping
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch
from torch import Tensor

from .muon import newton_schulz_orthogonalize

__all__ = ["FrequencyBucketBaseline", "scarcity_pressure_from_ce", "ScOptAllReduceConfig", "scopt_allreduce_config",
           "ScarcityAwareOptimizer", "scopt_optimizer_config"]


class FrequencyBucketBaseline:
    """EMA of the mean CE per log-frequency bucket of the target token: a cheap
    "expected loss" to measure surprise against."""

    def __init__(self, token_frequencies: Tensor, *, num_buckets: int = 16, decay: float = 0.99, device=None) -> None:
        if token_frequencies.ndim != 1:
            raise ValueError("token_frequencies must be 1D")
        if num_buckets < 1:
            raise ValueError(f"num_buckets must be >= 1, got {num_buckets}")
        if not 0.0 <= decay < 1.0:
            raise ValueError(f"decay must be in [0, 1), got {decay}")
        dev = device if device is not None else token_frequencies.device
        lf = torch.log1p(token_frequencies.float().clamp_min(0.0))
        lo, hi = float(lf.min()), float(lf.max())
        edges = torch.linspace(lo, lo + max(hi - lo, 1e-6) + 1e-6, num_buckets + 1, device=lf.device)
        self._token_bucket = torch.bucketize(lf, edges[1:-1]).clamp_(0, num_buckets - 1).to(dev)
        self._ema = torch.zeros(num_buckets, device=dev)
        self._initialized = torch.zeros(num_buckets, device=dev, dtype=torch.bool)
        self._decay, self._num_buckets = float(decay), int(num_buckets)

    def baseline(self, targets: Tensor) -> Tensor:
        return self._ema[self._token_bucket[targets]]

    @torch.no_grad()
    def update(self, ce: Tensor, targets: Tensor) -> None:
        """Buckets seen for the first time adopt the observed mean; the rest move by the EMA."""
        ce_f = ce.detach().to(device=self._ema.device, dtype=torch.float32).reshape(-1)
        b = self._token_bucket[targets.reshape(-1).to(self._ema.device)]
        s = torch.zeros_like(self._ema).index_add_(0, b, ce_f)
        c = torch.zeros_like(self._ema).index_add_(0, b, torch.ones_like(ce_f))
        seen = c > 0
        obs = torch.where(seen, s / c.clamp_min(1.0), self._ema)
        moved = torch.where(seen & ~self._initialized, obs, self._decay * self._ema + (1.0 - self._decay) * obs)
        self._ema = torch.where(seen, moved, self._ema)
        self._initialized |= seen

    def state_dict(self) -> dict[str, Any]:
        return {"ema": self._ema.detach().cpu().clone(), "initialized": self._initialized.detach().cpu().clone(),
                "token_bucket": self._token_bucket.detach().cpu().clone(), "decay": self._decay,
                "num_buckets": self._num_buckets}


@torch.no_grad()
def scarcity_pressure_from_ce(ce: Tensor, targets: Tensor, *, token_frequencies: Tensor,
                              baseline: Tensor | float | None = None, eps: float = 1e-8,
                              upper_c: Optional[float] = None, upper_floor: float = 1.0) -> Tensor:
    """Detached ``pressure = excess_CE / log1p(freq[target])``.  ``upper_c`` clamps it at
    ``max(upper_c * std(pressure below its p95), upper_floor)`` so a few exploded
    tokens cannot dominate the rare-gradient accumulation."""
    if token_frequencies.ndim != 1:
        raise ValueError("token_frequencies must be a 1D tensor indexed by token id")
    if ce.shape != targets.shape:
        raise ValueError(f"ce and targets must have matching shape, got {tuple(ce.shape)} and {tuple(targets.shape)}")
    rarity = 1.0 / torch.log1p(token_frequencies.to(device=targets.device, dtype=torch.float32)[targets]
                               .clamp_min(float(eps)))
    ce_d = ce.detach().float()
    if baseline is None:
        base = torch.zeros_like(ce_d)
    elif isinstance(baseline, Tensor):
        base = baseline.to(device=ce.device, dtype=torch.float32)
        if base.ndim == 0:
            base = torch.full_like(ce_d, float(base))
        elif base.shape != ce.shape:
            raise ValueError(f"baseline must match ce shape, got {tuple(base.shape)} and {tuple(ce.shape)}")
    else:
        base = torch.full_like(ce_d, float(baseline))
    pressure = rarity * (ce_d - base).clamp_min(0.0)
    if upper_c is not None:
        if pressure.numel() >= 10:
            scale = pressure.clamp_max(pressure.flatten().quantile(0.95)).std(unbiased=False)
        elif pressure.numel() > 1:
            scale = pressure.std(unbiased=False)
        else:
            scale = pressure.new_zeros(())
        pressure = pressure.clamp_max(torch.maximum(scale * float(upper_c), pressure.new_tensor(float(upper_floor))))
    return pressure.to(device=ce.device, dtype=torch.float32)


@dataclass(frozen=True)
class ScOptAllReduceConfig:
    op: str
    train_grad_scale: float
    train_rank_count: int
    materialize_zeros: bool


def scopt_allreduce_config(*, world_size: int, all_group: object | None) -> ScOptAllReduceConfig:
    """SUM with pre-scaled train-rank gradients.  With an ``all_group`` (one extra
    non-train rank that submits zeros) the scale is ``1 / (world - 1)``."""
    w = int(world_size)
    if w <= 1:
        return ScOptAllReduceConfig("sum", 1.0, 1, False)
    n = w if all_group is None else w - 1
    if n < 1:
        raise ValueError(f"ScOpt all_group topology requires world_size >= 2 (1 train + 1 non-train), got world_size={w}")
    return ScOptAllReduceConfig("sum", 1.0 / n, n, all_group is not None)


def scopt_optimizer_config(model: torch.nn.Module, layer_index: int) -> dict[str, Any]:
    """Two-sided scarcity map for one block: each projection is keyed by its own output
    (``<module>.__out__``) and input (``<module>.__in__``) activation pressure; ``log_a``
    follows the first content projection's output."""
    prefix = f"layers.{int(layer_index)}.core"
    params = {n for n, _ in model.named_parameters()}
    modules = {n for n, _ in model.named_modules()}
    if f"{prefix}.log_a" not in params:
        raise ValueError(f"ScOpt requires {prefix + '.log_a'!r}")
    present = [s for s in ("in_proj", "select_proj", "gate_proj", "delta_proj", "out_proj") if f"{prefix}.{s}" in modules]
    if not present:
        raise ValueError(f"ScOpt requires projection submodules under {prefix!r}")
    mmap = {f"{prefix}.{s}.weight": (f"{prefix}.{s}.__out__", f"{prefix}.{s}.__in__")
            for s in present if f"{prefix}.{s}.weight" in params}
    if not mmap:
        raise ValueError(f"ScOpt requires at least one channel-coupled matrix under {prefix!r}")
    src = next((s for s in ("in_proj", "select_proj", "gate_proj") if s in present), present[0])
    return {"row_param_names": {"embed.weight", "lm_head.weight"}, "matrix_scarcity_map": mmap,
            "recurrence_scarcity_map": {f"{prefix}.log_a": f"{prefix}.{src}.__out__"}}


def _by_name(values: Mapping, name_of: Callable[[Tensor], Optional[str]]) -> dict[str, Tensor]:
    out: dict[str, Tensor] = {}
    for k, v in values.items():
        if isinstance(k, str):
            out[k] = v
        elif isinstance(k, Tensor):
            n = name_of(k)
            if n is None:
                raise KeyError("tensor-keyed scarcity mappings require bind_param_names()")
            out[n] = v
        else:
            raise TypeError("scarcity mappings must be keyed by parameter name or Tensor")
    return out


class ScarcityAwareOptimizer(torch.optim.Optimizer):
    def __init__(self, params: Iterable[Tensor] | Iterable[dict[str, Any]], *, lr: float = 0.02, momentum: float = 0.95,
                 nesterov: bool = True, ns_steps: int = 5, weight_decay: float = 0.0,
                 adamw_betas: tuple[float, float] = (0.9, 0.95), adamw_eps: float = 1e-8,
                 adamw_lr: Optional[float] = None, adamw_weight_decay: Optional[float] = None,
                 matrix_param_names: Optional[set[str]] = None,
                 is_matrix: Optional[Callable[[Tensor, Optional[str]], bool]] = None,
                 compute_dtype: Optional[torch.dtype] = None, rare_ema_decay: float = 0.9,
                 rare_orthogonal_weight: float = 1.0, rare_macro_c: float = 0.5, warmup_steps: int = 200,
                 row_param_names: Optional[set[str]] = None, row_scarcity_power: float = 0.5,
                 matrix_scarcity_map: Optional[Mapping[str, tuple[Optional[str], Optional[str]]]] = None,
                 recurrence_scarcity_map: Optional[Mapping[str, str]] = None,
                 recurrence_timescale: Optional[Mapping[str, Tensor]] = None, recurrence_weight: float = 1.0,
                 tau_std_scale: float = 0.5, tau_out_floor: float = 1e-4, tau_in_floor: float = 1e-4,
                 tau_row_floor: float = 1e-4, eps: float = 1e-8) -> None:
        if lr <= 0.0 or ns_steps <= 0 or not 0.0 <= momentum < 1.0:
            raise ValueError(f"invalid ScOpt hparams: lr={lr} momentum={momentum} ns_steps={ns_steps}")
        if not 0.0 <= rare_ema_decay < 1.0:
            raise ValueError(f"rare_ema_decay must be in [0, 1), got {rare_ema_decay}")
        if rare_macro_c < 0.0:
            raise ValueError(f"rare_macro_c must be >= 0, got {rare_macro_c}")
        super().__init__(params, dict(
            lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps, weight_decay=weight_decay,
            adamw_betas=adamw_betas, adamw_eps=adamw_eps, adamw_lr=lr if adamw_lr is None else adamw_lr,
            adamw_weight_decay=weight_decay if adamw_weight_decay is None else adamw_weight_decay))
        self._matrix_param_names = None if matrix_param_names is None else set(matrix_param_names)
        self._is_matrix_fn = is_matrix or (lambda p, _n: p.ndim == 2)
        self._compute_dtype = compute_dtype
        self._rare_ema_decay, self._rare_orthogonal_weight = float(rare_ema_decay), float(rare_orthogonal_weight)
        self._rare_macro_c, self._warmup_steps = float(rare_macro_c), int(warmup_steps)
        self._row_param_names = set(row_param_names or {"embed.weight", "lm_head.weight"})
        self._row_scarcity_power = float(row_scarcity_power)
        self._matrix_scarcity_map = dict(matrix_scarcity_map or {})
        self._recurrence_scarcity_map = dict(recurrence_scarcity_map or {})
        self._recurrence_timescale = dict(recurrence_timescale or {})
        self._recurrence_weight, self._tau_std_scale = float(recurrence_weight), float(tau_std_scale)
        self._tau_out_floor, self._tau_in_floor, self._tau_row_floor = map(float, (tau_out_floor, tau_in_floor,
                                                                                  tau_row_floor))
        self._eps = float(eps)
        self._param_name_by_id: dict[int, str] = {}
        self._row_pressure_ema: Optional[Tensor] = None
        self._channel_pressure: dict[str, Tensor] = {}
        self._step_count = 0
        self._telemetry: dict[str, list] = defaultdict(list)
        self._pressure_stats: Optional[dict[str, float]] = None
        self._clip_events = self._clip_observations = 0

    # ------------------------------------------------------------------ wiring / gates
    def bind_param_names(self, named_params: Iterable[tuple[str, Tensor]]) -> None:
        self._param_name_by_id = {id(p): n for n, p in named_params}

    def _name_of(self, p: Tensor) -> Optional[str]:
        return self._param_name_by_id.get(id(p))

    def _is_matrix_param(self, p: Tensor) -> bool:
        n = self._name_of(p)
        if self._matrix_param_names is not None and n is not None:
            return n in self._matrix_param_names
        return self._is_matrix_fn(p, n)

    def _scarcity_enabled(self) -> bool:
        return self._step_count > self._warmup_steps

    def _writes_enabled(self) -> bool:
        """State writes happen before ``step()`` increments the counter: they open one step
        before reads do, so the EMAs hold one warm entry when scarcity switches on."""
        return self._step_count >= self._warmup_steps

    def _log(self, key: str, value) -> None:
        self._telemetry[key].append(value.detach() if isinstance(value, Tensor) else float(value))

    # ------------------------------------------------------------------ state feeds
    def set_rare_grad_ema(self, rare_grads: Mapping) -> None:
        m = _by_name(rare_grads, self._name_of)
        for g in self.param_groups:
            for p in g["params"]:
                n = self._name_of(p)
                if n in m:
                    self.state[p]["rare_grad_ema"] = m[n].detach().to(device=p.device, dtype=p.dtype).clone()

    def update_rare_grad_ema(self, rare_grads: Mapping, *, skip: bool = False) -> None:
        if skip or not self._writes_enabled():
            return
        m = _by_name(rare_grads, self._name_of)
        d = self._rare_ema_decay
        for g in self.param_groups:
            for p in g["params"]:
                n = self._name_of(p)
                if n not in m:
                    continue
                st = self.state[p]
                if "rare_grad_ema" not in st:
                    st["rare_grad_ema"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["rare_grad_ema"].mul_(d).add_(m[n].detach().to(device=p.device, dtype=p.dtype), alpha=1.0 - d)

    def set_row_pressure_ema(self, row_pressure: Optional[Tensor]) -> None:
        if self._writes_enabled():
            self._row_pressure_ema = None if row_pressure is None else row_pressure.detach().float().clone()

    def update_row_pressure_ema(self, targets: Tensor, pressure: Tensor, *, vocab_size: int,
                                decay: Optional[float] = None) -> Optional[Tensor]:
        """Mean pressure per target row folded into a per-vocabulary-row EMA (rows not hit keep their value)."""
        if not self._writes_enabled():
            return None
        if targets.shape != pressure.shape:
            raise ValueError(f"targets and pressure must match, got {tuple(targets.shape)} and {tuple(pressure.shape)}")
        V = int(vocab_size)
        if self._row_pressure_ema is None:
            self._row_pressure_ema = torch.zeros(V, dtype=torch.float32, device=pressure.device)
        elif self._row_pressure_ema.numel() != V:
            raise ValueError(f"existing row pressure has {self._row_pressure_ema.numel()} rows, got vocab_size={V}")
        cur = self._row_pressure_ema.to(pressure.device)
        t = targets.reshape(-1).to(pressure.device)
        pf = pressure.detach().float().reshape(-1)
        s = torch.zeros_like(cur).index_add_(0, t, pf)
        c = torch.zeros_like(cur).index_add_(0, t, torch.ones_like(pf))
        d = self._rare_ema_decay if decay is None else float(decay)
        self._row_pressure_ema = torch.where(c > 0, cur * d + (s / c.clamp_min(1.0)) * (1.0 - d), cur).detach()
        return self._row_pressure_ema

    def set_channel_pressure(self, channel_pressure: Mapping[str, Tensor]) -> None:
        if self._writes_enabled():
            self._channel_pressure = {k: v.detach().float().clone() for k, v in channel_pressure.items()}

    def set_recurrence_timescale(self, recurrence_timescale: Mapping[str, Tensor]) -> None:
        self._recurrence_timescale = {k: v.detach().float().clone() for k, v in recurrence_timescale.items()}

    # ------------------------------------------------------------------ geometry
    def _scarcity_factor(self, pressure: Tensor, *, floor: float, device, dtype, telemetry_key: Optional[str] = None):
        """``1 + tanh(p / tau)`` with ``tau = max(tau_std_scale * std(p), floor)``: in [1, 2)."""
        pf = pressure.detach().to(device=device, dtype=torch.float32).clamp_min(0.0)
        if pf.numel() == 0:
            return pf.to(dtype)
        tau = torch.clamp(pf.std(unbiased=False) * self._tau_std_scale, min=float(floor))
        f = torch.tanh(pf / tau.clamp_min(self._eps)) + 1.0
        if telemetry_key is not None:
            self._log(f"{telemetry_key}_min", f.min())
            self._log(f"{telemetry_key}_median", f.median())
            self._log(f"{telemetry_key}_max", f.max())
        return f.to(dtype)

    def _rare_adjusted_direction(self, *, p: Tensor, common: Tensor) -> Tensor:
        if not self._scarcity_enabled():
            return common
        rare = self.state[p].get("rare_grad_ema")
        if rare is None:
            return common
        c = common.float()
        r = rare.to(device=common.device, dtype=torch.float32)
        c_sq = c.square().sum().clamp_min(self._eps)
        dot = (r * c).sum()
        orth = r - (dot / c_sq) * c
        c_norm, r_norm = c_sq.sqrt(), r.square().sum().clamp_min(self._eps).sqrt()
        o_norm = orth.square().sum().clamp_min(0.0).sqrt()
        self._log("cos_rare_common", (dot / (r_norm * c_norm)).clamp(-1.0, 1.0))
        self._log("r_orth_over_common", o_norm / c_norm)
        w = self._rare_orthogonal_weight
        if self._rare_macro_c > 0.0 and w > 0.0:
            eff = torch.clamp(self._rare_macro_c * c_norm / o_norm.clamp_min(self._eps), max=w)
            self._log("rare_macro_effective_weight", eff)
            self._log("rare_macro_cap_fired", (eff < w - 1e-6).float())
            return (c + eff * orth).to(common.dtype)
        return (c + w * orth).to(common.dtype)

    def _apply_matrix_scarcity(self, name: Optional[str], direction: Tensor):
        if not self._scarcity_enabled() or name is None:
            return direction, None, None
        out_key, in_key = self._matrix_scarcity_map.get(name, (None, None))
        out_f = in_f = None
        if out_key is not None and out_key in self._channel_pressure:
            out_f = self._scarcity_factor(self._channel_pressure[out_key], floor=self._tau_out_floor,
                                          device=direction.device, dtype=direction.dtype, telemetry_key="out_scarcity")
            if out_f.numel() != direction.size(0):
                raise ValueError(f"out scarcity {out_key!r} has {out_f.numel()} channels for {name!r} "
                                 f"rows={direction.size(0)}")
            direction = out_f.sqrt()[:, None] * direction
        if in_key is not None and in_key in self._channel_pressure:
            in_f = self._scarcity_factor(self._channel_pressure[in_key], floor=self._tau_in_floor,
                                         device=direction.device, dtype=direction.dtype, telemetry_key="in_scarcity")
            if in_f.numel() != direction.size(1):
                raise ValueError(f"in scarcity {in_key!r} has {in_f.numel()} channels for {name!r} "
                                 f"cols={direction.size(1)}")
            direction = direction * in_f.sqrt()[None, :]
        return direction, out_f, in_f

    def _apply_row_scarcity(self, name: Optional[str], direction: Tensor):
        if (not self._scarcity_enabled() or name is None or name not in self._row_param_names
                or self._row_pressure_ema is None):
            return direction, None
        if self._row_pressure_ema.numel() != direction.size(0):
            raise ValueError(f"row pressure has {self._row_pressure_ema.numel()} rows for {name!r} "
                             f"rows={direction.size(0)}")
        f = self._scarcity_factor(self._row_pressure_ema, floor=self._tau_row_floor, device=direction.device,
                                  dtype=direction.dtype, telemetry_key="row_scarcity").pow(self._row_scarcity_power)
        return f[:, None] * direction, f

    def _apply_recurrence_scarcity(self, name: Optional[str], direction: Tensor) -> Tensor:
        if not self._scarcity_enabled() or name is None:
            return direction
        key = self._recurrence_scarcity_map.get(name)
        if key is None or key not in self._channel_pressure:
            return direction
        f = self._scarcity_factor(self._channel_pressure[key], floor=self._tau_out_floor, device=direction.device,
                                  dtype=direction.dtype, telemetry_key="recurrence_scarcity")
        ts = self._recurrence_timescale.get(key)
        if ts is not None:
            ts = ts.to(device=direction.device, dtype=direction.dtype)
            if ts.numel() != f.numel():
                raise ValueError(f"recurrence timescale {key!r} has {ts.numel()} channels but pressure has {f.numel()}")
            f = 1.0 + self._recurrence_weight * (f - 1.0) * ts
        if f.shape != direction.shape:
            raise ValueError(f"recurrence scarcity for {name!r} has shape {tuple(f.shape)} but direction has shape "
                             f"{tuple(direction.shape)}; broadcast is not supported")
        return direction * f

    def _enrichment(self, energy: Tensor, factor: Tensor, key: str) -> None:
        """Does the pre-orthogonalisation scaling survive it?  Ratio of mean update energy
        on scarce (factor >= median) vs common rows / columns, and the log-space correlation
        between factor and resulting norm."""
        scarce = factor >= factor.median()
        ns, nc = scarce.sum(), (~scarce).sum()
        ratio = (energy[scarce].sum() / ns.clamp_min(1)) / (energy[~scarce].sum() / nc.clamp_min(1)).clamp_min(self._eps)
        self._log(f"ns_{key}_energy_enrichment", torch.where((ns > 0) & (nc > 0), ratio, ratio.new_tensor(float("nan"))))
        lf, ln = factor.clamp_min(self._eps).log(), energy.clamp_min(self._eps).log() * 0.5
        sf, sn = lf.std(unbiased=False), ln.std(unbiased=False)
        corr = ((lf - lf.mean()) * (ln - ln.mean())).mean() / (sf * sn).clamp_min(self._eps)
        self._log(f"ns_{key}_factor_corr", torch.where((sf > self._eps) & (sn > self._eps), corr.clamp(-1.0, 1.0),
                                                       corr.new_tensor(float("nan"))))

    def _record_energy_enrichment(self, update: Tensor, *, row_factor: Optional[Tensor], col_factor: Optional[Tensor]):
        if update.ndim != 2:
            return
        u = update.detach().float()
        sq = u.square()
        tot = sq.sum().clamp_min(self._eps)
        if row_factor is not None and row_factor.numel() == update.size(0):
            self._enrichment(sq.sum(1) / tot, row_factor.detach().to(device=u.device, dtype=torch.float32), "row")
        if col_factor is not None and col_factor.numel() == update.size(1):
            self._enrichment(sq.sum(0) / tot, col_factor.detach().to(device=u.device, dtype=torch.float32), "col")

    # ------------------------------------------------------------------ diagnostics
    def record_pressure_stats(self, stats: Mapping[str, float]) -> None:
        self._pressure_stats = dict(stats)

    def record_clip_event(self, *, triggered: bool) -> None:
        self._clip_observations += 1
        self._clip_events += int(bool(triggered))

    def scarcity_trace(self) -> dict[str, Any]:
        """Window summary since the previous call (min / median / max / count per telemetry key)."""
        trace: dict[str, Any] = {"step": self._step_count, "scarcity_enabled": self._scarcity_enabled()}
        if self._row_pressure_ema is not None:
            row = self._row_pressure_ema.detach().float().cpu()
            trace["row_pressure"] = {"min": float(row.min()), "median": float(row.median()), "max": float(row.max())}
        if self._channel_pressure:
            trace["channel_pressure_keys"] = sorted(self._channel_pressure)
        if self._pressure_stats is not None:
            trace["pressure_stats"] = dict(self._pressure_stats)
        for key, vals in self._telemetry.items():
            t = torch.stack([v.detach().float().cpu().reshape(()) if isinstance(v, Tensor) else torch.tensor(float(v))
                             for v in vals])
            t = t[torch.isfinite(t)]
            if t.numel():
                trace[key] = {"min": float(t.min()), "median": float(t.median()), "max": float(t.max()),
                              "count": int(t.numel())}
        if self._clip_observations > 0:
            trace["clip_rate"] = self._clip_events / self._clip_observations
        self._telemetry = defaultdict(list)
        self._clip_events = self._clip_observations = 0
        return trace

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], Tensor]] = None) -> Optional[Tensor]:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step_count += 1
        for group in self.param_groups:
            lr, mu, nesterov, wd = group["lr"], group["momentum"], group["nesterov"], group["weight_decay"]
            b1, b2 = group["adamw_betas"]
            batches: dict[tuple, list] = defaultdict(list)
            for p in group["params"]:
                if p.grad is None:
                    continue
                g, st, name = p.grad, self.state[p], self._name_of(p)
                if self._is_matrix_param(p):
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    buf = st["momentum_buffer"]
                    buf.mul_(mu).add_(g)
                    d = self._rare_adjusted_direction(p=p, common=g.add(buf, alpha=mu) if nesterov else buf)
                    d, out_f, in_f = self._apply_matrix_scarcity(name, d)
                    d, row_f = self._apply_row_scarcity(name, d)
                    batches[(p.shape[-2], p.shape[-1], d.dtype, d.device)].append(
                        (p, d.contiguous(), row_f if row_f is not None else out_f, in_f))
                    continue
                adj = self._apply_recurrence_scarcity(name, self._rare_adjusted_direction(p=p, common=g))
                if "step" not in st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                t = st["step"]
                st["exp_avg"].mul_(b1).add_(adj, alpha=1.0 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(adj, adj, value=1.0 - b2)
                denom = (st["exp_avg_sq"].sqrt() / ((1.0 - b2 ** t) ** 0.5)).add_(group["adamw_eps"])
                if group["adamw_weight_decay"] > 0.0:
                    p.data.mul_(1.0 - group["adamw_lr"] * group["adamw_weight_decay"])
                p.data.addcdiv_(st["exp_avg"], denom, value=-group["adamw_lr"] / (1.0 - b1 ** t))
            for (rows, cols, _dt, _dev), items in batches.items():
                upd = newton_schulz_orthogonalize(torch.stack([d for _, d, _, _ in items], 0), steps=group["ns_steps"],
                                                  compute_dtype=self._compute_dtype)
                scale = max(1.0, rows / cols) ** 0.5
                for i, (p, _d, row_f, col_f) in enumerate(items):
                    if row_f is not None or col_f is not None:
                        self._record_energy_enrichment(upd[i], row_factor=row_f, col_factor=col_f)
                    if wd > 0.0:
                        p.data.mul_(1.0 - lr * wd)
                    p.data.add_(upd[i].to(p.dtype), alpha=-lr * scale)
        return loss
