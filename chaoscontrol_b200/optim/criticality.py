"""Criticality distillation: score SSM channels by how long their state keeps
energy after high-pressure events, give the best ``criticality_budget_frac`` of
them per layer a "seat", and pull the seated channels' ``1 - sigmoid(log_a)``
toward ``critical_value`` with a seat-masked MSE
(behaviour and buffer names of src/chaoscontrol/optim/criticality.py:15-738).

Evidence per step and layer = mean over event positions of
``max(future_energy - baseline, 0)`` where ``future_energy[t]`` is the mean
squared state over ``(t, t + H]`` and ``baseline`` an EMA over non-event
positions.  Evidence is kept in a TTL ring (for checkpoints and exact
re-scoring) and folded into running accumulators that decay with a half-life
(the hot-path scorer).

All layers are processed together: states are stacked ``[L, B, T, D]`` for the
device-side aggregation, and ring-slot choice, accumulator updates and seat
selection are batched over the layer axis instead of looping over layers.
"""
from __future__ import annotations

import torch
import torch.nn as nn

__all__ = ["CriticalityDistillation", "compute_event_mask", "compute_future_energy"]


def compute_event_mask(pressure: torch.Tensor, event_frac: float) -> torch.Tensor:
    """True at the top ``event_frac`` positions of ``pressure``, positive ones only."""
    if not 0.0 <= event_frac <= 1.0:
        raise ValueError(f"event_frac must be in [0, 1]; got {event_frac}")
    n = pressure.numel()
    k = int(round(event_frac * n))
    out = torch.zeros(n, dtype=torch.bool, device=pressure.device)
    if k > 0:
        flat = pressure.reshape(-1)
        k = min(k, int((flat > 0).sum()))
        if k > 0:
            out[torch.topk(flat, k=k, largest=True).indices] = True
    return out.reshape(pressure.shape) & (pressure > 0)


def compute_future_energy(states: torch.Tensor, horizon_H: int) -> torch.Tensor:
    """``[..., T, D]`` -> mean of ``states**2`` over ``(t, min(t + H, T - 1)]``; 0 where the
    window is empty.  One cumulative sum, no loop over time."""
    if horizon_H < 1:
        raise ValueError(f"horizon_H must be >= 1; got {horizon_H}")
    T = states.shape[-2]
    cs = torch.nn.functional.pad(states.pow(2).cumsum(dim=-2), (0, 0, 1, 0))        # [..., T+1, D]
    t = torch.arange(T, device=states.device)
    lo, hi = t + 1, torch.clamp(t + 1 + horizon_H, max=T)
    n = (hi - lo).clamp_min(0)
    win = cs.index_select(-2, torch.where(n > 0, hi, lo * 0)) - cs.index_select(-2, torch.where(n > 0, lo, lo * 0))
    return win / n.clamp_min(1).to(win.dtype).unsqueeze(-1) * (n > 0).to(win.dtype).unsqueeze(-1)


class CriticalityDistillation(nn.Module):
    def __init__(self, *, num_layers: int, dim: int, trace_ttl_steps: int = 1024, trace_half_life_steps: float = 256.0,
                 seat_refresh_interval: int = 64, criticality_budget_frac: float = 0.15, critical_value: float = 0.95,
                 min_weighted_events_per_layer: float = 256.0, criticality_distill_weight: float = 1e-3,
                 baseline_ema_decay: float = 0.99, score_permute_before_topk: bool = False,
                 fixed_random_seats: bool = False) -> None:
        super().__init__()
        if not 0.0 < criticality_budget_frac < 1.0:
            raise ValueError(f"criticality_budget_frac must be in (0, 1); got {criticality_budget_frac}")
        if not 0.0 < critical_value < 1.0:
            raise ValueError(f"critical_value must be in (0, 1); got {critical_value}")
        self.num_layers, self.dim = int(num_layers), int(dim)
        self.trace_ttl_steps, self.trace_half_life_steps = int(trace_ttl_steps), float(trace_half_life_steps)
        self.seat_refresh_interval = int(seat_refresh_interval)
        self.criticality_budget_frac, self.critical_value = float(criticality_budget_frac), float(critical_value)
        self.min_weighted_events_per_layer = float(min_weighted_events_per_layer)
        self.criticality_distill_weight = float(criticality_distill_weight)
        self.baseline_ema_decay = float(baseline_ema_decay)
        self.score_permute_before_topk, self.fixed_random_seats = bool(score_permute_before_topk), bool(fixed_random_seats)
        L, Tt, D = self.num_layers, self.trace_ttl_steps, self.dim
        self.register_buffer("bank_evidence", torch.zeros(L, Tt, D))
        self.register_buffer("bank_step", torch.full((L, Tt), -1, dtype=torch.int64))
        self.register_buffer("bank_event_count", torch.zeros(L, Tt))
        self.register_buffer("baseline_future_energy", torch.zeros(L, D))
        self.register_buffer("baseline_initialized", torch.zeros(L, dtype=torch.bool))
        self.register_buffer("seat_mask", torch.zeros(L, D, dtype=torch.bool))
        self.register_buffer("score_num", torch.zeros(L, D))
        self.register_buffer("score_den", torch.zeros(L))
        self.register_buffer("event_mass", torch.zeros(L))
        self.register_buffer("last_decay_step", torch.tensor(-1, dtype=torch.int64))
        if self.fixed_random_seats:
            for layer in range(L):
                self.seat_mask[layer, torch.randperm(D)[: self._k]] = True
        self._previous_seat_mask_snapshot: torch.Tensor | None = None

    @property
    def _k(self) -> int:
        return max(1, int(round(self.dim * self.criticality_budget_frac)))

    def _check_layer(self, layer: int) -> None:
        if not 0 <= layer < self.num_layers:
            raise IndexError(f"layer={layer} out of range for num_layers={self.num_layers}")

    def _check_evidence(self, evidence: torch.Tensor) -> None:
        if evidence.shape != (self.dim,):
            raise ValueError(f"evidence must have shape ({self.dim},); got {tuple(evidence.shape)}")

    # ------------------------------------------------------------------ ring bank
    def _pick_slots(self, layers: torch.Tensor) -> torch.Tensor:
        """Per layer: the first empty slot, else the slot holding the oldest step."""
        steps = self.bank_step[layers]
        idx = torch.arange(self.trace_ttl_steps, device=steps.device)
        key = torch.where(steps < 0, idx - (1 << 62), steps)
        return key.argmin(dim=1)

    def add_step_evidence(self, *, layer: int, step: int, evidence: torch.Tensor, event_count: float) -> None:
        """Writes one evidence vector into the ring (no accumulator update)."""
        self._check_layer(layer)
        self._check_evidence(evidence)
        slot = int(self._pick_slots(torch.tensor([layer], device=self.bank_step.device))[0])
        self.bank_evidence[layer, slot] = evidence.to(self.bank_evidence)
        self.bank_step[layer, slot] = int(step)
        self.bank_event_count[layer, slot] = float(event_count)

    def _age_weights(self, current_step: int) -> torch.Tensor:
        age = (int(current_step) - self.bank_step).clamp_min(0).float()
        return torch.exp2(-age / self.trace_half_life_steps) * (self.bank_step >= 0).float()

    def score(self, current_step: int) -> torch.Tensor:
        """``[L, D]``: mean of banked evidence weighted by ``2^(-age / half_life) * event_count``."""
        w = self._age_weights(current_step) * self.bank_event_count
        tot = w.sum(dim=1, keepdim=True)
        s = torch.einsum("lt,ltd->ld", w, self.bank_evidence) / tot.clamp_min(1e-12)
        return torch.where(tot > 0, s, torch.zeros_like(s))

    def score_from_accumulators(self) -> torch.Tensor:
        raw = self.score_num / self.score_den.clamp_min(1e-12).unsqueeze(-1)
        return torch.where((self.event_mass > 0).unsqueeze(-1), raw, torch.zeros_like(raw))

    # ------------------------------------------------------------------ baseline / accumulators
    @torch.no_grad()
    def update_baseline_ema(self, *, layer: int, future_energy: torch.Tensor, event_mask: torch.Tensor) -> None:
        self._check_layer(layer)
        if future_energy.shape[-1] != self.dim:
            raise ValueError(f"future_energy last dim must be {self.dim}; got {tuple(future_energy.shape)}")
        quiet = ~event_mask.reshape(-1)
        if not quiet.any():
            return
        obs = future_energy.reshape(-1, self.dim)[quiet].mean(dim=0).to(self.baseline_future_energy.dtype)
        self._fold_baseline(torch.tensor([layer]), obs.unsqueeze(0))

    def _fold_baseline(self, layers: torch.Tensor, obs: torch.Tensor) -> None:
        layers = layers.to(self.baseline_future_energy.device)
        init = self.baseline_initialized[layers].unsqueeze(-1)
        cur = self.baseline_future_energy[layers]
        d = self.baseline_ema_decay
        self.baseline_future_energy[layers] = torch.where(init, cur * d + obs * (1.0 - d), obs)
        self.baseline_initialized[layers] = True

    @torch.no_grad()
    def _step_decay_accumulators(self, current_step: int) -> None:
        """Ages the accumulators from ``last_decay_step`` to ``current_step`` (idempotent per step)."""
        last = int(self.last_decay_step)
        if int(current_step) <= last:
            return
        if last >= 0:
            f = 2.0 ** (-(int(current_step) - last) / self.trace_half_life_steps)
            self.score_num.mul_(f)
            self.score_den.mul_(f)
            self.event_mass.mul_(f)
        self.last_decay_step.fill_(int(current_step))

    @torch.no_grad()
    def _add_contribution(self, *, layer: int, evidence: torch.Tensor, event_count: float) -> None:
        self._check_layer(layer)
        self._check_evidence(evidence)
        self.score_num[layer].add_(evidence.to(self.score_num), alpha=float(event_count))
        self.score_den[layer].add_(float(event_count))
        self.event_mass[layer].add_(float(event_count))

    @torch.no_grad()
    def _subtract_expired_contribution(self, *, layer: int, evicted_step: int, current_step: int,
                                       evicted_evidence: torch.Tensor, evicted_event_count: float) -> None:
        rem = float(evicted_event_count) * 2.0 ** (-max(0, int(current_step) - int(evicted_step)) /
                                                   self.trace_half_life_steps)
        self.score_num[layer].sub_(evicted_evidence.to(self.score_num), alpha=rem)
        self.score_den[layer].sub_(rem)
        self.event_mass[layer].sub_(rem)

    @torch.no_grad()
    def _write_ring_slot(self, *, layer: int, step: int, evidence: torch.Tensor, event_count: float,
                         current_step: int) -> None:
        self._ingest_rows(torch.tensor([layer]), evidence.unsqueeze(0), torch.tensor([float(event_count)]), step,
                          add=False)

    @torch.no_grad()
    def _ingest_rows(self, layers: torch.Tensor, evidence: torch.Tensor, counts: torch.Tensor, step: int,
                     add: bool = True) -> None:
        """Batched over ``layers``: evict (subtracting what the evicted entry still weighs),
        write the ring slot, and optionally add the new contribution at weight 1."""
        dev = self.bank_step.device
        layers, counts = layers.to(dev), counts.to(device=dev, dtype=torch.float32)
        ev = evidence.to(device=dev, dtype=torch.float32)
        slots = self._pick_slots(layers)
        old_step = self.bank_step[layers, slots]
        occupied = old_step >= 0
        rem = torch.where(occupied, self.bank_event_count[layers, slots] *
                          torch.exp2(-(int(step) - old_step).clamp_min(0).float() / self.trace_half_life_steps),
                          torch.zeros_like(counts))
        new_mass = counts if add else torch.zeros_like(counts)
        self.score_num.index_add_(0, layers, ev * new_mass.unsqueeze(-1) - self.bank_evidence[layers, slots] * rem.unsqueeze(-1))
        self.score_den.index_add_(0, layers, new_mass - rem)
        self.event_mass.index_add_(0, layers, new_mass - rem)
        self.bank_evidence[layers, slots] = ev
        self.bank_step[layers, slots] = int(step)
        self.bank_event_count[layers, slots] = counts

    # ------------------------------------------------------------------ ingestion
    @torch.no_grad()
    def ingest_gpu(self, *, pressure: torch.Tensor, states_per_layer: list, horizon_H: int, event_frac: float) -> dict:
        """Device-side phase: returns only ``[L, D]`` / ``[L]`` aggregates and two scalars, so the
        transfer to wherever the bookkeeping lives stays tiny."""
        if len(states_per_layer) != self.num_layers:
            raise ValueError(f"states_per_layer must have {self.num_layers} entries; got {len(states_per_layer)}")
        for i, s in enumerate(states_per_layer):
            if s.shape[-1] != self.dim:
                raise ValueError(f"layer {i}: states last dim {s.shape[-1]} != self.dim {self.dim}")
        ev = compute_event_mask(pressure, event_frac=event_frac).reshape(-1)
        n_ev, n_quiet = ev.sum(), (~ev).sum()
        fe = compute_future_energy(torch.stack([s.float() for s in states_per_layer], 0), horizon_H)   # [L,B,T,D]
        fe = fe.reshape(self.num_layers, -1, self.dim)
        evf, qf = ev.to(fe.dtype), (~ev).to(fe.dtype)
        quiet_mean = torch.einsum("lnd,n->ld", fe, qf) / n_quiet.clamp_min(1)
        excess = (fe - self.baseline_future_energy.to(fe.device).unsqueeze(1)).clamp_min(0.0)
        agg = torch.einsum("lnd,n->ld", excess, evf) / n_ev.clamp_min(1)
        return {"aggregated_excess_per_layer": agg, "non_event_mean_future_energy_per_layer": quiet_mean,
                "event_count_per_layer": n_ev.float().expand(self.num_layers).clone(),
                "n_events_scalar": n_ev.to(torch.int64), "n_non_events_scalar": n_quiet.to(torch.int64)}

    @torch.no_grad()
    def ingest_cpu_from_prepared(self, *, step: int, prepared: dict) -> None:
        dev = self.bank_evidence.device
        agg = prepared["aggregated_excess_per_layer"].to(device=dev, dtype=torch.float32)
        counts = prepared["event_count_per_layer"].to(device=dev, dtype=torch.float32)
        self._step_decay_accumulators(current_step=step)
        if int(prepared["n_non_events_scalar"]) > 0:
            self._fold_baseline(torch.arange(self.num_layers),
                                prepared["non_event_mean_future_energy_per_layer"].to(device=dev, dtype=torch.float32))
        live = (counts > 0).nonzero(as_tuple=True)[0]
        if live.numel():
            self._ingest_rows(live, agg[live], counts[live], step, add=True)

    @torch.no_grad()
    def ingest_step(self, *, step: int, pressure: torch.Tensor, states_per_layer: list, horizon_H: int,
                    event_frac: float) -> None:
        self.ingest_cpu_from_prepared(step=step, prepared=self.ingest_gpu(
            pressure=pressure, states_per_layer=states_per_layer, horizon_H=horizon_H, event_frac=event_frac))

    # ------------------------------------------------------------------ seats
    def _seat(self, scores: torch.Tensor, mass: torch.Tensor) -> None:
        k, dev = self._k, self.seat_mask.device
        if self.score_permute_before_topk:
            idx = torch.stack([torch.randperm(self.dim, device=dev)[:k] for _ in range(self.num_layers)], 0)
        else:
            idx = torch.topk(scores, k=k, dim=1, largest=True).indices
        mask = torch.zeros_like(self.seat_mask).scatter_(1, idx, True)
        self.seat_mask.copy_(mask & (mass >= self.min_weighted_events_per_layer).unsqueeze(-1))

    @torch.no_grad()
    def allocate_seats(self, *, current_step: int) -> None:
        """Exact (bank-rescored) allocation; a layer below the weighted-event floor gets no seats."""
        if self.fixed_random_seats:
            return
        self._seat(self.score(current_step), (self._age_weights(current_step) * self.bank_event_count).sum(dim=1))

    @torch.no_grad()
    def allocate_seats_from_accumulators(self, *, current_step: int) -> None:
        if self.fixed_random_seats:
            return
        self._step_decay_accumulators(current_step=current_step)
        self._seat(self.score_from_accumulators(), self.event_mass)

    # ------------------------------------------------------------------ loss / diagnostics
    def criticality_loss(self, log_a_per_layer: list) -> torch.Tensor:
        """``weight * sum over seated layers of mean_seats (1 - sigmoid(log_a) - critical_value)^2``;
        unseated channels get exactly zero gradient."""
        if len(log_a_per_layer) != self.num_layers:
            raise ValueError(f"log_a_per_layer must have {self.num_layers} entries")
        crit = 1.0 - torch.sigmoid(torch.stack([la.float() for la in log_a_per_layer], 0))
        m = self.seat_mask.to(crit.device).float()
        per_layer = ((crit - self.critical_value) ** 2 * m).sum(dim=1) / m.sum(dim=1).clamp_min(1.0)
        return per_layer.sum() * self.criticality_distill_weight

    @torch.no_grad()
    def diagnostics_snapshot(self, *, log_a_per_layer: list, current_step: int) -> dict:
        """Seat churn since the previous snapshot, occupancy (seated channels already near the
        target), rank correlation of score vs criticality, event rate, seat fraction and indices,
        and score quantiles, per layer."""
        if len(log_a_per_layer) != self.num_layers:
            raise ValueError(f"log_a_per_layer must have {self.num_layers} entries; got {len(log_a_per_layer)}")
        scores = self.score_from_accumulators().float()
        crit = 1.0 - torch.sigmoid(torch.stack([la.detach().float() for la in log_a_per_layer], 0)).to(scores.device)
        cur = self.seat_mask
        k = cur.sum(dim=1)
        if self._previous_seat_mask_snapshot is None:
            churn = torch.zeros(self.num_layers)
        else:
            churn = (self._previous_seat_mask_snapshot != cur).sum(dim=1).float() / (2.0 * k.clamp_min(1).float())
        near = (crit >= 0.9 * self.critical_value) & cur
        occ = torch.where(k > 0, near.sum(dim=1).float() / k.clamp_min(1).float(), torch.zeros(self.num_layers, device=k.device))

        def _ranks(x):
            return torch.argsort(torch.argsort(x, dim=1), dim=1).float()
        rs, rc = _ranks(scores), _ranks(crit)
        rs = (rs - rs.mean(1, keepdim=True)) / rs.std(1, keepdim=True).clamp_min(1e-12)
        rc = (rc - rc.mean(1, keepdim=True)) / rc.std(1, keepdim=True).clamp_min(1e-12)
        flat = (scores.std(dim=1) < 1e-12) | (crit.std(dim=1) < 1e-12)
        corr = torch.where(flat, torch.zeros_like(flat, dtype=torch.float32), (rs * rc).mean(dim=1))
        populated = (self.bank_step != -1).sum(dim=1).clamp_min(1).float()
        q = torch.quantile(scores, torch.tensor([0.10, 0.50, 0.90], device=scores.device), dim=1)
        self._previous_seat_mask_snapshot = cur.clone()
        return {"step": int(current_step), "seat_churn_per_layer": churn.tolist(),
                "budget_occupancy_per_layer": occ.tolist(), "score_criticality_corr_per_layer": corr.tolist(),
                "event_rate_per_layer": (self.event_mass / populated).tolist(),
                "seat_mask_fraction_per_layer": cur.float().mean(dim=1).tolist(),
                "seat_indices_per_layer": [cur[i].nonzero(as_tuple=True)[0].tolist() for i in range(self.num_layers)],
                "score_p10_per_layer": q[0].tolist(), "score_p50_per_layer": q[1].tolist(),
                "score_p90_per_layer": q[2].tolist(), "score_max_per_layer": scores.max(dim=1).values.tolist()}
