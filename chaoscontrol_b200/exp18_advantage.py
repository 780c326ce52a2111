"""Sweep-then-target training (experiment 18, "throughput advantage").

Question of the experiment: a fast model can see the whole corpus once inside the
budget -- does spending the rest of the budget on the windows it found hardest beat
plain training?  Protocol of one run (reference: experiments/18_throughput_advantage/
runner_exp18.py:243-800, bench_throughput.py:57-516):

1. *sweep*: one pass over non-overlapping windows (unique next-token targets are the
   coverage unit) at the large batch, until ``sweep_budget_s``;
2. *rescore*: per-window mean CE under the swept weights, until ``rescore_budget_s``;
3. *select*: the top fraction by loss (or a random subset of the same size: the
   control that separates "selection" from "more steps");
4. *retarget*: train on the subset for whatever is left of the budget.

Every phase is charged to a :class:`PhaseBudget`; selection overhead (rescore +
select) is reported separately because it is the price of the idea.  Tokenizer choice
for the experiment is coverage first, quality second (:func:`choose_tokenizer`).
Scoring uses the fused per-row CE head where the model has one (no logits tensor).
"""
from __future__ import annotations

import math
import random
import time
from dataclasses import dataclass
from typing import Any, Callable, Optional, Sequence

import torch
import torch.nn.functional as F

DEFAULT_SWEEP_BUDGET_S, DEFAULT_RESCORE_BUDGET_S, DEFAULT_SELECTION_BUDGET_S = 400.0, 45.0, 5.0
DEFAULT_TOTAL_BUDGET_S, DEFAULT_BASE_LR, LOW_COVERAGE_FLOOR = 600.0, 2e-3, 0.25


@dataclass
class PhaseBudget:
    total_s: float
    sweep_s: float = 0.0
    rescore_s: float = 0.0
    subset_s: float = 0.0
    retarget_s: float = 0.0

    @property
    def remaining_s(self) -> float:
        return max(0.0, self.total_s - self.sweep_s - self.rescore_s - self.subset_s - self.retarget_s)

    @property
    def selection_overhead_s(self) -> float:
        return self.rescore_s + self.subset_s


@dataclass
class CoveragePlan:
    total_windows: int
    planned_windows: int
    unique_targets: int
    coverage_frac: float
    low_coverage_regime: bool


def generate_sweep_starts(num_tokens: int, seq_len: int, *, max_windows: Optional[int] = None) -> list[int]:
    """Non-overlapping window starts (stride = seq_len); the last start leaves room for its shifted targets."""
    starts = list(range(0, max(num_tokens - seq_len - 1, 0) + (1 if num_tokens > seq_len else 0), seq_len))
    starts = [s for s in starts if s + seq_len + 1 <= num_tokens]
    return starts if max_windows is None else starts[: max(max_windows, 0)]


def count_unique_targets(starts: Sequence[int], seq_len: int) -> int:
    return len(starts) * seq_len


def build_coverage_plan(num_tokens: int, *, seq_len: int, projected_windows: Optional[int] = None) -> CoveragePlan:
    total = len(generate_sweep_starts(num_tokens, seq_len))
    planned = total if projected_windows is None else min(projected_windows, total)
    frac = planned * seq_len / max(total * seq_len, 1)
    return CoveragePlan(total, planned, planned * seq_len, frac, frac < LOW_COVERAGE_FLOOR)


def choose_tokenizer(rows: Sequence[dict[str, Any]]) -> dict[str, Any]:
    """Among stable candidates: the one that covers more of the corpus in the budget (ties by speed); a
    candidate stuck in the low-coverage regime loses to one that is not; within 10 % of coverage the
    larger vocabulary wins when its prior quality is better (or when it is already ahead)."""
    stable = sorted((r for r in rows if r.get("stable")), reverse=True,
                    key=lambda r: (float(r.get("projected_coverage_frac", 0.0)), float(r.get("tokens_per_s", 0.0))))
    if not stable:
        raise ValueError("No stable tokenizer candidates available")
    if len(stable) == 1:
        return stable[0]
    best, nxt = stable[0], stable[1]
    if bool(best.get("low_coverage_regime")) != bool(nxt.get("low_coverage_regime")):
        return nxt if best.get("low_coverage_regime") else best
    cb, cn = float(best.get("projected_coverage_frac", 0.0)), float(nxt.get("projected_coverage_frac", 0.0))
    if (cb - cn) / max(cb, 1e-9) < 0.10 if cb > 0 else True:
        if (float(nxt.get("prior_mean_bpb", math.inf)) < float(best.get("prior_mean_bpb", math.inf))
                and nxt.get("tokenizer") == "sp16384"):
            return nxt
    return best


def select_subset(scored: Sequence[dict[str, float]], *, fraction: float, mode: str, seed: int) -> list[int]:
    if not 0.0 < fraction <= 1.0:
        raise ValueError(f"fraction must be in (0, 1], got {fraction}")
    if not scored:
        return []
    keep = max(1, int(len(scored) * fraction))
    if mode == "top":
        return [int(r["start"]) for r in sorted(scored, key=lambda r: r["loss"], reverse=True)[:keep]]
    if mode == "random":
        pool = list(scored)
        random.Random(seed).shuffle(pool)
        return [int(r["start"]) for r in pool[:keep]]
    raise ValueError(f"Unsupported subset mode: {mode}")


def _batch(tokens: torch.Tensor, starts: Sequence[int], seq_len: int, device: torch.device):
    idx = torch.as_tensor(list(starts), dtype=torch.long)[:, None] + torch.arange(seq_len + 1)[None, :]
    blk = tokens[idx].to(device=device, dtype=torch.long)
    return blk[:, :-1], blk[:, 1:]


@torch.no_grad()
def score_windows_by_loss(model: torch.nn.Module, *, tokens: torch.Tensor, starts: Sequence[int], seq_len: int,
                          batch_size: int, device: torch.device, time_budget_s: Optional[float] = None) -> dict:
    """Mean CE per window under the current weights; stops when the budget is spent (after at least one batch)."""
    if not starts:
        return {"scored": [], "elapsed_s": 0.0, "coverage_scored_frac": 0.0}
    from .scoring import _chunk_loss_rows
    was_training = model.training
    model.eval()
    scored: list[dict[str, float]] = []
    t0 = time.perf_counter()
    for i in range(0, len(starts), batch_size):
        if time_budget_s is not None and scored and time.perf_counter() - t0 >= time_budget_s:
            break
        bs = starts[i: i + batch_size]
        x, y = _batch(tokens, bs, seq_len, device)
        rows, _ = _chunk_loss_rows(model, x, y, None)
        for s, l in zip(bs, rows.float().mean(dim=1).tolist()):
            scored.append({"start": float(s), "loss": float(l)})
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    model.train(was_training)
    return {"scored": scored, "elapsed_s": time.perf_counter() - t0, "coverage_scored_frac": len(scored) / len(starts)}


def build_phase_a_conditions(phase0_summary: dict[str, Any], *, total_budget_s: float = DEFAULT_TOTAL_BUDGET_S) -> dict:
    """The four arms: small-batch baseline, sweep only, sweep + top-10 % retarget, sweep + random-10 % retarget."""
    sel = phase0_summary["selected"]
    cfg, big = dict(sel["model_config"]), int(sel["batch_size"])
    lr = float(sel.get("selected_lr", sel.get("base_lr", DEFAULT_BASE_LR)))
    phases = {"sweep_budget_s": float(sel.get("sweep_budget_s", min(DEFAULT_SWEEP_BUDGET_S, total_budget_s * 0.67))),
              "rescore_budget_s": float(sel.get("rescore_budget_s", min(DEFAULT_RESCORE_BUDGET_S, total_budget_s * 0.08))),
              "selection_budget_s": float(sel.get("selection_budget_s",
                                                  min(DEFAULT_SELECTION_BUDGET_S, total_budget_s * 0.01)))}
    large = dict(cfg, batch_size=big, base_lr=lr)
    target = lambda name, mode: {"condition": name, "model_config": dict(large), "train_mode": "target",    # noqa: E731
                                 "subset_fraction": 0.10, "subset_mode": mode, "total_budget_s": total_budget_s, **phases}
    return {"baseline_b32": {"condition": "baseline_b32", "model_config": dict(cfg, batch_size=32, base_lr=DEFAULT_BASE_LR),
                             "train_mode": "baseline", "total_budget_s": total_budget_s},
            "sweep_only": {"condition": "sweep_only", "model_config": dict(large), "train_mode": "sweep_only",
                           "total_budget_s": total_budget_s, "sweep_budget_s": total_budget_s},
            "sweep_target_top10": target("sweep_target_top10", "top"),
            "sweep_random_retrain": target("sweep_random_retrain", "random")}


def train_on_starts(model: torch.nn.Module, optimizer: torch.optim.Optimizer, *, tokens: torch.Tensor,
                    starts: Sequence[int], seq_len: int, batch_size: int, device: torch.device, budget_s: float,
                    shuffle_seed: Optional[int] = None, epochs: Optional[int] = 1,
                    clock: Callable[[], float] = time.perf_counter) -> dict[str, Any]:
    """Train on the given windows in order (or shuffled per epoch) until the budget or the epochs run out."""
    from .train_ssm import train_ssm_step
    t0, steps, seen, last = clock(), 0, 0, float("nan")
    ep = 0
    while (epochs is None or ep < epochs) and starts:
        order = list(starts)
        if shuffle_seed is not None:
            random.Random(shuffle_seed + ep).shuffle(order)
        for i in range(0, len(order), batch_size):
            if clock() - t0 >= budget_s:
                return {"steps": steps, "windows_seen": seen, "elapsed_s": clock() - t0, "final_loss": last, "epochs": ep}
            x, y = _batch(tokens, order[i: i + batch_size], seq_len, device)
            optimizer.zero_grad(set_to_none=True)
            loss = train_ssm_step(model, x, y, 64, precision="bf16" if device.type == "cuda" else "fp32")
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            optimizer.step()
            steps, seen, last = steps + 1, seen + x.size(0), float(loss)
        ep += 1
    return {"steps": steps, "windows_seen": seen, "elapsed_s": clock() - t0, "final_loss": last, "epochs": ep}


def run_sweep_target(model: torch.nn.Module, optimizer: torch.optim.Optimizer, *, tokens: torch.Tensor, seq_len: int,
                     batch_size: int, device: torch.device, condition: dict[str, Any], seed: int = 0) -> dict[str, Any]:
    """One arm of :func:`build_phase_a_conditions` (``sweep_only`` or a ``target`` arm) end to end."""
    budget = PhaseBudget(total_s=float(condition["total_budget_s"]))
    starts = generate_sweep_starts(int(tokens.numel()), seq_len)
    sweep = train_on_starts(model, optimizer, tokens=tokens, starts=starts, seq_len=seq_len, batch_size=batch_size,
                            device=device, budget_s=float(condition.get("sweep_budget_s", budget.total_s)))
    budget.sweep_s = sweep["elapsed_s"]
    out: dict[str, Any] = {"condition": condition["condition"], "sweep": sweep,
                           "coverage": build_coverage_plan(int(tokens.numel()), seq_len=seq_len,
                                                           projected_windows=sweep["windows_seen"]).__dict__}
    if condition.get("train_mode") == "target":
        sc = score_windows_by_loss(model, tokens=tokens, starts=starts[: max(sweep["windows_seen"], 1)], seq_len=seq_len,
                                   batch_size=batch_size, device=device,
                                   time_budget_s=float(condition.get("rescore_budget_s", DEFAULT_RESCORE_BUDGET_S)))
        budget.rescore_s = sc["elapsed_s"]
        t0 = time.perf_counter()
        subset = select_subset(sc["scored"], fraction=float(condition["subset_fraction"]),
                               mode=str(condition["subset_mode"]), seed=seed)
        budget.subset_s = time.perf_counter() - t0
        re = train_on_starts(model, optimizer, tokens=tokens, starts=subset, seq_len=seq_len, batch_size=batch_size,
                             device=device, budget_s=budget.remaining_s, shuffle_seed=seed, epochs=None)
        budget.retarget_s = re["elapsed_s"]
        out.update(rescore={k: v for k, v in sc.items() if k != "scored"}, subset_size=len(subset), retarget=re)
    out["budget"] = {**budget.__dict__, "remaining_s": budget.remaining_s,
                     "selection_overhead_s": budget.selection_overhead_s}
    return out
