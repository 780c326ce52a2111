"""Does policy-gradient learning on a near-uniform simplex policy move the
weights at all, and does a sharper starting temperature unblock it?
(scripts/simplex_bootstrap_microbench.py:1-308) -- plus the per-arm summary
of learner traces that answers the same question on real runs
(scripts/analyze_step3_v3_diagnostics.py:1-193, here without DuckDB).

The bench drives the native online learner exactly as the episodic runtime
does (record a sampled decision, later deliver its replay outcome) on
synthetic simplices where ONE vertex pays a consistently higher reward.
A policy that learns concentrates probability on that vertex: entropy falls
and the flat weights drift from their start.

``python -m chaoscontrol_b200.episodic.bootstrap_bench [--events 4000]``
"""
from __future__ import annotations

import argparse
import json
import math
from collections import defaultdict
from pathlib import Path
from typing import Any, Optional, Sequence

import numpy as np

from . import native as N

__all__ = ["run_bootstrap", "summarize_trace", "compare_traces", "headline_ratio", "main"]

# per-credit gradient diagnostics the learner writes on every ``credit`` row
GRADIENT_COLUMNS = ("grad_logits_l2", "grad_w_lh_l2", "grad_w_lh_accum_l2", "w_lh_l2")


def _near_uniform_policy(temperature: float, seed: int):
    """Head weights scaled down until max p is a few percent above uniform: the state a
    behaviour-cloned policy was observed in (max p 0.0667 against 0.0625)."""
    pol = N.SimplexPolicy(seed=seed, temperature=temperature)
    n_vp = pol.K_v * pol.H + pol.H
    pol.flat[n_vp:n_vp + pol.H] *= 0.05                      # W_lh
    pol.flat[n_vp + pol.H + 1:] = 0.0                        # W_sb, alpha
    return pol


def run_bootstrap(*, temperature: float = 1.0, events: int = 4000, seed: int = 0, good_vertex: int = 3,
                  reward_gap: float = 1.0, reward_std: float = 0.5, learning_rate: float = 1e-2,
                  sgd_interval: int = 16, entropy_beta: float = 0.0, num_slots: int = 64,
                  report_every: int = 500, trace_path: Optional[Path | str] = None) -> dict[str, Any]:
    rng = np.random.default_rng(seed)
    pol = _near_uniform_policy(temperature, seed)
    start = pol.flat.copy()
    learner = N.SimplexOnlineLearner(num_slots=num_slots, max_entries_per_slot=4, gamma=1.0,
                                     learning_rate=learning_rate, sgd_interval=sgd_interval, ema_interval=64,
                                     gerber_c=0.0, entropy_beta=entropy_beta)
    learner.initialize(pol)
    if trace_path is not None:
        learner.set_trace_path(str(trace_path))
    # one fixed simplex: the policy has to find the paying vertex from rewards alone
    V = rng.standard_normal((pol.N, pol.K_v)).astype(np.float32)
    Vn = V / np.linalg.norm(V, axis=1, keepdims=True)
    E = (Vn @ Vn.T).astype(np.float32)
    feats = np.zeros(pol.K_s, np.float32)
    curve, seen_steps = [], 0
    p0, _ = pol.forward(V, E, feats)
    try:
        for t in range(events):
            p, _ = pol.forward(V, E, feats)
            chosen = int(rng.choice(pol.N, p=p / p.sum()))
            slot = t % num_slots
            learner.record_decision(slot, t, chosen, float(p[chosen]), V, E, feats)
            out = np.zeros((), dtype=N.REPLAY_OUTCOME)
            out["event_type"], out["slot_id"], out["gpu_step"], out["selection_step"] = 3, slot, t, t
            reward = (reward_gap if chosen == good_vertex else 0.0) + reward_std * rng.standard_normal()
            out["reward_shaped"] = out["ce_delta_raw"] = reward
            learner.on_replay_outcome(out)
            steps = int(learner.telemetry()["sgd_steps"])
            if steps != seen_steps:
                pol.flat[:] = learner.weights(slow=False)
                seen_steps = steps
            if (t + 1) % report_every == 0 or t + 1 == events:
                q, _ = pol.forward(V, E, feats)
                curve.append({"event": t + 1, "entropy": float(-(q * np.log(np.maximum(q, 1e-12))).sum()),
                              "p_good": float(q[good_vertex]), "max_p": float(q.max()),
                              "weight_drift_l2": float(np.linalg.norm(pol.flat - start))})
        tel = learner.telemetry()
    finally:
        learner.close()
    return {"temperature": float(temperature), "events": int(events), "uniform_entropy": math.log(pol.N),
            "initial_max_p": float(p0.max()), "initial_p_good": float(p0[good_vertex]), "curve": curve,
            "final": curve[-1], "sgd_steps": int(tel["sgd_steps"]), "credited_actions": int(tel["credited_actions"])}


def summarize_trace(path: Path | str, *, max_rows: Optional[int] = None) -> dict[str, Any]:
    """Counts and means per row type of one learner NDJSON trace."""
    counts: dict[str, int] = defaultdict(int)
    sums: dict[str, list[float]] = defaultdict(list)
    reasons: dict[str, int] = defaultdict(int)
    last_sgd = 0
    with open(path) as fh:
        for i, line in enumerate(fh):
            if max_rows is not None and i >= max_rows:
                break
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                counts["malformed"] += 1
                continue
            kind = str(row.get("row_type", "unknown"))
            counts[kind] += 1
            last_sgd = max(last_sgd, int(row.get("sgd_steps", 0) or 0))
            if kind == "skip":
                reasons[str(row.get("status_reason", ""))] += 1
            for key in ("entropy", "p_chosen", "current_entropy", "advantage_final", "gerber_weight",
                        "reward_shaped", *GRADIENT_COLUMNS):
                if isinstance(row.get(key), (int, float)):
                    sums[f"{kind}.{key}"].append(float(row[key]))
            if kind == "credit" and all(isinstance(row.get(k), (int, float)) for k in ("entropy", "current_entropy")):
                sums["credit.entropy_drift"].append(float(row["current_entropy"]) - float(row["entropy"]))
    stats = {k: {"mean": float(np.mean(v)), "std": float(np.std(v, ddof=1)) if len(v) > 1 else 0.0,
                 "min": float(np.min(v)), "max": float(np.max(v)), "n": len(v)}
             for k, v in sums.items()}
    return {"path": str(path), "rows": dict(counts), "skip_reasons": dict(reasons), "sgd_steps": last_sgd,
            "stats": stats}


def compare_traces(paths_by_arm: dict[str, Sequence[Path | str]]) -> dict[str, Any]:
    """Per arm (several seeds each): decision entropy, credit volume, |advantage| and SGD steps, the
    quantities that separate a policy that learns from one stuck at uniform."""
    out = {}
    for arm, paths in paths_by_arm.items():
        per = [summarize_trace(p) for p in paths]

        def mean_of(key: str, field: str = "mean") -> Optional[float]:
            vals = [s["stats"][key][field] for s in per if key in s["stats"]]
            return float(np.mean(vals)) if vals else None
        out[arm] = {"seeds": len(per), "decisions": sum(s["rows"].get("decision", 0) for s in per),
                    "credits": sum(s["rows"].get("credit", 0) for s in per),
                    "skips": sum(s["rows"].get("skip", 0) for s in per),
                    "sgd_steps_mean": float(np.mean([s["sgd_steps"] for s in per])) if per else 0.0,
                    "decision_entropy_mean": mean_of("decision.entropy"),
                    "decision_entropy_min": mean_of("decision.entropy", "min"),
                    "credit_entropy_mean": mean_of("credit.current_entropy"),
                    "entropy_drift_mean": mean_of("credit.entropy_drift"),
                    **{f"{c}_mean": mean_of(f"credit.{c}") for c in GRADIENT_COLUMNS},
                    "abs_advantage_max": max((abs(s["stats"]["credit.advantage_final"][f]) for s in per
                                              if "credit.advantage_final" in s["stats"] for f in ("min", "max")),
                                             default=None)}
    return out


def headline_ratio(comparison: dict[str, Any], baseline_arm: str, sharp_arm: str) -> dict[str, Any]:
    """The load-bearing comparison of the trace analysis: per credited action, does the arm that starts
    sharp accumulate a larger gradient and end with larger weights than the arm at the default
    temperature?  Ratios above one on ``grad_w_lh_accum_l2`` and ``w_lh_l2`` confirm that a uniform
    start starves the policy gradient."""
    a, b = comparison[baseline_arm], comparison[sharp_arm]
    out: dict[str, Any] = {"baseline_arm": baseline_arm, "sharp_arm": sharp_arm}
    for c in ("grad_w_lh_accum_l2", "w_lh_l2", "grad_logits_l2"):
        x, y = a.get(f"{c}_mean"), b.get(f"{c}_mean")
        out[c] = {"baseline": x, "sharp": y, "ratio": (y / x) if x and y is not None else None}
    r1, r2 = out["grad_w_lh_accum_l2"]["ratio"], out["w_lh_l2"]["ratio"]
    out["confirmed"] = bool(r1 is not None and r2 is not None and r1 > 1.0 and r2 > 1.0)
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--events", type=int, default=4000)
    ap.add_argument("--temperatures", type=float, nargs="+", default=[1.0, 0.2, 0.05])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--traces", nargs="*", default=None, help="arm=path[,path...] learner traces to compare instead")
    ap.add_argument("--headline", nargs=2, metavar=("BASELINE_ARM", "SHARP_ARM"), default=None,
                    help="with --traces: gradient / weight-norm ratios of the second arm over the first")
    a = ap.parse_args(argv)
    if a.traces:
        arms = {spec.split("=", 1)[0]: spec.split("=", 1)[1].split(",") for spec in a.traces}
        cmp = compare_traces(arms)
        if a.headline:
            cmp = {"arms": cmp, "headline": headline_ratio(cmp, a.headline[0], a.headline[1])}
        print(json.dumps(cmp, indent=2))
        return 0
    print(f"{'T':>6} {'max_p0':>8} {'entropy':>8} {'p_good':>7} {'drift':>8} {'sgd':>5}")
    for T in a.temperatures:
        r = run_bootstrap(temperature=T, events=a.events, seed=a.seed)
        f = r["final"]
        print(f"{T:6.2f} {r['initial_max_p']:8.4f} {f['entropy']:8.4f} {f['p_good']:7.3f} "
              f"{f['weight_drift_l2']:8.4f} {r['sgd_steps']:5d}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
