"""Result analysis for experiment matrices: one module instead of one script per experiment.

* ``load_results``        result JSONs of a matrix run (one file per entry) -> flat metric rows
* ``summary_table``       mean / sample std / n per arm                  (analyze_phase3.py:71-88)
* ``paired_comparison``   seed-paired deltas against a control arm, paired t statistic and two-sided
                          p-value, fraction of seeds that beat the control (analyze_phase3.py:91-236,
                          experiments/19_phase1/summarize_phase1.py:388-500)
* ``lever_verdict``       SHIP / PARK / INCONCLUSIVE from throughput, loss and memory deltas
                          (summarize_phase1.py:1-60 rules)
* ``fit_power_law``       ``bpb = A * params^-alpha + bpb_irr`` (experiments/10_scaling_laws/
                          analyze_scaling.py:120-200), closed-form in log space over a grid of ``bpb_irr``
* ``curation_gate``       four-arm replay-curation falsifier: rare-bucket deltas, the tie band, the
                          spread that asks for more seeds, the four verdicts
                          (experiments/24_training_time_bundle/analyze_episodic_dw_curation_v1.py:52-170)
* ``render_markdown``     tables for a report
* CLI: ``python -m chaoscontrol_b200.analysis summarize|compare|scaling|curation ...``
"""
from __future__ import annotations

import argparse
import json
import math
import re
from pathlib import Path
from typing import Any, Iterable, Optional, Sequence

__all__ = ["load_results", "extract_metrics", "summary_table", "paired_ttest", "paired_comparison",
           "lever_verdict", "fit_power_law", "curation_gate", "load_curation_cells", "render_curation",
           "render_markdown", "main"]


# ---------------------------------------------------------------------------
# loading
# ---------------------------------------------------------------------------
def _get(d: dict, path: str, default=None):
    cur: Any = d
    for k in path.split("."):
        if not isinstance(cur, dict) or k not in cur:
            return default
        cur = cur[k]
    return cur


def extract_metrics(result: dict[str, Any]) -> dict[str, Any]:
    """Flat row from one runner result (``config / params / train / eval`` layout)."""
    cfg = result.get("config", {}) or {}
    row = {"name": cfg.get("name") or result.get("name"), "seed": cfg.get("seed"), "params": result.get("params"),
           "tokens_per_sec": _get(result, "train.aggregate_tokens_per_sec"),
           "steps": _get(result, "train.steps"), "final_loss": _get(result, "train.final_loss"),
           "peak_vram_mb": _get(result, "train.peak_vram_mb"), "bpb": _get(result, "eval.bpb"),
           "eval_loss": _get(result, "eval.loss"), "error": result.get("error")}
    arm = cfg.get("arm") or cfg.get("exp24_mechanism")
    if arm is None and isinstance(row["name"], str):
        arm = row["name"].rsplit("_s", 1)[0] if "_s" in row["name"] else row["name"]
    row["arm"] = arm
    return row


def load_results(paths: Iterable[Path | str]) -> list[dict[str, Any]]:
    """Every ``*.json`` under the given files / directories that parses as a result
    dict (error markers included, flagged by ``error``)."""
    rows = []
    for p in paths:
        p = Path(p)
        files = sorted(p.rglob("*.json")) if p.is_dir() else [p]
        for f in files:
            try:
                blob = json.loads(f.read_text())
            except (OSError, json.JSONDecodeError):
                continue
            for rec in (blob if isinstance(blob, list) else [blob]):
                if isinstance(rec, dict) and ("train" in rec or "eval" in rec or "error" in rec):
                    row = extract_metrics(rec)
                    row["path"] = str(f)
                    rows.append(row)
    return rows


# ---------------------------------------------------------------------------
# statistics
# ---------------------------------------------------------------------------
def _mean(v: Sequence[float]) -> float:
    return sum(v) / len(v) if v else float("nan")


def _std(v: Sequence[float]) -> float:
    if len(v) < 2:
        return 0.0
    m = _mean(v)
    return math.sqrt(sum((x - m) ** 2 for x in v) / (len(v) - 1))


def _betacf(a: float, b: float, x: float) -> float:
    tiny, qab, qap, qam = 1e-300, a + b, a + 1.0, a - 1.0
    c, d = 1.0, 1.0 - qab * x / qap
    d = 1.0 / (d if abs(d) > tiny else tiny)
    h = d
    for m in range(1, 300):
        m2 = 2 * m
        aa = m * (b - m) * x / ((qam + m2) * (a + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        h *= d * c
        aa = -(a + m) * (qab + m) * x / ((a + m2) * (qap + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        delta = d * c
        h *= delta
        if abs(delta - 1.0) < 3e-16:
            break
    return h


def _betainc(a: float, b: float, x: float) -> float:
    if x <= 0.0:
        return 0.0
    if x >= 1.0:
        return 1.0
    ln = math.lgamma(a + b) - math.lgamma(a) - math.lgamma(b) + a * math.log(x) + b * math.log(1.0 - x)
    if x < (a + 1.0) / (a + b + 2.0):
        return math.exp(ln) * _betacf(a, b, x) / a
    return 1.0 - math.exp(ln) * _betacf(b, a, 1.0 - x) / b


def paired_ttest(a: Sequence[float], b: Sequence[float]) -> tuple[float, float]:
    """Dependent-samples t statistic of ``a - b`` and its two-sided p-value
    (Student t with n-1 degrees of freedom via the regularised incomplete beta)."""
    if len(a) != len(b):
        raise ValueError("paired_ttest needs samples of equal length")
    n = len(a)
    if n < 2:
        return float("nan"), float("nan")
    d = [x - y for x, y in zip(a, b)]
    sd = _std(d)
    if sd == 0.0:
        m = _mean(d)
        return (0.0, 1.0) if m == 0 else (math.copysign(float("inf"), m), 0.0)
    t = _mean(d) / (sd / math.sqrt(n))
    df = n - 1
    return t, _betainc(df / 2.0, 0.5, df / (df + t * t))


def summary_table(rows: Sequence[dict], metric: str = "bpb", by: str = "arm") -> list[dict[str, Any]]:
    groups: dict[Any, list[float]] = {}
    for r in rows:
        v = r.get(metric)
        if r.get("error") or v is None or not math.isfinite(float(v)):
            continue
        groups.setdefault(r.get(by), []).append(float(v))
    return [{"arm": k, "n": len(v), "mean": _mean(v), "std": _std(v), "min": min(v), "max": max(v)}
            for k, v in sorted(groups.items(), key=lambda kv: _mean(kv[1]))]


def paired_comparison(rows: Sequence[dict], *, control: str, metric: str = "bpb", by: str = "arm",
                      lower_is_better: bool = True) -> list[dict[str, Any]]:
    """Every arm against ``control`` on the seeds both have."""
    table: dict[Any, dict[Any, float]] = {}
    for r in rows:
        v = r.get(metric)
        if r.get("error") or v is None or r.get("seed") is None or not math.isfinite(float(v)):
            continue
        table.setdefault(r.get(by), {})[r["seed"]] = float(v)
    if control not in table:
        raise KeyError(f"control arm {control!r} has no usable rows")
    out = []
    for arm, per_seed in sorted(table.items(), key=lambda kv: str(kv[0])):
        if arm == control:
            continue
        seeds = sorted(set(per_seed) & set(table[control]))
        a, b = [per_seed[s] for s in seeds], [table[control][s] for s in seeds]
        deltas = [x - y for x, y in zip(a, b)]
        t, p = paired_ttest(a, b)
        wins = sum(1 for d in deltas if (d < 0 if lower_is_better else d > 0))
        out.append({"arm": arm, "control": control, "n_pairs": len(seeds), "mean_delta": _mean(deltas),
                    "std_delta": _std(deltas), "t": t, "p": p,
                    "fraction_beating_control": wins / len(seeds) if seeds else float("nan")})
    return out


def lever_verdict(rows: Sequence[dict], *, on: str, off: str, by: str = "arm", alpha: float = 0.05,
                  max_loss_delta: float = 0.02, max_vram_frac: float = 0.05) -> dict[str, Any]:
    """``SHIP`` when the lever raises tokens/s significantly without moving the final
    loss by more than ``max_loss_delta`` or peak memory by more than ``max_vram_frac``;
    ``PARK`` when throughput does not improve or a quality bound breaks;
    ``INCONCLUSIVE`` when the mean is positive but not significant."""
    sub = [r for r in rows if r.get(by) in (on, off)]
    tok = paired_comparison(sub, control=off, metric="tokens_per_sec", by=by, lower_is_better=False)
    if not tok or tok[0]["n_pairs"] == 0:
        return {"verdict": "INCONCLUSIVE", "reason": "no seed-paired runs"}
    tok = tok[0]
    loss = paired_comparison(sub, control=off, metric="final_loss", by=by)
    vram = paired_comparison(sub, control=off, metric="peak_vram_mb", by=by)
    base_vram = _mean([float(r["peak_vram_mb"]) for r in sub if r.get(by) == off and r.get("peak_vram_mb")])
    d_loss = abs(loss[0]["mean_delta"]) if loss and loss[0]["n_pairs"] else 0.0
    d_vram = abs(vram[0]["mean_delta"]) / base_vram if vram and vram[0]["n_pairs"] and base_vram else 0.0
    quality_ok = d_loss <= max_loss_delta and d_vram <= max_vram_frac
    if tok["mean_delta"] <= 0 or not quality_ok:
        verdict = "PARK"
    elif tok["p"] < alpha:
        verdict = "SHIP"
    else:
        verdict = "INCONCLUSIVE"
    return {"verdict": verdict, "delta_tokens_per_sec": tok["mean_delta"], "p": tok["p"], "n_pairs": tok["n_pairs"],
            "abs_delta_final_loss": d_loss, "rel_delta_peak_vram": d_vram}


# ---------------------------------------------------------------------------
# scaling law
# ---------------------------------------------------------------------------
def fit_power_law(params: Sequence[float], bpbs: Sequence[float]) -> dict[str, float]:
    """``bpb = A * N^-alpha + bpb_irr``.  For a fixed ``bpb_irr`` the model is a
    line in log-log space, so ``bpb_irr`` is scanned over ``[0, min(bpb))`` and the
    best least-squares line wins.  Needs at least three points."""
    if len(params) != len(bpbs) or len(params) < 3:
        raise ValueError("fit_power_law needs at least three (params, bpb) points")
    lx = [math.log(float(p)) for p in params]
    lo = min(bpbs)
    best = None
    for i in range(0, 400):
        irr = lo * i / 400.0 * 0.999
        ly = [math.log(float(b) - irr) for b in bpbs]
        mx, my = _mean(lx), _mean(ly)
        sxx = sum((x - mx) ** 2 for x in lx)
        if sxx == 0:
            raise ValueError("all parameter counts are equal")
        slope = sum((x - mx) * (y - my) for x, y in zip(lx, ly)) / sxx
        icpt = my - slope * mx
        sse = sum((math.exp(icpt + slope * x) + irr - float(b)) ** 2 for x, b in zip(lx, bpbs))
        if best is None or sse < best[0]:
            best = (sse, math.exp(icpt), -slope, irr)
    sse, A, alpha, irr = best
    mean_b = _mean([float(b) for b in bpbs])
    sst = sum((float(b) - mean_b) ** 2 for b in bpbs)
    return {"A": A, "alpha": alpha, "bpb_irr": irr, "sse": sse, "r2": 1.0 - sse / sst if sst > 0 else float("nan")}


# ---------------------------------------------------------------------------
# rendering / CLI
# ---------------------------------------------------------------------------
def render_markdown(rows: Sequence[dict], columns: Optional[Sequence[str]] = None) -> str:
    if not rows:
        return "(no rows)\n"
    cols = list(columns or rows[0].keys())

    def fmt(v):
        if isinstance(v, float):
            return "nan" if math.isnan(v) else (f"{v:.3g}" if abs(v) < 1e-3 or abs(v) >= 1e5 else f"{v:.4f}")
        return str(v)
    lines = ["| " + " | ".join(cols) + " |", "|" + "|".join("---" for _ in cols) + "|"]
    lines += ["| " + " | ".join(fmt(r.get(c)) for c in cols) + " |" for r in rows]
    return "\n".join(lines) + "\n"


# ---------------------------------------------------------------------------
# replay-curation falsifier (uncurated / cosine x utility / pressure only / no replay)
# ---------------------------------------------------------------------------
CURATION_ARMS = ("arm_a_uncurated", "arm_b_cosine_utility", "arm_bp_pressure_only", "arm_c_no_dw")
CURATION_DELTA_MIN = 0.005          # rare-bucket gain (bpb) that counts as a pass
CURATION_SIGMA_ESCALATE = 0.008     # spread of the curated arm above which three more seeds are due
CURATION_VERDICTS = {
    "pass_mechanism_specific": "PASS, mechanism-specific: the curated query beats both uncurated replay and the "
                               "pressure-only query on the rarest bucket",
    "pass_mechanism_agnostic": "PASS, mechanism-agnostic: curated beats uncurated but ties the pressure-only query",
    "mixed_null": "MIXED / NULL: curation did not beat uncurated replay",
    "regression": "REGRESSION: curation is worse than uncurated replay",
}


def _mean_se(v: Sequence[float]) -> tuple[float, float]:
    if len(v) < 2:
        return (float(v[0]) if v else float("nan")), float("nan")
    return _mean(v), _std(v) / math.sqrt(len(v))


def load_curation_cells(results_dir: Path | str) -> dict[str, list[dict[str, float]]]:
    """``{arm: [{"rare", "overall", "seed"}]}`` from the result files of the curation matrix.  The rare
    figure is the first entry of the per-bucket validation list (buckets are ordered rarest first), read
    from the result itself, its ``train`` block, or the summary file it points at."""
    out: dict[str, list[dict[str, float]]] = {a: [] for a in CURATION_ARMS}
    files = sorted(Path(results_dir).glob("*episodic_dw_curation_v1_*.json"))
    if not files:
        raise FileNotFoundError(f"no curation cells under {results_dir}")
    for f in files:
        cell = json.loads(f.read_text())
        name = str(cell.get("name") or _get(cell, "config.name") or f.stem)
        arm = next((a for a in CURATION_ARMS if a in name), None)
        if arm is None:
            raise ValueError(f"cannot tell the arm of {name!r}")
        tr = cell.get("train") or {}
        buckets = (cell.get("val_per_bucket_bpb") or tr.get("val_per_bucket_bpb") or cell.get("per_bucket_val_ce")
                   or tr.get("per_bucket_val_ce"))
        if buckets is None and cell.get("val_summary_path"):
            buckets = json.loads(Path(cell["val_summary_path"]).read_text()).get("val_per_bucket_bpb")
        if not buckets:
            raise ValueError(f"{name!r} carries no per-bucket validation figures")
        overall = cell.get("val_bpb", _get(cell, "eval.bpb"))
        out[arm].append({"rare": float(buckets[0]), "overall": float("nan") if overall is None else float(overall),
                         "seed": float(_get(cell, "config.seed", cell.get("seed", -1)))})
    return out


def curation_gate(cells: dict[str, list[dict[str, float]]]) -> dict[str, Any]:
    rare = {a: [c["rare"] for c in cells.get(a, [])] for a in CURATION_ARMS}
    a_mean, _ = _mean_se(rare["arm_a_uncurated"])
    b_mean, b_se = _mean_se(rare["arm_b_cosine_utility"])
    bp_mean, bp_se = _mean_se(rare["arm_bp_pressure_only"])
    c_mean, _ = _mean_se(rare["arm_c_no_dw"])
    nz = lambda x: 0.0 if math.isnan(x) else x                                                # noqa: E731
    d_a, d_bp = b_mean - a_mean, b_mean - bp_mean                  # negative = the curated arm is better
    sigma_b = _std(rare["arm_b_cosine_utility"]) if len(rare["arm_b_cosine_utility"]) >= 2 else float("nan")
    ties_bp = abs(d_bp) < 2.0 * math.hypot(nz(b_se), nz(bp_se))
    if d_a >= 0:
        verdict = "regression" if d_a > 2.0 * nz(b_se) else "mixed_null"
    elif abs(d_a) < CURATION_DELTA_MIN:
        verdict = "mixed_null"
    else:
        verdict = "pass_mechanism_agnostic" if ties_bp else "pass_mechanism_specific"
    return {"verdict": verdict, "delta_b_vs_a": d_a, "delta_b_vs_bp": d_bp, "sigma_b": sigma_b,
            "needs_escalation": (not math.isnan(sigma_b)) and sigma_b > CURATION_SIGMA_ESCALATE,
            "rare_means": {"A": a_mean, "B": b_mean, "Bp": bp_mean, "C": c_mean},
            "by_arm_count": {a: len(rare[a]) for a in CURATION_ARMS}}


def render_curation(cells: dict[str, list[dict[str, float]]], gate: dict[str, Any]) -> str:
    rows = []
    for a in CURATION_ARMS:
        m, se = _mean_se([c["rare"] for c in cells.get(a, [])])
        om, _ = _mean_se([c["overall"] for c in cells.get(a, [])])
        rows.append({"arm": a, "n": len(cells.get(a, [])), "rare_mean": m, "rare_stderr": se, "overall_mean": om})
    tail = [f"rare-bucket delta, curated - uncurated: {gate['delta_b_vs_a']:+.4f} bpb (negative = curated better)",
            f"rare-bucket delta, curated - pressure-only: {gate['delta_b_vs_bp']:+.4f} bpb",
            f"spread of the curated arm: {gate['sigma_b']:.4f} bpb"
            + (f" (> {CURATION_SIGMA_ESCALATE}: run three more seeds of A, B and B' before deciding)"
               if gate["needs_escalation"] else ""),
            "verdict: " + CURATION_VERDICTS[gate["verdict"]]]
    return render_markdown(rows) + "\n" + "\n".join(tail) + "\n"


# ---------------------------------------------------------------------------------------------------------
# Controller arms: throughput, loss, event-path health and learner-trace gradient diagnostics per arm
# (scripts/analyze_step3_v3_diagnostics.py:31-190, without DuckDB).
_ARM_NAME = re.compile(r"(arm_[a-z]+(?:_[a-z]+)*)_s(\d+)$")


def load_controller_arms(results_dir: Path | str, prefix: str = "") -> dict[str, list[dict[str, Any]]]:
    """Result files ``<prefix><arm>_s<seed>.json`` grouped by arm (``arm_d_simplex_online`` and the like)."""
    arms: dict[str, list[dict[str, Any]]] = {}
    for f in sorted(Path(results_dir).glob(f"{prefix}*.json")):
        m = _ARM_NAME.search(f.stem[len(prefix):])
        if not m:
            continue
        arms.setdefault(m.group(1), []).append({"seed": int(m.group(2)), "name": f.stem[len(prefix):],
                                                "data": json.loads(f.read_text())})
    for cells in arms.values():
        cells.sort(key=lambda c: c["seed"])
    return arms


def controller_arm_report(results_dir: Path | str, traces_dir: Optional[Path | str] = None, *, prefix: str = "",
                          trace_prefix: str = "", headline: Optional[tuple[str, str]] = None) -> dict[str, Any]:
    """Per arm: cells, mean steps, steps per second and final loss (mean, sample std); per cell: how many
    write / query events were emitted, dropped and ingested and how many SGD steps the learner took; per
    arm over its learner traces (``<trace_prefix><arm>_s<seed>.ndjson``): the gradient-norm columns and the
    entropy drift of credited actions; with ``headline=(baseline, sharp)`` the ratio table that says whether
    the sharper start accumulates more gradient and weight."""
    from .episodic.bootstrap_bench import compare_traces, headline_ratio, summarize_trace
    arms = load_controller_arms(results_dir, prefix)
    summary, health = [], []
    trace_paths: dict[str, list[Path]] = {}
    for arm in sorted(arms):
        trains = [c["data"].get("train") or {} for c in arms[arm]]
        sps = [t["steps"] / t["elapsed_s"] for t in trains if t.get("steps") and t.get("elapsed_s")]
        losses = [float(t["final_loss"]) for t in trains if t.get("final_loss") is not None]
        summary.append({"arm": arm, "n": len(trains), "mean_steps": _mean([float(t.get("steps", 0)) for t in trains]),
                        "steps_per_s": _mean(sps) if sps else None, "steps_per_s_std": _std(sps) if len(sps) > 1 else None,
                        "final_loss": _mean(losses) if losses else None,
                        "final_loss_std": _std(losses) if len(losses) > 1 else None})
        for c in arms[arm]:
            tr = c["data"].get("train") or {}
            ep = tr.get("episodic") or c["data"].get("episodic") or {}
            aw = _get(c["data"], "train.mechanisms.episodic_async_writes") or {}
            row = {"cell": c["name"],
                   "emitted": int(ep.get("write_events_emitted", aw.get("pushed", 0)) or 0),
                   "dropped": int(ep.get("write_events_dropped", aw.get("publish_drops", 0)) or 0),
                   "ingested": int(ep.get("write_events_ingested", 0) or 0),
                   "query_dropped": int(ep.get("query_events_dropped", 0) or 0),
                   "errors": int(aw.get("drain_errors", 0) or 0), "sgd_steps": None}
            if traces_dir is not None:
                t = Path(traces_dir) / f"{trace_prefix}{c['name']}.ndjson"
                if t.exists():
                    row["sgd_steps"] = summarize_trace(t)["sgd_steps"]
                    trace_paths.setdefault(arm, []).append(t)
            health.append(row)
    out: dict[str, Any] = {"arms": summary, "health": health}
    if trace_paths:
        out["traces"] = compare_traces(trace_paths)
        if headline is not None and all(h in out["traces"] for h in headline):
            out["headline"] = headline_ratio(out["traces"], headline[0], headline[1])
    return out


def render_controller_arms(rep: dict[str, Any]) -> str:
    pm = lambda m, s_: "-" if m is None else (f"{m:.4f}" if s_ is None else f"{m:.4f} +/- {s_:.4f}")          # noqa: E731
    parts = ["## Per arm", render_markdown([{"arm": r["arm"], "n": r["n"], "steps": int(r["mean_steps"]),
                                              "steps/s": pm(r["steps_per_s"], r["steps_per_s_std"]),
                                              "final loss": pm(r["final_loss"], r["final_loss_std"])} for r in rep["arms"]]),
             "", "## Event path health", render_markdown(rep["health"])]
    if "traces" in rep:
        cols = ("credits", "sgd_steps_mean", "entropy_drift_mean", "grad_logits_l2_mean", "grad_w_lh_l2_mean",
                "grad_w_lh_accum_l2_mean", "w_lh_l2_mean")
        parts += ["", "## Credited actions (means over each arm's traces)",
                  render_markdown([{"arm": a, **{c: v.get(c) for c in cols}} for a, v in rep["traces"].items()])]
    if "headline" in rep:
        h = rep["headline"]
        parts += ["", f"## {h['sharp_arm']} over {h['baseline_arm']}: " + ("confirmed" if h["confirmed"] else "not confirmed"),
                  render_markdown([{"column": c, **h[c]} for c in ("grad_w_lh_accum_l2", "w_lh_l2", "grad_logits_l2")])]
    return "\n".join(parts)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="chaoscontrol_b200.analysis")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("summarize")
    s.add_argument("paths", nargs="+")
    s.add_argument("--metric", default="bpb")
    s.add_argument("--by", default="arm")
    c = sub.add_parser("compare")
    c.add_argument("paths", nargs="+")
    c.add_argument("--control", required=True)
    c.add_argument("--metric", default="bpb")
    c.add_argument("--by", default="arm")
    c.add_argument("--higher-is-better", action="store_true")
    g = sub.add_parser("scaling")
    g.add_argument("paths", nargs="+")
    g.add_argument("--by", default="arm")
    q = sub.add_parser("curation")
    q.add_argument("results_dir")
    ca = sub.add_parser("controller-arms")
    ca.add_argument("results_dir")
    ca.add_argument("--traces-dir", default=None)
    ca.add_argument("--prefix", default="")
    ca.add_argument("--trace-prefix", default="")
    ca.add_argument("--headline", nargs=2, default=None, metavar=("BASELINE_ARM", "SHARP_ARM"))
    ca.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "controller-arms":
        rep = controller_arm_report(a.results_dir, a.traces_dir, prefix=a.prefix, trace_prefix=a.trace_prefix,
                                    headline=tuple(a.headline) if a.headline else None)
        print(json.dumps(rep, indent=2) if a.json else render_controller_arms(rep))
        return 0
    if a.cmd == "curation":
        cells = load_curation_cells(a.results_dir)
        print(render_curation(cells, curation_gate(cells)))
        return 0
    rows = load_results(a.paths)
    if a.cmd == "summarize":
        print(render_markdown(summary_table(rows, a.metric, a.by)))
        bad = [r for r in rows if r.get("error")]
        if bad:
            print(f"{len(bad)} run(s) ended in an error: " + ", ".join(str(r.get("name")) for r in bad[:10]))
    elif a.cmd == "compare":
        print(render_markdown(paired_comparison(rows, control=a.control, metric=a.metric, by=a.by,
                                                lower_is_better=not a.higher_is_better)))
    else:
        groups: dict[Any, list[dict]] = {}
        for r in rows:
            if r.get("params") and r.get("bpb") is not None and not r.get("error"):
                groups.setdefault(r.get(a.by), []).append(r)
        fits = []
        for k, rs in groups.items():
            sizes = sorted({int(r["params"]) for r in rs})
            if len(sizes) < 3:
                continue
            pts = [(n, _mean([float(r["bpb"]) for r in rs if int(r["params"]) == n])) for n in sizes]
            fits.append({"arm": k, "points": len(pts), **fit_power_law([p for p, _ in pts], [b for _, b in pts])})
        print(render_markdown(fits))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
