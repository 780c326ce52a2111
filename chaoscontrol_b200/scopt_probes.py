"""Pre-quality sanity gates for the scarcity-aware optimizer, evaluated over the
trace dicts that ``ScarcityAwareOptimizer.scarcity_trace()`` emits during a short run
(gates of src/chaoscontrol/scopt_probes.py:28-224).  Only post-warm-up traces count.

0.1 signal distribution   the median ``out_scarcity`` factor must vary across the run
0.2 NS convergence        not instrumented: always "skip"
0.3 rare/common alignment mean |median cos(rare, common)| inside a safe band (too small:
                          the rare direction is orthogonal everywhere and will destabilise;
                          too large: it is parallel and the mechanism is inert)
0.4 pressure sparsity     mean ``fraction_positive`` inside the calibrated band

Each gate is one declarative band check (value, low, high, messages).
"""
from __future__ import annotations

from typing import Any, Optional

__all__ = ["evaluate_tier0_gates", "summarize_gates"]


def _result(status: str, metric=None, reason: Optional[str] = None) -> dict[str, Any]:
    return {"status": status, "metric": metric, "reason": reason}


def _medians(traces: list[dict[str, Any]], key: str) -> list[float]:
    return [float(t[key]["median"]) for t in traces if isinstance(t.get(key), dict) and "median" in t[key]]


def _band(value: float, metric_key: str, low: float, high: float, below: str, above: str) -> dict[str, Any]:
    metric = {metric_key: value}
    if value < low:
        return _result("fail", metric, below.format(v=value, lo=low, hi=high))
    if value > high:
        return _result("fail", metric, above.format(v=value, lo=low, hi=high))
    return _result("pass", metric)


def _probe_signal_distribution(late, *, ratio_threshold: float) -> dict[str, Any]:
    med = _medians(late, "out_scarcity")
    if len(med) < 2:
        return _result("skip", reason="need >=2 post-warmup traces with out_scarcity telemetry")
    lo, hi = min(med), max(med)
    metric = {"min": lo, "max": hi, "ratio": hi / max(lo, 1e-9)}
    if metric["ratio"] < ratio_threshold:
        return _result("fail", metric, f"out_scarcity median range too narrow ({lo:.4f}-{hi:.4f}); channel pressure "
                                       "likely degenerate")
    return _result("pass", metric)


def _probe_alignment(late, *, safe_range: tuple[float, float]) -> dict[str, Any]:
    med = _medians(late, "cos_rare_common")
    if not med:
        return _result("skip", reason="no cos_rare_common telemetry in late traces")
    return _band(sum(abs(m) for m in med) / len(med), "mean_abs_cos", *safe_range,
                 "|cos(rare, common)| mean = {v:.3f} below {lo}; rare direction nearly orthogonal everywhere — "
                 "destabilization risk",
                 "|cos(rare, common)| mean = {v:.3f} above {hi}; rare direction nearly parallel to common — "
                 "mechanism inert")


def _probe_sparsity(late, *, target: tuple[float, float]) -> dict[str, Any]:
    fr = [float(t["pressure_stats"]["fraction_positive"]) for t in late
          if isinstance(t.get("pressure_stats"), dict) and "fraction_positive" in t["pressure_stats"]]
    if not fr:
        return _result("skip", reason="no pressure_stats.fraction_positive in late traces")
    return _band(sum(fr) / len(fr), "mean_fraction_positive", *target,
                 "mean fraction_positive = {v:.3f} below {lo}; pressure too sparse — baseline too strong or "
                 "calibration wrong",
                 "mean fraction_positive = {v:.3f} above {hi}; pressure too dense — degenerates to weighted "
                 "ordinary CE")


def evaluate_tier0_gates(traces: list[dict[str, Any]], *, min_late_steps: int = 200,
                         sparsity_target: tuple[float, float] = (0.05, 0.25),
                         alignment_safe_range: tuple[float, float] = (0.1, 0.9),
                         distribution_degenerate_ratio: float = 1.05) -> dict[str, dict[str, Any]]:
    late = [t for t in traces if int(t.get("step", 0)) >= min_late_steps and t.get("scarcity_enabled", False)]
    return {
        "0.1_signal_distribution": _probe_signal_distribution(late, ratio_threshold=distribution_degenerate_ratio),
        "0.2_ns_convergence": _result("skip", reason="NS residual not currently captured in scarcity_trace"),
        "0.3_rare_common_alignment": _probe_alignment(late, safe_range=alignment_safe_range),
        "0.4_pressure_sparsity": _probe_sparsity(late, target=sparsity_target),
    }


def summarize_gates(results: dict[str, dict[str, Any]]) -> str:
    return "\n".join(f"{name}: {body['status'].upper()}  {body.get('reason') or ''}" for name, body in results.items())
