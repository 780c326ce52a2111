"""Architecture and mechanism studies (experiments 09-17) as data.

The reference keeps one runner script per study (experiments/09_revised_architecture/
run_layered.py, 10_scaling_laws/run_scaling.py, 11_sleep_cycle/run_sleep_ablation.py,
12_polyphasic_sleep/run_polyphasic_ablation.py, 13_constants_validation/
run_constants_sweep.py, 14_vram_buffer/run_exp14.py, 15_chaospiece/run_exp15.py,
16_entropy_sparse_attention/run_exp16.py, 17_local_attn_sidecar/run_exp17.py, and
experiments/baselines/run_mamba2_baseline.py), each
repeating the launch loop and its own copy of the statistics.  Here a study is a
:class:`Study` value -- base envelopes, named conditions, seeds, pre-registered
contrasts and a decision rule -- and one engine does the rest:

* ``entries(study)``: ``<condition>_s<seed>`` matrix entries for ``launch.run_matrix``;
* ``analyse(study, results_dir)``: per-condition mean / SEM / bootstrap CI, the
  confirmatory family with exact paired Wilcoxon signed-rank p-values under Holm's
  step-down correction, exploratory contrasts uncorrected with effect sizes;
* ``LayeredStudy``: the layer-by-layer protocol of experiment 09, where each layer's
  winner (lowest mean bpb; Welch test and Cohen's d against the runner-up) hands a
  named subset of its settings to the layers after it.

Condition names, config keys and values are the reference's: result files and
downstream summaries are keyed by them.
"""
from __future__ import annotations

import json
import math
import random
import re
import statistics
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Optional, Sequence

from .analysis import _betainc, paired_ttest  # noqa: F401  (paired_ttest re-exported for study scripts)

SEEDS3 = (1337, 2674, 4011)
SEEDS7 = (1337, 2674, 4011, 5348, 6685, 8022, 9359)


# ---------------------------------------------------------------------------
# statistics (pure Python; cf. experiments/09_revised_architecture/stats.py:19-240)
# ---------------------------------------------------------------------------
def sem(v: Sequence[float]) -> float:
    return statistics.stdev(v) / math.sqrt(len(v)) if len(v) > 1 else 0.0


def bootstrap_ci(v: Sequence[float], *, n_boot: int = 2000, alpha: float = 0.05, seed: int = 0) -> tuple[float, float]:
    """Percentile bootstrap interval of the mean (deterministic for a given seed)."""
    v = list(v)
    if not v:
        return (float("nan"), float("nan"))
    if len(v) == 1:
        return (v[0], v[0])
    rng = random.Random(seed)
    n = len(v)
    means = sorted(sum(v[rng.randrange(n)] for _ in range(n)) / n for _ in range(n_boot))
    return (means[int(alpha / 2 * n_boot)], means[min(n_boot - 1, int((1 - alpha / 2) * n_boot))])


def cohens_d(a: Sequence[float], b: Sequence[float]) -> float:
    if len(a) < 2 or len(b) < 2:
        return 0.0
    va, vb = statistics.variance(a), statistics.variance(b)
    pooled = math.sqrt(((len(a) - 1) * va + (len(b) - 1) * vb) / (len(a) + len(b) - 2))
    return (statistics.fmean(a) - statistics.fmean(b)) / pooled if pooled > 0 else 0.0


def welch_ttest(a: Sequence[float], b: Sequence[float]) -> tuple[float, float]:
    """Two-sided Welch test (unequal variances); ``(t, p)``."""
    if len(a) < 2 or len(b) < 2:
        return 0.0, 1.0
    va, vb = statistics.variance(a) / len(a), statistics.variance(b) / len(b)
    if va + vb == 0:
        return 0.0, 1.0
    t = (statistics.fmean(a) - statistics.fmean(b)) / math.sqrt(va + vb)
    df = (va + vb) ** 2 / (va ** 2 / (len(a) - 1) + vb ** 2 / (len(b) - 1))
    return t, _betainc(df / 2.0, 0.5, df / (df + t * t))


def wilcoxon_signed_rank_p(deltas: Sequence[float]) -> float:
    """Exact two-sided p of the signed-rank statistic by enumerating all sign patterns
    (zero differences dropped, tied magnitudes given average ranks).  With 7 pairs the
    smallest attainable value is 2 / 128."""
    nz = sorted(abs(d) for d in deltas if d != 0.0)
    n = len(nz)
    if n == 0:
        return 1.0
    ranks: dict[float, float] = {}
    i = 0
    while i < n:
        j = i
        while j < n and nz[j] == nz[i]:
            j += 1
        ranks[nz[i]] = (i + 1 + j) / 2.0
        i = j
    r = [ranks[abs(d)] for d in deltas if d != 0.0]
    w_plus = sum(rk for rk, d in zip(r, (d for d in deltas if d != 0.0)) if d > 0)
    total = sum(r)
    w = min(w_plus, total - w_plus)
    # distribution of the positive-rank sum over all 2^n sign patterns (ranks doubled to stay integral)
    counts = {0: 1}
    for rk in r:
        step = int(round(2 * rk))
        nxt: dict[int, int] = {}
        for s, c in counts.items():
            nxt[s] = nxt.get(s, 0) + c
            nxt[s + step] = nxt.get(s + step, 0) + c
        counts = nxt
    lim = int(round(2 * w))
    tail = sum(c for s, c in counts.items() if s <= lim)
    return min(1.0, 2.0 * tail / float(1 << n))


def holm_bonferroni(named_p: Sequence[tuple[str, float]], alpha: float = 0.05) -> list[tuple[str, float, float, bool]]:
    """Step-down correction with the running maximum; ``[(name, raw, corrected, significant)]`` in input order."""
    order = sorted(range(len(named_p)), key=lambda i: named_p[i][1])
    m, run = len(named_p), 0.0
    corr = [0.0] * m
    for k, i in enumerate(order):
        run = max(run, min(1.0, named_p[i][1] * (m - k)))
        corr[i] = run
    return [(n, p, c, c < alpha) for (n, p), c in zip(named_p, corr)]


# ---------------------------------------------------------------------------
# study description
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class Contrast:
    name: str
    a: str                 # reference condition
    b: str                 # treatment: delta = bpb(b) - bpb(a), negative means b is better
    question: str = ""


@dataclass(frozen=True)
class Study:
    key: str
    title: str
    conditions: dict[str, dict[str, Any]]
    seeds: Sequence[int] = SEEDS7
    confirmatory: Sequence[Contrast] = ()
    exploratory: Sequence[Contrast] = ()
    decide: Optional[Callable[[dict], str]] = None
    budget_seconds: float = 600.0
    metric: str = "bpb"


def entries(study: Study, *, seeds: Optional[Sequence[int]] = None, only: Optional[Sequence[str]] = None) -> list[dict]:
    out = []
    for c, cfg in study.conditions.items():
        if only is not None and c not in only:
            continue
        for s in (seeds or study.seeds):
            out.append(dict(cfg, name=f"{c}_s{s}", condition=c, seed=int(s), study=study.key,
                            budget_seconds=study.budget_seconds))
    return out


def load_metric(results_dir: Path, conditions: Sequence[str], metric: str = "bpb") -> dict[str, dict[int, float]]:
    """``condition -> seed -> value`` from ``<condition>_s<seed>.json`` (``eval.bpb_gated`` wins over
    ``eval.bpb`` when a gate was active during evaluation); error markers and non-finite values are skipped."""
    out: dict[str, dict[int, float]] = {}
    for c in conditions:
        pat = re.compile(rf"^{re.escape(c)}_s(?:eed)?(\d+)\.json$")
        for f in sorted(Path(results_dir).glob(f"{c}_s*.json")):
            m = pat.match(f.name)
            if not m:
                continue
            try:
                ev = json.loads(f.read_text()).get("eval") or {}
            except json.JSONDecodeError:
                continue
            v = ev.get(f"{metric}_gated", ev.get(metric))
            if v is not None and math.isfinite(float(v)):
                out.setdefault(c, {})[int(m.group(1))] = float(v)
    return out


def _contrast_row(c: Contrast, data: dict[str, dict[int, float]]) -> Optional[dict[str, Any]]:
    a, b = data.get(c.a, {}), data.get(c.b, {})
    shared = sorted(set(a) & set(b))
    if not shared:
        return None
    deltas = [b[s] - a[s] for s in shared]
    return {"name": c.name, "a": c.a, "b": c.b, "question": c.question, "n": len(shared),
            "mean_delta": statistics.fmean(deltas), "ci_95": bootstrap_ci(deltas),
            "effect_size": cohens_d([b[s] for s in shared], [a[s] for s in shared]),
            "p_raw": wilcoxon_signed_rank_p(deltas)}


def analyse(study: Study, results_dir: Path) -> dict[str, Any]:
    data = load_metric(results_dir, list(study.conditions), study.metric)
    table = {c: {"n": len(v), "mean": statistics.fmean(v.values()), "sem": sem(list(v.values())),
                 "ci_95": bootstrap_ci(list(v.values()))} for c, v in data.items()}
    conf = [r for r in (_contrast_row(c, data) for c in study.confirmatory) if r]
    for r, (_, _, pc, sig) in zip(conf, holm_bonferroni([(r["name"], r["p_raw"]) for r in conf])):
        r["p_holm"], r["significant"] = pc, sig
    expl = [r for r in (_contrast_row(c, data) for c in study.exploratory) if r]
    out = {"study": study.key, "conditions": table, "confirmatory": conf, "exploratory": expl,
           "ranked": sorted(table, key=lambda c: table[c]["mean"])}
    if study.decide is not None and conf:
        out["decision"] = study.decide({r["name"]: r for r in conf})
    return out


def pick_winner(per_config: dict[str, Sequence[float]]) -> tuple[Optional[str], dict[str, Any]]:
    """Lowest mean; significance, effect size against the runner-up, bootstrap CI of the winner."""
    ranked = sorted(((k, list(v)) for k, v in per_config.items() if v), key=lambda kv: statistics.fmean(kv[1]))
    if not ranked:
        return None, {"significant": False, "p_value": 1.0, "effect_size": 0.0, "n_seeds": 0}
    name, vals = ranked[0]
    info = {"mean": statistics.fmean(vals), "std": statistics.stdev(vals) if len(vals) > 1 else 0.0,
            "ci_95": bootstrap_ci(vals), "n_seeds": len(vals), "significant": False, "p_value": 1.0,
            "effect_size": 0.0, "runner_up": ranked[1][0] if len(ranked) > 1 else None}
    if len(ranked) > 1 and len(vals) >= 2 and len(ranked[1][1]) >= 2:
        _, p = welch_ttest(vals, ranked[1][1])
        info.update(p_value=p, significant=p < 0.05, effect_size=cohens_d(vals, ranked[1][1]))
    return name, info


# ---------------------------------------------------------------------------
# experiment 09: layers that inherit from earlier winners
# ---------------------------------------------------------------------------
_SHARED = {"model_dim": 128, "num_layers": 4, "a_mode": "diag", "model_type": "ssm"}
_GATE = {"metabolic_gate": True, "metabolic_threshold": 0.1, "metabolic_threshold_mode": "fixed"}
_VQ = {"tokenizer_type": "fixed_stride", "tokenizer_stride": 4, "tokenizer_byte_dim": 64, "tokenizer_token_dim": 128,
       "tokenizer_beta": 0.25}
_WERNICKE = {"wernicke_enabled": True, "wernicke_router": "moe", "wernicke_k_max": 16}
_EPI = {"outer_model_dim": 64, "outer_model_type": "multislot"}
_BEST_MEM = {**_EPI, "semantic_tier_bases": 8, "eval_warmup": True, "consolidation_write": "full_sequence",
             "latent_persistence": True, "typed_consolidation": True}

CARRY_KEYS = {
    "tokenizer": ("tokenizer_type", "tokenizer_stride", "tokenizer_byte_dim", "tokenizer_token_dim",
                  "tokenizer_codebook_size", "tokenizer_beta", "vocab_size", "align_type", "align_weight"),
    "gate": ("metabolic_gate", "metabolic_k", "metabolic_mode", "mcts_horizon", "metabolic_threshold",
             "metabolic_threshold_mode"),
    "memory": ("outer_model_dim", "outer_model_type", "semantic_tier_bases", "eval_warmup", "consolidation_write",
               "latent_persistence", "typed_consolidation"),
    "wernicke": ("wernicke_enabled", "wernicke_router", "wernicke_k_max", "cfr_enabled", "typed_storage",
                 "compression_consequence"),
}


def _gate_passthrough(base: dict) -> dict:
    return {"metabolic_gate": True, "metabolic_mode": base.get("metabolic_mode", "fork"),
            "metabolic_k": base.get("metabolic_k", 4), "metabolic_threshold": base.get("metabolic_threshold", 0.1)}


def _l0(won: dict) -> dict[str, dict]:
    base = {**_SHARED, "metabolic_gate": False, "vocab_size": 256}
    return {"L0_bytes": {**base, "tokenizer_type": "none"},
            "L0_fixed_k512": {**base, **_VQ, "tokenizer_codebook_size": 512, "vocab_size": 512},
            "L0_fixed_k1024": {**base, **_VQ, "tokenizer_codebook_size": 1024, "vocab_size": 1024},
            "L0_bytes_tfm": {**base, "tokenizer_type": "none", "model_type": "transformer"}}


def _l05(won: dict) -> dict[str, dict]:
    if won.get("tokenizer", {}).get("tokenizer_type") != "fixed_stride":
        return {}                                   # alignment only means something for a learned tokenizer
    base = {**_SHARED, **won["tokenizer"], "metabolic_gate": False, **_WERNICKE}
    return {"L05_align_none": {**base, "align_type": "none"},
            **{f"L05_align_{n}": {**base, "align_type": t, "align_weight": 0.05}
               for n, t in (("contrastive", "contrastive"), ("diversity", "diversity"), ("distill", "distillation"))}}


def _l1(won: dict) -> dict[str, dict]:
    base = {**_SHARED, **won.get("tokenizer", {})}
    g = lambda mode, k, **kw: {**base, **_GATE, "metabolic_k": k, "metabolic_mode": mode, **kw}   # noqa: E731
    return {"L1_baseline_ssm": dict(base), "L1_baseline_tfm": {**base, "model_type": "transformer"},
            "L1_gate_fork_k4": g("fork", 4), "L1_gate_mc_k4": g("monte_carlo", 4),
            "L1_gate_mcts_k4": g("mcts", 4, mcts_horizon=8), "L1_gate_mcts_k8": g("mcts", 8, mcts_horizon=8),
            "L1_gate_random_k4": g("mcts", 4, mcts_horizon=8, metabolic_threshold_mode="random")}


def _l2(won: dict) -> dict[str, dict]:
    base = {**_SHARED, **won.get("tokenizer", {}), **won.get("gate", {})}
    both = {**_EPI, "semantic_tier_bases": 8}
    return {"L2_mem_none_cold": {**base, "eval_warmup": False},
            "L2_mem_epi_cold": {**base, **_EPI, "eval_warmup": False},
            "L2_mem_epi_warm": {**base, **_EPI, "eval_warmup": True},
            "L2_mem_both_cold": {**base, **both, "eval_warmup": False},
            "L2_mem_both_warm": {**base, **both, "eval_warmup": True},
            "L2_mem_both_warm_fullseq": {**base, **_BEST_MEM}}


def _l3(won: dict) -> dict[str, dict]:
    base = {**_SHARED, **won.get("tokenizer", {}), **won.get("gate", {}), **won.get("memory", {})}
    cfr = {**_WERNICKE, "cfr_enabled": True, "typed_storage": True, **_gate_passthrough(base)}
    return {"L3_no_wernicke": dict(base), "L3_wernicke": {**base, **_WERNICKE}, "L3_wernicke_cfr": {**base, **cfr},
            "L3_wernicke_cfr_consequence": {**base, **cfr, "compression_consequence": True}}


def _l35(won: dict) -> dict[str, dict]:
    tok = won.get("tokenizer", {})
    wc = {**_WERNICKE, "cfr_enabled": True, "typed_storage": True}
    g = lambda mode, **kw: {**_SHARED, **tok, **_GATE, "metabolic_k": 4, "metabolic_mode": mode, **kw}   # noqa: E731
    return {"L35_mcts_with_memory": {**g("mcts", mcts_horizon=8), **_BEST_MEM},
            "L35_fork_with_cfr": {**g("fork"), **wc, **won.get("memory", {})},
            "L35_full_stack_mc": {**g("monte_carlo"), **_BEST_MEM, **wc}}


def _full_stack(won: dict) -> dict:
    return {**_SHARED, **won.get("tokenizer", {}), **won.get("gate", {}), **won.get("memory", {}), **won.get("wernicke", {})}


def _l4(won: dict) -> dict[str, dict]:
    fs = _full_stack(won)
    tok = {k: v for k, v in won.get("tokenizer", {}).items()}
    return {**{f"L4_full_{d}": {**fs, "model_dim": d} for d in (128, 256, 384)},
            "L4_tfm_384": {"model_type": "transformer", "model_dim": 384, "num_layers": 4, "a_mode": "diag", **tok}}


def _l5(won: dict) -> dict[str, dict]:
    return {f"L5_full_{d}": {**_full_stack(won), "model_dim": d, "a_mode": "full"} for d in (128, 256, 384)}


def _l6(won: dict) -> dict[str, dict]:
    base = {**_full_stack(won), "eval_warmup": False}
    deep = {"eval_warmup": True, "warmup_write_mode": "full_sequence", "warmup_latent": True}
    return {"L6_wm_only": dict(base), "L6_wm_plus_episodic": {**base, "eval_warmup": True},
            "L6_wm_plus_all": {**base, **deep, "warmup_cold_start": True},
            "L6_wm_plus_all_seeded": {**base, **deep, "warmup_cold_start": False}}


@dataclass(frozen=True)
class Layer:
    tag: str
    title: str
    variants: Callable[[dict], dict[str, dict]]
    carries: Optional[str] = None         # which CARRY_KEYS group the winner hands on
    budget_scale: float = 1.0


LAYERS: tuple[Layer, ...] = (
    Layer("L0", "tokenizer architecture", _l0, "tokenizer"),
    Layer("L05", "codebook alignment", _l05, "tokenizer"),
    Layer("L1", "gate modes", _l1, "gate"),
    Layer("L2", "memory", _l2, "memory"),
    Layer("L3", "typed routing and regret", _l3, "wernicke"),
    Layer("L35", "dark horses", _l35),
    Layer("L4", "scaling", _l4),
    Layer("L5", "full state matrix", _l5, budget_scale=2.0),
    Layer("L6", "inference-time adaptation depth", _l6),
)


class LayeredStudy:
    """Run layers in order; each layer's winner injects its carried settings into the next ones.
    ``run_layer(configs, seeds) -> {name: {seed: bpb}}`` does the training (``launch.run_matrix`` in
    production, a stub in tests); progress is written after every layer so a crash resumes."""

    def __init__(self, run_layer: Callable[[dict[str, dict], Sequence[int], float], dict[str, dict[int, float]]],
                 *, seeds: Sequence[int] = SEEDS3, budget_seconds: float = 600.0,
                 state_path: Optional[Path] = None, layers: Sequence[Layer] = LAYERS) -> None:
        self.run_layer, self.seeds, self.budget, self.layers = run_layer, tuple(seeds), float(budget_seconds), layers
        self.state_path = Path(state_path) if state_path else None
        self.won: dict[str, dict] = {}
        self.report: dict[str, Any] = {}
        if self.state_path and self.state_path.exists():
            saved = json.loads(self.state_path.read_text())
            self.won, self.report = saved.get("won", {}), saved.get("report", {})

    def run(self, *, until: Optional[str] = None) -> dict[str, Any]:
        for layer in self.layers:
            if layer.tag in self.report:
                if until == layer.tag:
                    break
                continue
            cfgs = layer.variants(self.won)
            if not cfgs:
                self.report[layer.tag] = {"skipped": "not applicable to the earlier winners"}
            else:
                res = self.run_layer(cfgs, self.seeds, self.budget * layer.budget_scale)
                name, info = pick_winner({k: list(v.values()) for k, v in res.items()})
                self.report[layer.tag] = {"title": layer.title, "winner": name, **info,
                                          "means": {k: statistics.fmean(v.values()) for k, v in res.items() if v}}
                if name is not None and layer.carries:
                    keep = {k: cfgs[name][k] for k in CARRY_KEYS[layer.carries] if k in cfgs[name]}
                    self.won[layer.carries] = {**self.won.get(layer.carries, {}), **keep}
            if self.state_path:
                self.state_path.write_text(json.dumps({"won": self.won, "report": self.report}, indent=2, default=str))
            if until == layer.tag:
                break
        return self.report


# ---------------------------------------------------------------------------
# experiments 11-17: flat studies
# ---------------------------------------------------------------------------
def _byte_stack(**over: Any) -> dict:
    cfg = {"model_type": "ssm", "vocab_size": 256, "model_dim": 128, "num_layers": 4, "ff_mult": 2, "seq_len": 256,
           "stride": 128, "batch_size": 32, "base_lr": 2e-3}
    cfg.update(over)
    return cfg


_MEM_STACK = {"outer_model_type": "multislot", "outer_model_dim": 64, "outer_max_slots": 64,
              "consolidation_write": "full_sequence", "latent_persistence": True, **_WERNICKE, "typed_storage": True}
_SLEEP = {"sleep_interval": 256, "sleep_budget": 128, "sleep_n2_budget": 64, "sleep_rem_budget": 64}


def _sleep_base(**over: Any) -> dict:
    return {**_byte_stack(batch_size=64, eval_batches=32, a_mode="diag", weight_decay=1e-2, grad_clip_norm=1.0,
                          metabolic_gate=False, cfr_enabled=False, **_MEM_STACK), **over}


def _decide_sleep(conf: dict) -> str:
    r = conf.get("sleep_vs_none")
    if r is None:
        return "no data"
    if r["mean_delta"] < 0 and r["significant"]:
        return "ADOPT FULL CYCLE"
    if r["mean_delta"] < 0:
        return "CAUTIOUS ADOPTION"
    return "SLEEP NOT HELPFUL YET"


def _decide_polyphasic(conf: dict) -> str:
    vs_none, vs_off = conf.get("polyphasic_vs_none"), conf.get("polyphasic_vs_offline")
    if vs_none is None or vs_off is None:
        return "no data"
    helps = vs_none["mean_delta"] < 0 and vs_none["significant"]
    if not helps:
        return "POLYPHASIC NOT HELPFUL YET"
    worse_than_offline = vs_off["mean_delta"] > 0 and vs_off["significant"]
    return "POLYPHASIC HELPS BUT OFFLINE STILL BETTER" if worse_than_offline else "ADOPT POLYPHASIC"


_STAGES = ("n3_only", "n2_n3", "n2_n3_rem_base", "n2_n3_rem_validate", "n2_n3_rem_cfr", "n2_n3_rem_reactivate",
           "n2_n3_rem_all", "full_cycle")

SLEEP_CYCLE = Study(
    "exp11_sleep_cycle", "does structured offline consolidation improve bpb?",
    {"no_sleep": _sleep_base(sleep_enabled=False),
     **{s: _sleep_base(sleep_enabled=True, sleep_stages=s, **_SLEEP) for s in _STAGES}},
    confirmatory=(Contrast("sleep_vs_none", "no_sleep", "full_cycle", "does sleep help at all?"),
                  Contrast("n2_value", "n3_only", "n2_n3", "does N2 tagging add value?"),
                  Contrast("rem_value", "n2_n3", "n2_n3_rem_all", "does REM add value?")),
    exploratory=(Contrast("validate_vs_base", "n2_n3_rem_base", "n2_n3_rem_validate"),
                 Contrast("cfr_vs_base", "n2_n3_rem_base", "n2_n3_rem_cfr"),
                 Contrast("reactivate_vs_base", "n2_n3_rem_base", "n2_n3_rem_reactivate"),
                 Contrast("n1_value", "n2_n3_rem_all", "full_cycle")),
    decide=_decide_sleep)

POLYPHASIC = Study(
    "exp12_polyphasic_sleep", "does partition-scoped sleep match global offline consolidation?",
    {"no_sleep": _sleep_base(sleep_enabled=False, polyphasic_enabled=False),
     "full_offline_sleep": _sleep_base(sleep_enabled=True, polyphasic_enabled=False, sleep_stages="full_cycle", **_SLEEP),
     "polyphasic_K3_N4_striped": _sleep_base(sleep_enabled=True, polyphasic_enabled=True, polyphasic_n_partitions=4,
                                             polyphasic_k_awake=3, polyphasic_topology="slot_striped",
                                             sleep_stages="full_cycle", **_SLEEP)},
    confirmatory=(Contrast("polyphasic_vs_none", "no_sleep", "polyphasic_K3_N4_striped", "does polyphasic sleep help?"),
                  Contrast("polyphasic_vs_offline", "full_offline_sleep", "polyphasic_K3_N4_striped",
                           "is it competitive with a global pause?")),
    decide=_decide_polyphasic)


def _rate_tag(rate: float) -> str:
    return f"{rate:.0e}".replace(".", "").replace("+", "").replace("-", "m")


def _constants_conditions() -> dict[str, dict]:
    full = lambda **kw: {**_byte_stack(**_MEM_STACK), **kw}                                   # noqa: E731
    sleep = lambda **kw: full(sleep_enabled=True, sleep_stages="n3_only", **_SLEEP, **kw)     # noqa: E731
    c: dict[str, dict] = {}
    for v in (0.80, 0.85, 0.88, 0.92, 0.96):
        c[f"crit_{int(v * 100):03d}"] = _byte_stack(crit_target_coupling=v)
    for d in (32, 64, 128):
        c[f"memdim_{d:03d}"] = full(outer_model_dim=d)
    for n in (32, 64, 128):
        c[f"slots_{n:03d}"] = full(outer_max_slots=n)
    c["sem_off"] = full(semantic_tier_bases=0)
    for b in (4, 8, 16):
        for r in (0.001, 0.01, 0.1):
            c[f"sem_b{b}_r{_rate_tag(r)}"] = full(semantic_tier_bases=b, semantic_tier_update_rate=r)
    for t in (0.75, 0.80, 0.85, 0.90, 0.95):
        c[f"merge_{int(t * 100):03d}"] = sleep(sleep_merge_sim_threshold=t)
    return c


CONSTANTS = Study(
    "exp13_constants_validation", "exploratory sweeps of unvalidated constants", _constants_conditions(),
    exploratory=tuple(Contrast(f"{n}_vs_default", d, n) for d, names in (
        ("crit_092", ("crit_080", "crit_085", "crit_088", "crit_096")), ("memdim_064", ("memdim_032", "memdim_128")),
        ("slots_064", ("slots_032", "slots_128")), ("merge_085", ("merge_075", "merge_080", "merge_090", "merge_095")),
        ("sem_off", tuple(f"sem_b{b}_r{_rate_tag(r)}" for b in (4, 8, 16) for r in (0.001, 0.01, 0.1))))
        for n in names))


def _buffer_base(**over: Any) -> dict:
    return {**_byte_stack(a_mode="diag", crit_target_coupling=0.92, outer_model_type="multislot", outer_model_dim=64,
                          outer_max_slots=0, buffer_mode="append_only", **_WERNICKE), **over}


def expert_dim(n_experts: int, budget: int = 16 * 128) -> int:
    """Expert width that keeps the total routing parameter budget roughly constant."""
    return max(8, budget // n_experts)


_TOPK8 = {"retrieval_mode": "bucket_topk", "retrieval_k": 8}
_BARE = _byte_stack(a_mode="diag", crit_target_coupling=0.92, outer_model_dim=0, wernicke_enabled=False)
BUFFER_RETRIEVAL = Study(
    "exp14_T2_retrieval", "retrieval mode x capacity of the typed key-value buffer",
    {"softmax_all_32": _buffer_base(outer_max_slots=32, retrieval_mode="softmax_all", buffer_mode="legacy"),
     "softmax_all_uncapped": _buffer_base(retrieval_mode="softmax_all"),
     "mean_uncapped": _buffer_base(retrieval_mode="bucket_mean"),
     "recent_uncapped": _buffer_base(retrieval_mode="bucket_recent", retrieval_k=8),
     "topk_8k_8": _buffer_base(outer_max_slots=8192, **_TOPK8),
     **{f"topk_uncapped_{k}": _buffer_base(retrieval_mode="bucket_topk", retrieval_k=k) for k in (4, 8, 16)}})
BUFFER_ROUTING = Study(
    "exp14_T3_routing", "flat against hierarchical routing at a matched parameter budget",
    {**{f"flat_{k}": _buffer_base(wernicke_k_max=k, wernicke_expert_dim=expert_dim(k), **_TOPK8) for k in (8, 16, 64)},
     **{f"hier_8x{f}": _buffer_base(wernicke_layers=2, wernicke_k_max=8, wernicke_k_max_fine=f,
                                    wernicke_expert_dim=expert_dim(8 + f), **_TOPK8) for f in (8, 32)}})
BUFFER_COMPOSITION = Study(
    "exp14_T6_composition", "winners against the plain baselines",
    {"bare_ssm": dict(_BARE), "transformer": _byte_stack(model_type="transformer"),
     "mamba2": {k: v for k, v in _byte_stack(model_type="mamba2").items() if k != "ff_mult"}})


def _sp(dim: int, layers: int, vocab: int = 8192, **over: Any) -> dict:
    return {"model_type": "ssm", "vocab_size": vocab, "model_dim": dim, "num_layers": layers, "ff_mult": 2,
            "seq_len": 512, "stride": 256, "batch_size": 32, "base_lr": 2e-3, "a_mode": "diag",
            "crit_target_coupling": 0.92, **over}


SUBWORD_SHAPES = Study(
    "exp15_chaospiece", "sub-word vocabularies at several trunk shapes against the byte control",
    {**{f"sp_d{d}_L{l}": _sp(d, l) for d, l in ((128, 4), (192, 4), (128, 6), (192, 6), (256, 4))},
     "bare_ssm_byte256": _byte_stack(a_mode="diag", crit_target_coupling=0.92)})
VOCAB_VARIANTS = {4096: ("fineweb10B_sp4096", "fineweb_4096_bpe.model"), 8192: ("fineweb10B_sp8192", "fineweb_8192_bpe.model"),
                  16384: ("fineweb10B_sp16384", "fineweb_16384_bpe.model")}


def resolve_data_paths(data_root: str, vocab_size: int) -> tuple[str, str]:
    suffix, model = VOCAB_VARIANTS[vocab_size]
    return str(Path(data_root) / "datasets" / suffix), str(Path(data_root) / "tokenizers" / model)


def _oracle(**over: Any) -> dict:
    return {**_sp(256, 4, eval_batches=16, oracle_eval_batches=12, oracle_max_examples=4096, oracle_layer_index=3,
                  oracle_query_source="x_state", oracle_write_source="x_state", oracle_selector_epochs=10,
                  oracle_selector_batch_size=128, oracle_selector_lr=1e-3, sparse_attn_selector_dim=0), **over}


SPARSE_ATTENTION = Study(
    "exp16_entropy_sparse_attention", "how much would an oracle sparse-attention side buffer buy?",
    {**{f"oracle_buf{b}_k{k}": _oracle(sparse_attn_buffer_size=b, sparse_attn_k=k) for b in (64, 128) for k in (4, 8)},
     "oracle_buf128_k8_xonly": _oracle(sparse_attn_buffer_size=128, sparse_attn_k=8, oracle_query_source="x",
                                       oracle_write_source="x"),
     "oracle_buf128_k8_stateonly": _oracle(sparse_attn_buffer_size=128, sparse_attn_k=8, oracle_query_source="state",
                                           oracle_write_source="state")})


def _side(**over: Any) -> dict:
    return {**_sp(256, 4, eval_batches=16, local_attn_window=0, local_attn_heads=1, local_attn_dim=64), **over}


LOCAL_ATTENTION = Study(
    "exp17_local_attn_sidecar", "does a small local-attention side path pay for itself?",
    {"bare_fast_ssm": _side(),
     **{f"local_w{w}": _side(local_attn_window=w) for w in (16, 32, 64)},
     **{f"topk_{k}": _side(local_attn_window=64, local_attn_topk=k) for k in (8, 16, 32)},
     **{f"topk_random_{k}": _side(local_attn_window=64, local_attn_topk=k, local_attn_topk_random=True) for k in (8, 16, 32)}},
    exploratory=tuple(Contrast(f"{n}_vs_bare", "bare_fast_ssm", n) for n in
                      ("local_w16", "local_w32", "local_w64", "topk_8", "topk_16", "topk_32"))
    + tuple(Contrast(f"topk_{k}_vs_random", f"topk_random_{k}", f"topk_{k}", "does the selection matter, or only the compute?")
            for k in (8, 16, 32)))

# architecture baseline ablation (experiments/baselines/run_mamba2_baseline.py:57-110): external SSM vs this
# core vs typed routing vs the full stack, and the routing width sweep at a constant expert parameter budget
EXPERT_DIM_FOR_K = {16: 0, 32: 32, 64: 16}          # 0 = full-rank experts; k_max * 2 * expert_dim * 128 stays at 262 144


def _routed(k: int, **over: Any) -> dict:
    return _byte_stack(wernicke_enabled=True, wernicke_router="moe", wernicke_k_max=k, typed_storage=True,
                       wernicke_expert_dim=EXPERT_DIM_FOR_K.get(k, 0), **over)


def _routed_mem(k: int) -> dict:
    return _routed(k, outer_model_type="multislot", outer_model_dim=64, outer_max_slots=64,
                   consolidation_write="full_sequence", latent_persistence=True)


def _decide_architecture(conf: dict) -> str:
    full, core = conf.get("full_vs_mamba2"), conf.get("core_vs_mamba2")
    if full is None or core is None:
        return "no data"
    beats = lambda r: r["mean_delta"] < 0 and r["significant"]       # noqa: E731
    if beats(full):
        return "FULL STACK BEATS MAMBA-2" + (" (CORE ALONE TOO)" if beats(core) else "")
    return "CORE COMPETITIVE, STACK NOT AHEAD" if not (core["mean_delta"] > 0 and core["significant"]) else "MAMBA-2 AHEAD"


ARCHITECTURE_BASELINES = Study(
    "baselines_mamba2", "how much does each architectural layer contribute, against an external SSM?",
    {"mamba2": _byte_stack(model_type="mamba2"), "bare_ssm": _byte_stack(),
     "ssm_wernicke_k16": _routed(16), "full_stack_k16": _routed_mem(16),
     "ssm_wernicke_k32": _routed(32), "ssm_wernicke_k64": _routed(64),
     "full_stack_k32": _routed_mem(32), "full_stack_k64": _routed_mem(64)},
    confirmatory=(Contrast("full_vs_mamba2", "mamba2", "full_stack_k16", "does the full architecture beat Mamba-2?"),
                  Contrast("core_vs_mamba2", "mamba2", "bare_ssm", "is the SSM core competitive with Mamba-2?")),
    exploratory=(Contrast("wernicke_contribution", "bare_ssm", "ssm_wernicke_k16"),
                 Contrast("memory_contribution", "ssm_wernicke_k16", "full_stack_k16"),
                 Contrast("wernicke_k32", "ssm_wernicke_k16", "ssm_wernicke_k32"),
                 Contrast("wernicke_k64", "ssm_wernicke_k16", "ssm_wernicke_k64"),
                 Contrast("full_k32", "full_stack_k16", "full_stack_k32"),
                 Contrast("full_k64", "full_stack_k16", "full_stack_k64")),
    decide=_decide_architecture)

STUDIES: dict[str, Study] = {s.key: s for s in (SLEEP_CYCLE, POLYPHASIC, CONSTANTS, BUFFER_RETRIEVAL, BUFFER_ROUTING,
                                                BUFFER_COMPOSITION, SUBWORD_SHAPES, SPARSE_ATTENTION, LOCAL_ATTENTION,
                                                ARCHITECTURE_BASELINES)}


# ---------------------------------------------------------------------------
# experiment 10: scaling laws
# ---------------------------------------------------------------------------
SIZE_TABLE = {"XS": (64, 2), "S": (128, 4), "M": (256, 6), "L": (384, 8), "XL": (512, 10)}
BYTE_VOCAB = 256


def count_ssm_params(dim: int, layers: int, ff_mult: int = 2, vocab: int = BYTE_VOCAB) -> int:
    per_layer = 5 * dim * dim + dim + 2 * dim * dim * ff_mult + 2 * dim       # five projections + log_a, FF, two norms
    return 2 * vocab * dim + dim + layers * per_layer


def count_transformer_params(dim: int, layers: int, ff_mult: int = 2, vocab: int = BYTE_VOCAB) -> int:
    return 2 * vocab * dim + dim + layers * (4 * dim * dim + 2 * dim * dim * ff_mult + 2 * dim)


def match_transformer_to_ssm(dim: int, layers: int, ff_mult: int = 2, *, target_params: Optional[int] = None) -> dict:
    """Transformer (layers, ff_mult) at the same width whose parameter count is closest to the SSM's
    (first within 5 % wins, scanning ff_mult 2..4 and 1..19 layers)."""
    target = target_params if target_params is not None else count_ssm_params(dim, layers, ff_mult)
    best, err = None, float("inf")
    for ff in (2, 3, 4):
        for nl in range(1, 20):
            p = count_transformer_params(dim, nl, ff)
            e = abs(p - target) / target
            if e < err:
                best, err = {"num_layers": nl, "ff_mult": ff, "param_count": p}, e
            if e < 0.05:
                return best
    return best


def estimate_flops_per_step(model_type: str, dim: int, layers: int, ff_mult: int, seq_len: int, batch: int, *,
                            wernicke_enabled: bool = False, wernicke_k_max: int = 16, outer_model_dim: int = 0,
                            outer_max_slots: int = 64, metabolic_gate: bool = False, metabolic_k: int = 4) -> int:
    """6 x parameters x tokens, plus the attention quadratic term and the mechanisms' own cost."""
    tokens = batch * seq_len
    if model_type == "transformer":
        per_layer = 4 * dim * dim + 2 * dim * dim * ff_mult
        extra = 2 * layers * 2 * seq_len * seq_len * dim * batch
    elif model_type == "mamba2":
        inner = 2 * dim
        per_layer, extra = 2 * dim * inner + inner * 64 + inner, 0
    else:
        per_layer, extra = 5 * dim * dim + 2 * dim * dim * ff_mult, 0
    flops = 6 * (layers * per_layer + 2 * BYTE_VOCAB * dim) * tokens + extra
    if wernicke_enabled:
        flops += 6 * 2 * dim * wernicke_k_max * tokens
    if outer_model_dim > 0:
        flops += 6 * 2 * dim * outer_max_slots * tokens
    if metabolic_gate:
        flops += metabolic_k * per_layer * tokens
    return int(flops)


def scaling_configs(*, full_stack: Optional[dict] = None, include_mamba2: bool = False) -> dict[str, dict]:
    """``<condition>_<size>`` for bare_ssm / full_ssm (the experiment-09 winners on top) / our_tfm (parameter
    matched) / mamba2_ssm over the five sizes."""
    out: dict[str, dict] = {}
    for tag, (d, nl) in SIZE_TABLE.items():
        bare = {"model_type": "ssm", "model_dim": d, "num_layers": nl, "ff_mult": 2, "a_mode": "diag", "vocab_size": BYTE_VOCAB}
        out[f"bare_ssm_{tag}"] = bare
        if full_stack:
            out[f"full_ssm_{tag}"] = {**bare, **{k: v for k, v in full_stack.items() if k not in ("model_dim", "num_layers")}}
        m = match_transformer_to_ssm(d, nl)
        out[f"our_tfm_{tag}"] = {"model_type": "transformer", "model_dim": d, "num_layers": m["num_layers"],
                                 "ff_mult": m["ff_mult"], "vocab_size": BYTE_VOCAB}
        if include_mamba2:
            out[f"mamba2_ssm_{tag}"] = {"model_type": "mamba2", "model_dim": d, "num_layers": nl, "vocab_size": BYTE_VOCAB}
    return out


def scaling_table(results_dir: Path, configs: dict[str, dict]) -> dict[str, Any]:
    """Per condition family: (parameters, mean bpb) points and the fitted ``bpb = A N^-alpha + bpb_irr``."""
    from .analysis import fit_power_law
    data = load_metric(results_dir, list(configs))
    fam: dict[str, list[tuple[int, float]]] = {}
    for name, by_seed in data.items():
        cfg = configs[name]
        family = name.rsplit("_", 1)[0]
        n = (count_transformer_params if cfg["model_type"] == "transformer" else count_ssm_params)(
            cfg["model_dim"], cfg["num_layers"], cfg.get("ff_mult", 2))
        fam.setdefault(family, []).append((n, statistics.fmean(by_seed.values())))
    out = {}
    for f, pts in fam.items():
        pts.sort()
        out[f] = {"points": pts, "fit": fit_power_law([p for p, _ in pts], [b for _, b in pts]) if len(pts) >= 3 else None}
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="matrix entries or analysis of one study")
    ap.add_argument("study", choices=sorted(STUDIES) + ["exp09_layers", "exp10_scaling"])
    ap.add_argument("--results-dir", type=Path, default=None, help="analyse result files instead of printing the matrix")
    a = ap.parse_args(argv)
    if a.study == "exp09_layers":
        print(json.dumps({l.tag: sorted(l.variants({"tokenizer": {"tokenizer_type": "fixed_stride"}})) for l in LAYERS}, indent=2))
    elif a.study == "exp10_scaling":
        cfgs = scaling_configs()
        print(json.dumps(scaling_table(a.results_dir, cfgs) if a.results_dir else cfgs, indent=2, default=str))
    elif a.results_dir:
        print(json.dumps(analyse(STUDIES[a.study], a.results_dir), indent=2, default=str))
    else:
        print(json.dumps(entries(STUDIES[a.study]), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
