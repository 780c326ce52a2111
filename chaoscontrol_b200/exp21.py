"""Embedding-prior study (experiment 21): run families, slot launcher, verdict report, registry import.

Reference: experiments/21_sgns_tokenizer/runner_phase0.py:34-107 (transformer rate screen),
runner_4cell.py:35-186 (SSM x transformer x {random, SGNS}), runner_controls.py:47-140 (full-covariance,
shuffled-row and all-zero controls on the SSM arm), runner_exp21b.py:43-152 (six mechanism cells),
scripts/exp21_analyze.py:54-330 (paired one-sided tests and the thesis verdict),
scripts/exp21_register_all.py:33-170 (bulk import into the results registry).

Here the four orchestrators are one table of :class:`Family` values -- conditions, seeds and result
folder -- driven by one launcher.  The launcher keeps ``num_slots`` data-parallel groups of
``ws_per_slot`` GPUs busy at once (each group is a ``torch.distributed.run`` of
``chaoscontrol_b200.runner_exp21`` pinned to its GPUs through ``CUDA_VISIBLE_DEVICES``), skips runs
whose result file exists, and leaves ``{"config", "error"}`` in place of a failed run so the rest of
the family still runs.  Result files are ``<family dir>/<condition>_s<seed>.json``.

Verdict: primary ``delta_SSM = bpb(C) - bpb(D) > 0`` and secondary ``delta_SSM > delta_Trans``, both
one-sided paired t-tests at p < 0.01 on the seeds that all four cells finished; *validating* also
needs both the full-covariance and the shuffled control to be worse than the mean/std-matched SGNS
arm at p < 0.01.  Runs flagged non-finite by the trainer are dropped from every test.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import queue
import re
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Iterable, Optional, Sequence

from .analysis import paired_ttest

MAIN_SEEDS = (1337, 42, 123, 7, 8)
SSM_LR = 0.064                      # rate of the 2-GPU x 1024-sequence screen that this study inherits
PHASE0_LRS = (0.016, 0.032, 0.064)
SGNS_INIT = "artifacts/sgns_init_meanstd.pt"
ALPHA = 0.01

MECHANISM_ARTIFACTS = {
    "ssm_norm_only": "artifacts/sgns_init_norm_only.pt",                         # random directions, SGNS row norms
    "ssm_norm_only_shuffled": "artifacts/sgns_init_norm_only_shuffled.pt",       # ... norms permuted
    "ssm_freq_bucket_shuffle": "artifacts/sgns_init_freq_bucket_shuffle.pt",     # rows permuted within frequency buckets
    "ssm_class_bucket_shuffle": "artifacts/sgns_init_class_bucket_shuffle.pt",   # ... within coarse token classes
    "ssm_fullcov_shuffled": "artifacts/sgns_init_fullcov_shuffled.pt",           # full-cov control, rows permuted
    "ssm_random_fullcov": "artifacts/sgns_init_random_fullcov.pt",               # Gaussian cloud with the same mean / cov
}


def shared_axes() -> dict[str, Any]:
    return {"vocab_size": 8192, "seq_len": 512, "stride": 256, "batch_size": 1024, "eval_batches": 16,
            "optimizer": "muon", "weight_decay": 1e-2, "grad_clip_norm": 1.0, "chunk_size": 64, "dtype": "bf16",
            "precision": "bf16", "activation_checkpoint": True}


def transformer_cell(*, base_lr: float, embed_init_path: Optional[str]) -> dict[str, Any]:
    return dict(shared_axes(), model_type="transformer_nanogpt_lean", model_dim=256, num_layers=8, n_head=4, ff_mult=4,
                base_lr=float(base_lr), embed_init_path=embed_init_path)


def ssm_cell(*, base_lr: float = SSM_LR, embed_init_path: Optional[str], **over: Any) -> dict[str, Any]:
    return dict(shared_axes(), model_type="ssm", model_dim=256, num_layers=4, ff_mult=2, a_mode="diag", a_full_rank=8,
                a_full_gamma=0.05, base_lr=float(base_lr), embed_init_path=embed_init_path, local_attn_window=0,
                local_attn_heads=1, local_attn_dim=64, **over)


@dataclass(frozen=True)
class Family:
    key: str
    subdir: str
    conditions: dict[str, dict[str, Any]]
    seeds: tuple[int, ...] = MAIN_SEEDS
    summary_name: str = "summary.json"

    def entries(self, *, budget_seconds: Optional[float] = None, world_size: int = 2) -> list[dict[str, Any]]:
        out = []
        for cond, cfg in self.conditions.items():
            for seed in self.seeds:
                e = dict(cfg, name=f"{cond}_s{seed}", condition=cond, seed=int(seed), world_size=int(world_size))
                if budget_seconds is not None:
                    e["budget_seconds"] = float(budget_seconds)
                out.append(e)
        return out


def lr_tag(lr: float) -> str:
    return f"lr_{lr:.3f}".replace(".", "p")


def phase0_family() -> Family:
    """Three rates x one seed on the transformer arm; the lowest bpb becomes the arm's rate."""
    return Family("phase0", "phase0", {lr_tag(lr): transformer_cell(base_lr=lr, embed_init_path=None)
                                      for lr in PHASE0_LRS}, seeds=(1337,), summary_name="phase0_summary.json")


def four_cell_family(transformer_lr: float) -> Family:
    return Family("four_cell", "four_cell", {
        "A_transformer_random": transformer_cell(base_lr=transformer_lr, embed_init_path=None),
        "B_transformer_sgns": transformer_cell(base_lr=transformer_lr, embed_init_path=SGNS_INIT),
        "C_ssm_random": ssm_cell(embed_init_path=None),
        "D_ssm_sgns": ssm_cell(embed_init_path=SGNS_INIT)}, summary_name="four_cell_summary.json")


def control_families() -> list[Family]:
    """Stronger nulls on the SSM arm.  The all-zero table may diverge (every token starts identical); its
    cell tolerates non-finite training so the divergence is kept as a data point."""
    return [Family("fullcov", "fullcov", {"ssm_fullcov": ssm_cell(embed_init_path="artifacts/sgns_init_fullcov.pt")}),
            Family("shuffled", "shuffled", {"ssm_shuffled": ssm_cell(embed_init_path="artifacts/sgns_init_shuffled.pt")}),
            Family("zero", "zero", {"ssm_zero": ssm_cell(embed_init_path="artifacts/sgns_init_zero.pt",
                                                          allow_nonfinite=True)})]


def mechanism_family(selected: Optional[Iterable[str]] = None) -> Family:
    names = list(MECHANISM_ARTIFACTS) if selected is None else list(selected)
    unknown = [n for n in names if n not in MECHANISM_ARTIFACTS]
    if unknown:
        raise ValueError(f"unknown mechanism condition(s): {unknown}; valid: {', '.join(MECHANISM_ARTIFACTS)}")
    return Family("exp21b", "exp21b_mechanisms", {n: ssm_cell(embed_init_path=MECHANISM_ARTIFACTS[n]) for n in names},
                  summary_name="exp21b_summary.json")


def parse_condition_names(raw: Optional[str]) -> Optional[list[str]]:
    names = [n.strip() for n in (raw or "").split(",") if n.strip()]
    return names or None


def validate_embed_artifacts(conditions: dict[str, dict[str, Any]], root: Path) -> None:
    """Every referenced table exists under ``root`` and is ``[vocab, dim]``."""
    import torch
    missing, bad = [], []
    for name, cfg in conditions.items():
        rel = cfg.get("embed_init_path")
        if rel is None:
            continue
        path = Path(root) / str(rel)
        if not path.is_file():
            missing.append(f"{name}: {rel}")
            continue
        got = tuple(torch.load(path, map_location="cpu").shape)
        want = (int(cfg["vocab_size"]), int(cfg["model_dim"]))
        if got != want:
            bad.append(f"{name}: {rel} is {got}, expected {want}")
    if missing:
        raise FileNotFoundError("missing embedding tables (python -m chaoscontrol_b200.sgns.cli prepare-inits writes "
                                "them; or select the conditions that exist):\n  " + "\n  ".join(missing))
    if bad:
        raise ValueError("embedding tables of the wrong shape:\n  " + "\n  ".join(bad))


# ---------------------------------------------------------------------------
# launcher: num_slots data-parallel groups at a time
# ---------------------------------------------------------------------------
def slot_gpus(num_slots: int, ws_per_slot: int) -> list[str]:
    return [",".join(str(s * ws_per_slot + i) for i in range(ws_per_slot)) for s in range(num_slots)]


def run_family(family: Family, *, results_root: Path, data_path: str, sp_model_path: str, budget_seconds: float = 600.0,
               num_slots: int = 2, ws_per_slot: int = 2, dry_run: bool = False, artifact_root: Optional[Path] = None,
               runner: Callable[..., Any] = subprocess.run) -> dict[str, Any]:
    from .launch import build_torchrun_cmd, write_entry_config
    rdir = Path(results_root) / family.subdir
    entries = family.entries(budget_seconds=budget_seconds, world_size=ws_per_slot)
    todo = [e for e in entries if not (rdir / f"{e['name']}.json").exists()]
    plan = {"family": family.key, "skipped": [e["name"] for e in entries if e not in todo], "commands": [], "failed": []}
    if not dry_run:
        if artifact_root is not None:
            validate_embed_artifacts(family.conditions, artifact_root)
        rdir.mkdir(parents=True, exist_ok=True)
    free: "queue.Queue[str]" = queue.Queue()
    for g in slot_gpus(num_slots, ws_per_slot):
        free.put(g)
    lock = threading.Lock()

    def one(e: dict[str, Any]) -> None:
        out = rdir / f"{e['name']}.json"
        gpus = free.get()
        try:
            cfg_path = (rdir / "configs" / f"{e['name']}.yaml") if dry_run else write_entry_config(e, rdir / "configs")
            cmd = build_torchrun_cmd(runner_path="chaoscontrol_b200.runner_exp21", config_path=cfg_path,
                                     data_path=data_path, sp_model_path=sp_model_path, output_json=out,
                                     world_size=ws_per_slot, budget_seconds=budget_seconds, dry_run=dry_run)
            with lock:
                plan["commands"].append({"name": e["name"], "gpus": gpus, "cmd": cmd})
            if dry_run:
                return
            proc = runner(cmd, env=dict(os.environ, CUDA_VISIBLE_DEVICES=gpus), capture_output=True, text=True)
            if proc.returncode != 0 and not out.exists():
                out.write_text(json.dumps({"config": e, "error": str(proc.stderr)[-2000:]}, indent=2, default=str))
                with lock:
                    plan["failed"].append(e["name"])
        finally:
            free.put(gpus)

    if dry_run:
        for e in todo:
            one(e)
    elif todo:
        with ThreadPoolExecutor(max_workers=num_slots) as pool:
            list(pool.map(one, todo))
    return plan


# ---------------------------------------------------------------------------
# results
# ---------------------------------------------------------------------------
def _pattern(cell: str) -> "re.Pattern[str]":
    return re.compile(rf"^{re.escape(cell)}_s(\d+)\.json$")


def collect(results_dir: Path, cell: str) -> dict[int, float]:
    """``{seed: bpb}`` as written (NaN where there is no eval block) -- the orchestrators' raw view."""
    out: dict[int, float] = {}
    if not Path(results_dir).exists():
        return out
    pat = _pattern(cell)
    for f in sorted(Path(results_dir).iterdir()):
        m = pat.match(f.name)
        if m:
            data = json.loads(f.read_text())
            ev = data.get("eval") or {}
            out[int(m.group(1))] = float(ev.get("bpb", float("nan"))) if ev else float("nan")
    return out


def summarize_family(family: Family, results_root: Path) -> dict[str, Any]:
    rdir = Path(results_root) / family.subdir
    per = {c: collect(rdir, c) for c in family.conditions}
    rows = {}
    for c, by in per.items():
        finite = [v for v in by.values() if math.isfinite(v)]
        rows[c] = {"n": len(by), "finite": len(finite), "mean_bpb": sum(finite) / len(finite) if finite else float("nan"),
                   "seeds": sorted(by)}
    return {"family": family.key, "seeds": list(family.seeds), "per_cell": per, "rows": rows,
            "artifact_paths": {c: cfg.get("embed_init_path") for c, cfg in family.conditions.items()}}


def phase0_summary(results_root: Path) -> dict[str, Any]:
    fam = phase0_family()
    rdir = Path(results_root) / fam.subdir
    rows = []
    for cond, cfg in fam.conditions.items():
        pat = _pattern(cond)
        for f in sorted(rdir.iterdir()) if rdir.exists() else []:
            m = pat.match(f.name)
            if not m:
                continue
            data = json.loads(f.read_text())
            ev = data.get("eval") or {}
            rows.append({"name": cond, "seed": int(m.group(1)), "base_lr": cfg["base_lr"],
                         "bpb": float(ev.get("bpb", float("nan"))) if ev else float("nan"),
                         "final_loss": float((data.get("train") or {}).get("final_loss", float("nan")))})
    rows.sort(key=lambda r: r["bpb"] if math.isfinite(r["bpb"]) else float("inf"))
    ok = bool(rows) and math.isfinite(rows[0]["bpb"])
    return {"rows": rows, "winner_condition": rows[0]["name"] if ok else None,
            "winner_lr": rows[0]["base_lr"] if ok else None}


def load_transformer_lr(results_root: Path, override: Optional[float] = None) -> float:
    if override is not None:
        return float(override)
    p = Path(results_root) / "phase0" / "phase0_summary.json"
    if not p.exists():
        raise FileNotFoundError(f"{p} not found: run the phase0 family first or pass the transformer rate")
    lr = json.loads(p.read_text()).get("winner_lr")
    if lr is None:
        raise ValueError(f"{p} has no winner_lr: rerun phase0 or pass the transformer rate")
    return float(lr)


# ---------------------------------------------------------------------------
# verdict
# ---------------------------------------------------------------------------
def paired_t_one_sided(x: Sequence[float], y: Sequence[float], alternative: str = "greater") -> float:
    """p-value of the paired t-test with H1 ``mean(x) > mean(y)`` ("greater") or ``<`` ("less")."""
    if alternative not in ("greater", "less"):
        raise ValueError(f"alternative must be 'greater' or 'less', got {alternative!r}")
    if len(x) != len(y):
        raise ValueError(f"paired inputs must have equal length; got {len(x)} and {len(y)}")
    if len(x) < 2:
        raise ValueError(f"need at least 2 paired observations, got {len(x)}")
    t, p2 = paired_ttest(list(x), list(y))
    if math.isnan(t) or math.isnan(p2) or (t == 0.0 and p2 == 1.0):
        return 0.5
    if math.isinf(t):                                  # identical non-zero differences: certain either way
        return 0.0 if (t > 0) == (alternative == "greater") else 1.0
    hit = t > 0 if alternative == "greater" else t < 0
    return p2 / 2.0 if hit else 1.0 - p2 / 2.0


def load_cell_bpbs(results_dir: Path, cell: str, *, warn: Callable[[str], None] = print) -> dict[int, float]:
    """``{seed: bpb}`` of the runs that may enter a test: readable, not flagged non-finite, finite bpb."""
    out: dict[int, float] = {}
    if not Path(results_dir).exists():
        return out
    pat = _pattern(cell)
    for f in sorted(Path(results_dir).iterdir()):
        m = pat.match(f.name)
        if not m:
            continue
        try:
            data = json.loads(f.read_text())
        except (OSError, json.JSONDecodeError) as exc:
            warn(f"  warn: could not read {f.name}: {exc}")
            continue
        nf = data.get("nonfinite") or {}
        if nf.get("flag"):                             # even when the final bpb happens to be finite
            warn(f"  warn: {f.name} is flagged non-finite ({nf.get('reason', 'unspecified')}); skipping")
            continue
        bpb = (data.get("eval") or {}).get("bpb")
        if bpb is None or not math.isfinite(float(bpb)):
            warn(f"  warn: {f.name} has no finite eval.bpb; skipping")
            continue
        out[int(m.group(1))] = float(bpb)
    return out


def _stats(v: Sequence[float]) -> dict[str, Any]:
    n = len(v)
    if n == 0:
        return {"n": 0, "mean": float("nan"), "std": float("nan")}
    mean = sum(v) / n
    return {"n": n, "mean": mean, "std": math.sqrt(sum((x - mean) ** 2 for x in v) / (n - 1)) if n > 1 else 0.0}


def _paired_p(worse: dict[int, float], better: dict[int, float]) -> tuple[Optional[float], int]:
    shared = sorted(set(worse) & set(better))
    if len(shared) < 2:
        return None, len(shared)
    return paired_t_one_sided([worse[s] for s in shared], [better[s] for s in shared], "greater"), len(shared)


def build_report(results_root: Path, *, warn: Callable[[str], None] = print) -> dict[str, Any]:
    root = Path(results_root)
    four = {c: load_cell_bpbs(root / "four_cell", c, warn=warn)
            for c in ("A_transformer_random", "B_transformer_sgns", "C_ssm_random", "D_ssm_sgns")}
    A, B, C, D = four.values()
    common = sorted(set(A) & set(B) & set(C) & set(D))        # one seed set for both tests and both means
    d_ssm = [C[s] - D[s] for s in common]
    d_tr = [A[s] - B[s] for s in common]
    p_primary = paired_t_one_sided([C[s] for s in common], [D[s] for s in common]) if len(common) >= 2 else None
    p_secondary = paired_t_one_sided(d_ssm, d_tr) if len(common) >= 2 else None
    fullcov = load_cell_bpbs(root / "fullcov", "ssm_fullcov", warn=warn)
    shuffled = load_cell_bpbs(root / "shuffled", "ssm_shuffled", warn=warn)
    zero = load_cell_bpbs(root / "zero", "ssm_zero", warn=warn)
    p_fc, n_fc = _paired_p(fullcov, D)
    p_sh, n_sh = _paired_p(shuffled, D)
    p_zero, n_zero = _paired_p(zero, C)
    complete = n_fc >= 2 and n_sh >= 2
    support = p_fc is not None and p_fc < ALPHA and p_sh is not None and p_sh < ALPHA
    validating = (p_primary is not None and p_secondary is not None and p_primary < ALPHA and p_secondary < ALPHA
                  and complete and support)
    mean = lambda v: sum(v) / len(v) if v else float("nan")                                   # noqa: E731
    return {"cells": {c: _stats(list(v.values())) for c, v in four.items()}, "n_common_seeds": len(common),
            "n_ssm_pairs": len(common), "n_trans_pairs": len(common), "n_common_seeds_for_secondary": len(common),
            "delta_ssm_mean": mean(d_ssm), "delta_trans_mean": mean(d_tr), "p_primary": p_primary,
            "p_secondary": p_secondary, "thesis_validating": validating,
            "thesis_weak": p_primary is not None and p_primary < ALPHA and not validating,
            "fullcov": _stats(list(fullcov.values())), "shuffled": _stats(list(shuffled.values())),
            "zero": _stats(list(zero.values())), "p_fullcov_vs_meanstd": p_fc, "n_fullcov_pairs": n_fc,
            "p_shuffled_vs_meanstd": p_sh, "n_shuffled_pairs": n_sh, "p_zero_vs_random": p_zero, "n_zero_pairs": n_zero,
            "controls_complete": complete, "controls_support_semantics": support}


def _fmt_p(p: Optional[float]) -> str:
    return "n/a (insufficient data)" if p is None else f"{p:.2e}" if p < 1e-4 else f"{p:.4f}"


def format_report(r: dict[str, Any]) -> str:
    def cell(label: str, s: dict) -> str:
        return (f"  {label:<28} n=0  (no runs found)" if not s["n"]
                else f"  {label:<28} n={s['n']}  mean={s['mean']:.4f}  std={s['std']:.4f}")
    n = r["n_common_seeds"]
    lines = ["== embedding-prior study ==",
             cell("A transformer x random", r["cells"]["A_transformer_random"]),
             cell("B transformer x SGNS", r["cells"]["B_transformer_sgns"]),
             cell("C SSM x random", r["cells"]["C_ssm_random"]), cell("D SSM x SGNS", r["cells"]["D_ssm_sgns"]), "",
             f"  delta_SSM   = C - D (mean over {n} common seeds): {r['delta_ssm_mean']:+.4f}",
             f"  delta_Trans = A - B (mean over {n} common seeds): {r['delta_trans_mean']:+.4f}", "",
             f"  primary   (delta_SSM > 0)            p = {_fmt_p(r['p_primary'])}",
             f"  secondary (delta_SSM > delta_Trans)  p = {_fmt_p(r['p_secondary'])}", "",
             f"  thesis-validating: {r['thesis_validating']}", f"  thesis-weak:       {r['thesis_weak']}"]
    if r["fullcov"]["n"] or r["shuffled"]["n"] or r["zero"]["n"]:
        lines += ["", "== controls =="]
        if r["fullcov"]["n"]:
            lines += [cell("SSM x SGNS (full-cov)", r["fullcov"]),
                      f"  full-cov worse than mean/std ({r['n_fullcov_pairs']} seeds): p = {_fmt_p(r['p_fullcov_vs_meanstd'])}"]
        if r["shuffled"]["n"]:
            lines += [cell("SSM x SGNS (shuffled rows)", r["shuffled"]),
                      f"  shuffled worse than mean/std ({r['n_shuffled_pairs']} seeds): p = {_fmt_p(r['p_shuffled_vs_meanstd'])}"]
        if r["zero"]["n"]:
            lines += [cell("SSM x all-zero table", r["zero"]),
                      f"  zero worse than random ({r['n_zero_pairs']} seeds): p = {_fmt_p(r['p_zero_vs_random'])}"]
        lines += [f"  controls-complete:          {r['controls_complete']}",
                  f"  controls-support-semantics: {r['controls_support_semantics']}"]
    return "\n".join(lines)


# ---------------------------------------------------------------------------
# registry import
# ---------------------------------------------------------------------------
REGISTERED_DIRS = ("four_cell", "fullcov", "shuffled", "zero")
REGISTERED_CONDITIONS = {"A_transformer_random", "B_transformer_sgns", "C_ssm_random", "D_ssm_sgns", "ssm_fullcov",
                         "ssm_shuffled", "ssm_zero"}
_FILE_RE = re.compile(r"^(?P<cell>[A-Za-z0-9_]+?)_s(?P<seed>\d+)\.json$")


def config_hash(config: dict) -> str:
    return "sha256:" + hashlib.sha256(json.dumps(config, sort_keys=True).encode()).hexdigest()


def discover_results(results_root: Path) -> list[tuple[str, int, Path]]:
    found = []
    for sub in REGISTERED_DIRS:
        d = Path(results_root) / sub
        for p in sorted(d.iterdir()) if d.is_dir() else []:
            m = _FILE_RE.match(p.name)
            if m and m.group("cell") in REGISTERED_CONDITIONS:
                found.append((m.group("cell"), int(m.group("seed")), p))
    return sorted(found)


def register_all(results_root: Path, *, status: str = "confirmatory", registry_path=None, canonical_path=None,
                 say: Callable[[str], None] = print) -> int:
    """One registry record per (cell, seed).  A confirmatory import takes only configs declared canonical
    for that very cell.  Returns 0, 1 (nothing found) or 2 (everything was refused)."""
    from .paper_results import is_canonical, register
    records = discover_results(results_root)
    if not records:
        say(f"no result files under {results_root}")
        return 1
    done, refused = 0, 0
    for cell, seed, path in records:
        data = json.loads(path.read_text())
        ev, tr = data.get("eval") or {}, data.get("train") or {}
        metrics = {"bpb": float(ev.get("bpb", float("nan"))), "wall_clock_s": float(tr.get("elapsed_s", float("nan"))),
                   "final_loss": float(tr.get("final_loss", float("nan")))}
        if (data.get("nonfinite") or {}).get("flag"):
            metrics["nonfinite_flag"] = 1.0
        h = config_hash(data.get("config", {}))
        if status == "confirmatory" and not is_canonical(config_hash=h, experiment="exp21", condition=cell,
                                                         path=canonical_path):
            refused += 1
            say(f"  SKIP exp21/{cell} seed={seed} {h}: not declared canonical (declare it with its rationale, "
                "or import as exploratory)")
            continue
        rec = register(experiment="exp21", condition=cell, seed=seed, status=status, metrics=metrics, config_hash=h,
                       artifacts=[str(path)], registry_path=registry_path)
        done += 1
        say(f"  exp21/{cell} seed={seed} bpb={metrics['bpb']:.4f}" + (" [NONFINITE]" if "nonfinite_flag" in metrics else "")
            + f" dirty={rec.git_dirty}")
    if refused:
        say(f"refused {refused}, registered {done} as {status}")
        return 2 if done == 0 else 0
    return 0


# ---------------------------------------------------------------------------
def _families(key: str, results_root: Path, transformer_lr: Optional[float], conditions: Optional[str]) -> list[Family]:
    if key == "phase0":
        return [phase0_family()]
    if key == "four_cell":
        return [four_cell_family(load_transformer_lr(results_root, transformer_lr))]
    if key == "controls":
        return control_families()
    if key == "exp21b":
        return [mechanism_family(parse_condition_names(conditions))]
    raise ValueError(key)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("family", choices=("phase0", "four_cell", "controls", "exp21b"))
    r.add_argument("--results-root", type=Path, required=True)
    r.add_argument("--data-path", required=True)
    r.add_argument("--sp-model-path", required=True)
    r.add_argument("--budget", type=float, default=600.0)
    r.add_argument("--num-slots", type=int, default=2)
    r.add_argument("--transformer-lr", type=float, default=None)
    r.add_argument("--conditions", default=None)
    r.add_argument("--artifact-root", type=Path, default=Path.cwd())
    r.add_argument("--summarize-only", action="store_true")
    r.add_argument("--dry-run", action="store_true")
    a_ = sub.add_parser("analyze")
    a_.add_argument("--results-root", type=Path, required=True)
    a_.add_argument("--json-out", type=Path, default=None)
    g = sub.add_parser("register")
    g.add_argument("--results-root", type=Path, required=True)
    g.add_argument("--status", choices=("confirmatory", "exploratory"), default="confirmatory")
    g.add_argument("--registry", default=None)
    a = ap.parse_args(argv)
    if a.cmd == "analyze":
        rep = build_report(a.results_root)
        print(format_report(rep))
        if a.json_out is not None:
            a.json_out.parent.mkdir(parents=True, exist_ok=True)
            a.json_out.write_text(json.dumps(rep, indent=2, default=str))
        return 0
    if a.cmd == "register":
        return register_all(a.results_root, status=a.status, registry_path=a.registry)
    for fam in _families(a.family, a.results_root, a.transformer_lr, a.conditions):
        if not a.summarize_only:
            plan = run_family(fam, results_root=a.results_root, data_path=a.data_path, sp_model_path=a.sp_model_path,
                              budget_seconds=a.budget, num_slots=a.num_slots, dry_run=a.dry_run,
                              artifact_root=a.artifact_root)
            if a.dry_run:
                for c in plan["commands"]:
                    print(f"CUDA_VISIBLE_DEVICES={c['gpus']} " + " ".join(c["cmd"]))
                continue
        summary = phase0_summary(a.results_root) if fam.key == "phase0" else summarize_family(fam, a.results_root)
        out = Path(a.results_root) / fam.subdir
        out.mkdir(parents=True, exist_ok=True)
        (out / fam.summary_name).write_text(json.dumps(summary, indent=2, default=str))
        print(json.dumps(summary.get("rows", summary), indent=2, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
