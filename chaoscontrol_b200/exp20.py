"""Test-time-training ablation (experiment 20): config matrix and GPU job queue.

Reference: experiments/20_ssm_native_ttt/build_matrix.py:38-213 (first-wave matrix) and
run_queue.py:22-140 (one config per free GPU, resumable).  Three phases:

* ``floor``  -- score-only timing under ``reset`` and ``carry_state`` persistence (this is the
  score floor that the budget of the adaptation runs is charged against);
* ``axis1``  -- which parameters to adapt (``log_a``, ``delta_proj``, both, B side, C side,
  ``lm_head``) x evaluation learning rate, at the chosen persistence mode;
* ``axis3``  -- no-gradient modulation: scale of the delta projection, shift of ``log_a``.

``adapt_set="all"`` is refused: it is an envelope check, not a hypothesis of the experiment.
Every config is one JSON file the evaluation driver takes (``python -m
chaoscontrol_b200.eval_stream.run_eval --config <file>``); ``run_queue`` hands each pending file
to the next free GPU (``CUDA_VISIBLE_DEVICES``), skips those whose summary exists when resuming,
and logs each run to its own file.  On a GPU the driver itself picks the batched score-then-adapt
runner for the ``log_a`` / ``delta_proj`` adapt sets.
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import subprocess
import sys
from collections import Counter
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable, Optional, Sequence

DEFAULT_SEEDS = (0, 1, 2)
DEFAULT_AXIS1_ADAPT_SETS = ("log_a", "delta_proj", "log_a+delta_proj", "B_side", "C_side", "lm_head")
DEFAULT_AXIS1_EVAL_LRS = (0.016, 0.064)
DEFAULT_DELTA_SCALES = (0.5, 1.0, 2.0)
DEFAULT_LOG_A_SHIFTS = (-0.5, 0.0, 0.5)
PHASES = ("floor", "axis1", "axis3")


def float_tag(v: float) -> str:
    return f"{v:g}".replace("-", "m").replace(".", "p")


@dataclass
class MatrixSpec:
    checkpoint_path: Path
    sp_model_path: Optional[Path] = None
    jsonl_paths: Sequence[Path] = ()
    val_cache_dir: Optional[Path] = None
    output_root: Path = Path("results_exp20")
    config_dir: Path = Path("configs_exp20")
    matrix: str = "first_wave"
    phase: str = "all"
    seeds: Sequence[int] = DEFAULT_SEEDS
    chunk_size: int = 256
    steps_per_chunk: int = 1
    default_eval_lr: float = 0.064
    warmup_steps: int = 0
    max_docs: int = 50_000
    budget_seconds: float = 600.0
    score_floor_seconds: float = 0.0
    safety_margin_seconds: float = 0.0
    persistence_winner: str = "reset"
    axis1_adapt_sets: Sequence[str] = DEFAULT_AXIS1_ADAPT_SETS
    axis1_eval_lrs: Sequence[float] = DEFAULT_AXIS1_EVAL_LRS
    delta_scales: Sequence[float] = DEFAULT_DELTA_SCALES
    log_a_shifts: Sequence[float] = DEFAULT_LOG_A_SHIFTS

    def base(self, *, name: str, phase: str, seed: int) -> dict[str, Any]:
        d = Path(self.output_root) / phase
        cfg = {"name": name, "phase": phase, "adapt_set": "none", "persistence_mode": "reset", "delta_scale": 1.0,
               "log_a_shift": 0.0, "chunk_size": self.chunk_size, "steps_per_chunk": 1, "eval_lr": self.default_eval_lr,
               "persistent_muon_moments": False, "warmup_steps": self.warmup_steps, "seed": int(seed),
               "max_docs": self.max_docs, "budget_seconds": self.budget_seconds,
               "score_floor_seconds": self.score_floor_seconds, "safety_margin_seconds": self.safety_margin_seconds,
               "checkpoint_path": str(self.checkpoint_path), "output_path": str(d / f"{name}.jsonl"),
               "summary_path": str(d / f"{name}_summary.json"), "jsonl_paths": [str(p) for p in self.jsonl_paths],
               "sp_model_path": None if self.sp_model_path is None else str(self.sp_model_path)}
        if self.val_cache_dir is not None:
            cfg["val_cache_dir"] = str(self.val_cache_dir)
        return cfg


def _floor(s: MatrixSpec) -> Iterable[dict]:
    for mode in ("reset", "carry_state"):
        for seed in s.seeds:
            yield dict(s.base(name=f"floor_{mode}_s{seed}", phase="floor", seed=seed), adapt_set="none",
                       persistence_mode=mode, steps_per_chunk=0, score_floor_seconds=0.0)


def _axis1(s: MatrixSpec) -> Iterable[dict]:
    for adapt in s.axis1_adapt_sets:
        if adapt == "all":
            raise ValueError("first-wave axis1 screen must not include adapt_set='all'")
        for lr in s.axis1_eval_lrs:
            for seed in s.seeds:
                name = f"axis1_{adapt}_lr{float_tag(lr)}_{s.persistence_winner}_s{seed}"
                yield dict(s.base(name=name, phase="axis1", seed=seed), adapt_set=adapt,
                           persistence_mode=s.persistence_winner, steps_per_chunk=s.steps_per_chunk, eval_lr=float(lr))


def _axis3(s: MatrixSpec) -> Iterable[dict]:
    knobs: list[tuple[str, float, float]] = []
    seen: set[tuple[float, float]] = set()
    for scale in s.delta_scales:
        if (scale, 0.0) not in seen:
            seen.add((scale, 0.0))
            knobs.append((f"delta_scale_{float_tag(scale)}", float(scale), 0.0))
    for shift in s.log_a_shifts:
        if (1.0, shift) not in seen:                   # (1, 0) is the identity both lists contain: once
            seen.add((1.0, shift))
            knobs.append((f"log_a_shift_{float_tag(shift)}", 1.0, float(shift)))
    for label, scale, shift in knobs:
        for seed in s.seeds:
            yield dict(s.base(name=f"axis3_{label}_{s.persistence_winner}_s{seed}", phase="axis3", seed=seed),
                       adapt_set="none", persistence_mode=s.persistence_winner, steps_per_chunk=0, delta_scale=scale,
                       log_a_shift=shift)


_BUILDERS = {"floor": _floor, "axis1": _axis1, "axis3": _axis3}


def build_configs(spec: MatrixSpec) -> list[dict[str, Any]]:
    phases = PHASES if spec.phase == "all" else (spec.phase,)
    out: list[dict[str, Any]] = []
    for ph in phases:
        if ph not in _BUILDERS:
            raise ValueError(f"unknown phase: {ph}")
        out.extend(_BUILDERS[ph](spec))
    return out


def write_configs(spec: MatrixSpec, configs: Sequence[dict[str, Any]]) -> dict[str, Any]:
    Path(spec.config_dir).mkdir(parents=True, exist_ok=True)
    for cfg in configs:
        Path(cfg["output_path"]).parent.mkdir(parents=True, exist_ok=True)
        (Path(spec.config_dir) / f"{cfg['name']}.json").write_text(json.dumps(cfg, indent=2, sort_keys=True) + "\n")
    manifest = {"matrix": spec.matrix, "phase": spec.phase, "total_configs": len(configs),
                "counts_by_phase": dict(sorted(Counter(str(c["phase"]) for c in configs).items())),
                "seeds": [int(s) for s in spec.seeds], "checkpoint_path": str(spec.checkpoint_path),
                "sp_model_path": None if spec.sp_model_path is None else str(spec.sp_model_path),
                "jsonl_paths": [str(p) for p in spec.jsonl_paths], "output_root": str(spec.output_root)}
    (Path(spec.config_dir) / "manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    return manifest


# ---------------------------------------------------------------------------
# queue
# ---------------------------------------------------------------------------
def pending_configs(config_dir: Path, *, resume: bool) -> tuple[list[Path], list[tuple[str, Path]]]:
    pending, skipped = [], []
    for path in sorted(p for p in Path(config_dir).glob("*.json") if p.name != "manifest.json"):
        cfg = json.loads(path.read_text())
        name = str(cfg.get("name") or path.stem)
        done = bool(cfg.get("summary_path")) and Path(str(cfg["summary_path"])).exists()
        (skipped.append((name, path)) if resume and done else pending.append(path))
    return pending, skipped


def default_command(python: str, config_path: Path) -> list[str]:
    cfg = json.loads(Path(config_path).read_text())
    cmd = [python, "-m", "chaoscontrol_b200.eval_stream.run_eval", "--config", str(config_path)]
    if cfg.get("val_cache_dir"):
        cmd += ["--val-cache-dir", str(cfg["val_cache_dir"])]
    if cfg.get("jsonl_paths"):
        cmd += ["--jsonl-paths", *[str(p) for p in cfg["jsonl_paths"]]]
    if cfg.get("sp_model_path"):
        cmd += ["--sp-model-path", str(cfg["sp_model_path"])]
    return cmd


def run_queue(config_dir: Path, gpus: Sequence[str], *, log_dir: Path, resume: bool = False, dry_run: bool = False,
              python: str = sys.executable, command=default_command, runner=subprocess.run) -> dict[str, Any]:
    """Each pending config runs on the next free GPU; returns ``{"ran", "skipped", "failures", "plan"}``."""
    pending, skipped = pending_configs(config_dir, resume=resume)
    plan = [(json.loads(p.read_text()).get("name") or p.stem, str(gpus[i % len(gpus)]), str(p))
            for i, p in enumerate(pending)]
    out: dict[str, Any] = {"skipped": [n for n, _ in skipped], "plan": plan, "ran": [], "failures": []}
    if dry_run or not pending:
        return out
    free: "queue.Queue[str]" = queue.Queue()
    for g in gpus:
        free.put(str(g))

    def one(path: Path) -> tuple[str, int, str]:
        name = str(json.loads(path.read_text()).get("name") or path.stem)
        gpu = free.get()
        try:
            Path(log_dir).mkdir(parents=True, exist_ok=True)
            log_path = Path(log_dir) / f"{name}.log"
            env = dict(os.environ, CUDA_VISIBLE_DEVICES=gpu, LOCAL_RANK="0", PYTHONUNBUFFERED="1")
            cmd = command(python, path)
            with log_path.open("w") as log:
                log.write(f"$ {' '.join(cmd)}\nCUDA_VISIBLE_DEVICES={gpu} LOCAL_RANK=0\n\n")
                log.flush()
                res = runner(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, text=True)
            return name, int(res.returncode), str(log_path)
        finally:
            free.put(gpu)

    with ThreadPoolExecutor(max_workers=len(gpus)) as pool:
        for name, rc, log_path in pool.map(one, pending):
            out["ran"].append(name)
            if rc != 0:
                out["failures"].append({"name": name, "returncode": rc, "log": log_path})
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build")
    b.add_argument("--checkpoint-path", type=Path, required=True)
    b.add_argument("--sp-model-path", type=Path, default=None)
    b.add_argument("--jsonl-path", type=Path, nargs="*", default=[])
    b.add_argument("--val-cache-dir", type=Path, default=None)
    b.add_argument("--config-dir", type=Path, required=True)
    b.add_argument("--output-root", type=Path, required=True)
    b.add_argument("--phase", choices=("all",) + PHASES, default="all")
    b.add_argument("--seeds", type=int, nargs="+", default=list(DEFAULT_SEEDS))
    b.add_argument("--persistence-winner", default="reset")
    b.add_argument("--max-docs", type=int, default=50_000)
    b.add_argument("--budget-seconds", type=float, default=600.0)
    b.add_argument("--score-floor-seconds", type=float, default=0.0)
    q = sub.add_parser("queue")
    q.add_argument("--config-dir", type=Path, required=True)
    q.add_argument("--gpus", nargs="+", required=True)
    q.add_argument("--log-dir", type=Path, default=Path("logs_exp20"))
    q.add_argument("--resume", action="store_true")
    q.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "build":
        spec = MatrixSpec(checkpoint_path=a.checkpoint_path, sp_model_path=a.sp_model_path, jsonl_paths=a.jsonl_path,
                          val_cache_dir=a.val_cache_dir, config_dir=a.config_dir, output_root=a.output_root, phase=a.phase,
                          seeds=a.seeds, persistence_winner=a.persistence_winner, max_docs=a.max_docs,
                          budget_seconds=a.budget_seconds, score_floor_seconds=a.score_floor_seconds)
        print(json.dumps(write_configs(spec, build_configs(spec)), indent=2))
        return 0
    res = run_queue(a.config_dir, a.gpus, log_dir=a.log_dir, resume=a.resume, dry_run=a.dry_run)
    for n in res["skipped"]:
        print(f"SKIP {n}")
    for n, g, p in (res["plan"] if a.dry_run else []):
        print(f"RUN {n} gpu={g} config={p}")
    for f in res["failures"]:
        print(f"FAIL {f['name']} rc={f['returncode']} log={f['log']}")
    return 1 if res["failures"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
