"""Launcher for the training-time bundle matrices: build a matrix, write
``matrix.json``, optionally smoke one heavily instrumented cell first, run
every cell through the throughput runner under torchrun, then (optionally)
score each saved checkpoint on the full validation cache
(experiments/24_training_time_bundle/run_exp24.py:1-730).

``python -m chaoscontrol_b200.run_exp24 --matrix crct_v1 --config speed.yaml
--data-path shards/ --output-dir results/ [--dry-run]``
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path
from typing import Any, Optional, Sequence

from . import exp24
from .launch import DRY_RUN_RDZV_PORT, pick_free_port, run_matrix

__all__ = ["MATRICES", "SMOKE_BUDGET_SECONDS", "SMOKE_ARM_BY_MATRIX", "build_entries",
           "default_world_size", "default_budget", "smoke_check_result", "run_smoke",
           "full_val_commands", "main"]

# matrix name -> (builder, name of its seed keyword; "seed" = one call per seed)
MATRICES: dict[str, tuple[Any, str]] = {
    "ring0_control": (exp24.build_ring0_control_matrix, "seeds"),
    "phase_a_sampling": (exp24.build_phase_a_sampling_matrix, "seeds"),
    "semantic_overhead_gate": (exp24.build_semantic_overhead_gate_matrix, "seed"),
    "scopt_overhead_gate": (exp24.build_scopt_overhead_gate_matrix, "seed"),
    "scopt_calibration_sweep": (exp24.build_scopt_calibration_sweep_matrix, "seed"),
    "first_wave": (exp24.build_first_wave_mechanism_matrix, "seed_values"),
    "fastslow_dreamworld": (exp24.build_fastslow_dreamworld_matrix, "seed_values"),
    "phase0_dreamworld_sweep": (exp24.build_phase0_dreamworld_sweep, "seed_values"),
    "phase0_fastslow_sweep": (exp24.build_phase0_fastslow_sweep, "seed_values"),
    "phase0_confirm": (exp24.build_phase0_confirm, "seed_values"),
    "phase0_fastslow_only_control": (exp24.build_phase0_fastslow_only_control, "seed_values"),
    "episodic_dw_curation_v1": (exp24.build_episodic_dw_curation_v1_matrix, "seed_values"),
    "episodic_ttt_v1": (exp24.build_episodic_ttt_v1_matrix, "seed_values"),
    "cd_first_smoke": (exp24.build_criticality_distillation_first_smoke_matrix, "seed_values"),
    "cd_multiseed": (exp24.build_criticality_distillation_multiseed_matrix, "seed_values"),
    "episodic_controller_v1": (exp24.build_episodic_controller_v1_matrix, "seed_values"),
    "crct_v1": (exp24.build_crct_v1_matrix, "seed_values"),
}
# "all" = the original first-wave bundle
_ALL = ("ring0_control", "phase_a_sampling", "semantic_overhead_gate", "first_wave")
_ONE_GPU = {"semantic_overhead_gate", "scopt_overhead_gate", "scopt_calibration_sweep",
            "cd_first_smoke", "cd_multiseed"}
_EIGHT_GPU = {"ring0_control", "phase_a_sampling", "first_wave", "fastslow_dreamworld", "all"}
_BUDGETS = {"semantic_overhead_gate": 90.0, "scopt_overhead_gate": 180.0, "scopt_calibration_sweep": 1200.0}

# Before a matrix runs, its most instrumented cell runs alone for a short budget and the result is
# checked for signs that a mechanism silently fell back to a cheaper path.
SMOKE_BUDGET_SECONDS = 90.0
SMOKE_ARM_BY_MATRIX = {"episodic_controller_v1": "arm_e_simplex_warm_online"}


def default_world_size(matrix: str) -> int:
    return 1 if matrix in _ONE_GPU else 8 if matrix in _EIGHT_GPU else 4


def default_budget(matrix: str) -> float:
    """Gate matrices need a budget that clears the optimizer's warm-up
    (run_exp24.py:522-537)."""
    return _BUDGETS.get(matrix, 600.0)


def build_entries(*, matrix: str, speed_config: dict[str, Any], world_size: int, budget_seconds: float,
                  seeds: Sequence[int]) -> list[dict[str, Any]]:
    if matrix == "all":
        return [e for m in _ALL for e in build_entries(matrix=m, speed_config=speed_config, world_size=world_size,
                                                       budget_seconds=budget_seconds, seeds=seeds)]
    if matrix not in MATRICES:
        raise ValueError(f"unsupported matrix: {matrix}")
    fn, seed_kw = MATRICES[matrix]
    kw = dict(speed_config=speed_config, world_size=world_size, budget_seconds=budget_seconds)
    if seed_kw == "seed":
        return [e for s in seeds for e in fn(seed=int(s), **kw)]
    return fn(**{seed_kw: [int(s) for s in seeds]}, **kw)


def smoke_check_result(*, result_path: Path, entry: dict[str, Any]) -> tuple[bool, list[str]]:
    """``(ok, failures)`` for a smoke cell's result file (run_exp24.py:63-142).  With the episodic
    runtime on, the producer must have emitted events, the episodic rank must have ingested and
    replayed them, and nothing may have been dropped for a full ring; a simplex cell must leave a
    trace with decision and credit rows and at least one decision that is not near-uniform."""
    fails: list[str] = []
    if not result_path.exists():
        return False, [f"result JSON not produced at {result_path}"]
    try:
        d = json.loads(result_path.read_text())
    except Exception as exc:  # noqa: BLE001
        return False, [f"result JSON malformed: {exc!r}"]
    if "error" in d:
        return False, [f"runner reported error: {d.get('error')!r}"]
    train = d.get("train", {})
    if not isinstance(train, dict) or "steps" not in train:
        return False, ["result JSON missing train block / train.steps"]
    epi = train.get("episodic") or {}
    if entry.get("episodic_enabled"):
        if not epi.get("enabled"):
            fails.append("episodic_enabled cell reports no episodic runtime")
        else:
            if int(epi.get("write_events_emitted", 0)) == 0:
                fails.append("write_events_emitted=0: no write event left the train ranks")
            if epi.get("role") in ("episodic", "solo"):
                if int(epi.get("write_events_ingested", 0)) == 0:
                    fails.append("write_events_ingested=0: nothing reached the episodic cache")
                if entry.get("controller_query_enabled") and int(epi.get("replays", 0)) == 0:
                    fails.append("replays=0: the controller never tagged a replay")
            emitted = max(int(epi.get("write_events_emitted", 0)), 1)
            if int(epi.get("write_events_dropped", 0)) > emitted:
                fails.append(f"write_events_dropped={epi['write_events_dropped']} exceeds emitted")
    if "simplex" in str(entry.get("name", "")) and entry.get("episodic_controller_simplex_trace_path"):
        tp = Path(entry["episodic_controller_simplex_trace_path"])
        if not tp.exists():
            fails.append(f"simplex trace not produced at {tp}")
        else:
            n_dec = n_credit = 0
            min_ent = float("inf")
            with tp.open() as fh:
                for i, line in enumerate(fh):
                    if i >= 2000:
                        break
                    try:
                        row = json.loads(line)
                    except Exception:  # noqa: BLE001
                        continue
                    if row.get("row_type") == "decision":
                        n_dec += 1
                        if isinstance(row.get("entropy"), (int, float)):
                            min_ent = min(min_ent, float(row["entropy"]))
                    elif row.get("row_type") == "credit":
                        n_credit += 1
            if n_dec == 0:
                fails.append("simplex trace has no decision rows")
            if n_credit == 0 and entry.get("controller_train_online", True):
                fails.append("simplex trace has no credit rows (no replay reached the learner)")
            if n_dec and min_ent > 2.5:                     # ln 16 = 2.77: every decision near-uniform
                fails.append(f"all {n_dec} sampled decisions have entropy > 2.5 (min={min_ent:.4f})")
    return not fails, fails


def run_smoke(*, matrix: str, entries: list[dict[str, Any]], data_path: str, sp_model_path: Optional[str],
              results_dir: Path, world_size: int) -> tuple[bool, list[str]]:
    arm = SMOKE_ARM_BY_MATRIX.get(matrix)
    if arm is None:
        return True, [f"smoke skipped: no smoke arm registered for {matrix}"]
    hits = [e for e in entries if arm in str(e.get("name", ""))]
    if not hits:
        return False, [f"smoke arm {arm!r} matched no entries in matrix {matrix}"]
    cell = dict(hits[0], budget_seconds=SMOKE_BUDGET_SECONDS, name=f"smoke_{hits[0]['name']}")
    smoke_dir = results_dir / ".smoke"
    smoke_dir.mkdir(parents=True, exist_ok=True)
    if cell.get("episodic_controller_simplex_trace_path"):     # keep a real run's trace intact
        cell["episodic_controller_simplex_trace_path"] = str(smoke_dir / "smoke_simplex_trace.ndjson")
    print(f"[smoke] running 1 cell ({cell['name']}) for {SMOKE_BUDGET_SECONDS:.0f}s before the matrix", flush=True)
    run_matrix([cell], results_dir=smoke_dir, data_path=data_path, sp_model_path=sp_model_path,
               world_size=world_size, skip_existing=False)
    return smoke_check_result(result_path=smoke_dir / f"{cell['name']}.json", entry=cell)


def full_val_commands(*, entries: list[dict[str, Any]], checkpoint_dir: Path, results_dir: Path, world_size: int,
                      cache_dir: Path, budget_seconds: float, dry_run: bool = False,
                      run: bool = True) -> list[list[str]]:
    """One document-parallel scoring command per saved checkpoint without a summary yet
    (run_exp24.py:253-317); runs them unless ``dry_run``.  Cells whose eval uses the episodic
    cache or test-time training list ``calc_types`` in their config and are evaluated by the
    runner itself; this pass is the plain full-validation bpb."""
    out_dir, logs = results_dir / "full_val", results_dir / "logs"
    out_dir.mkdir(parents=True, exist_ok=True)
    logs.mkdir(parents=True, exist_ok=True)
    cmds = []
    for e in entries:
        name = str(e["name"])
        ckpt, done = Path(checkpoint_dir) / f"{name}.pt", out_dir / f"{name}.summary.json"
        if done.exists() or (not dry_run and not ckpt.exists()):
            continue
        adapt, steps = str(e.get("eval_adapt_set", "none")), int(e.get("eval_steps_per_chunk", 0) or 0)
        if adapt != "none" and steps > 0:
            # a test-time-training cell: score-then-adapt per chunk, one process (weights change per document)
            cmd = [sys.executable, "-m", "chaoscontrol_b200.eval_stream.run_eval", "--val-cache-dir", str(cache_dir),
                   "--checkpoint-path", str(ckpt), "--output-path", str(out_dir / f"{name}.jsonl"),
                   "--summary-path", str(done), "--adapt-set", adapt, "--steps-per-chunk", str(steps),
                   "--chunk-size", "256", "--budget-seconds", str(float(budget_seconds))]
        else:
            port = DRY_RUN_RDZV_PORT if dry_run else pick_free_port()
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={int(world_size)}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "chaoscontrol_b200.fast_score",
                   "--cache-dir", str(cache_dir), "--checkpoint-path", str(ckpt),
                   "--output-path", str(out_dir / f"{name}.jsonl"), "--chunk-size", "256",
                   "--budget-seconds", str(float(budget_seconds)), "--doc-batch-size", "4096",
                   "--max-forward-tokens", "auto", "--doc-packing", "chunk_count_tail"]
        cmds.append(cmd)
        if dry_run or not run:
            continue
        with (logs / f"{name}.full_val.log").open("w") as log:
            log.write("+ " + " ".join(cmd) + "\n")
            proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            log.write(proc.stdout + f"\n[returncode] {proc.returncode}\n")
        last = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
        if proc.returncode == 0 and last and not done.exists():
            done.write_text(last[-1])
    return cmds


def main(argv: Optional[Sequence[str]] = None) -> int:
    import yaml
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--matrix", choices=[*MATRICES, "all"], default="all")
    ap.add_argument("--config", type=Path, default=None, help="speed config (YAML); empty config when omitted")
    ap.add_argument("--output-dir", type=Path, default=Path("results/exp24"))
    ap.add_argument("--seeds", type=int, nargs="+", default=list(exp24.DEFAULT_CONTROL_SEEDS))
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--show", action="store_true", help="print every entry; implies --dry-run")
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--world-size", type=int, default=None)
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--data-path", type=Path, default=Path("data"))
    ap.add_argument("--sp-model-path", "--sp-model-path-16384", dest="sp_model_path", type=Path, default=None)
    ap.add_argument("--skip-existing", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--checkpoint-dir", type=Path, default=None)
    ap.add_argument("--full-val-score", action=argparse.BooleanOptionalAction, default=False)
    ap.add_argument("--val-cache-dir", type=Path, default=None)
    ap.add_argument("--val-budget-seconds", type=float, default=600.0)
    ap.add_argument("--smoke", action=argparse.BooleanOptionalAction, default=True)
    a = ap.parse_args(argv)

    world = int(a.world_size) if a.world_size is not None else default_world_size(a.matrix)
    budget = float(a.budget) if a.budget is not None else default_budget(a.matrix)
    ckpt_dir = a.checkpoint_dir
    if a.full_val_score:
        if a.val_cache_dir is None:
            ap.error("--full-val-score needs --val-cache-dir")
        ckpt_dir = ckpt_dir or a.output_dir / "checkpoints"
    speed = (yaml.safe_load(a.config.read_text()) or {}) if a.config else {}
    entries = build_entries(matrix=a.matrix, speed_config=speed, world_size=world, budget_seconds=budget,
                            seeds=a.seeds)
    a.output_dir.mkdir(parents=True, exist_ok=True)
    for e in entries:                                          # the native trace writer appends; it creates no folders
        for key in ("episodic_controller_simplex_trace_path", "replay_eviction_trace_path",
                    "crct_gradient_conflict_trace_path"):
            if e.get(key):
                Path(e[key]).parent.mkdir(parents=True, exist_ok=True)
    (a.output_dir / "matrix.json").write_text(json.dumps(entries, indent=2, default=str))
    dry = bool(a.dry_run or a.show)
    selected = entries[:a.limit] if a.limit is not None else entries
    if dry:
        print(f"[exp24] matrix={a.matrix} entries={len(selected)} world_size={world} dry_run=True", flush=True)
        for e in selected:
            print(f"[exp24] {e['name']}")
            if a.show:
                print(json.dumps(e, indent=2, sort_keys=True, default=str))
    elif a.smoke:
        ok, msgs = run_smoke(matrix=a.matrix, entries=entries, data_path=str(a.data_path),
                             sp_model_path=None if a.sp_model_path is None else str(a.sp_model_path),
                             results_dir=a.output_dir, world_size=world)
        if not ok:
            print("[smoke] FAILED: the matrix was NOT launched.", flush=True)
            for m in msgs:
                print(f"  - {m}", flush=True)
            return 2
        for m in msgs or ["passed; launching the matrix"]:
            print(f"[smoke] {m}", flush=True)
    summary = run_matrix(entries, results_dir=a.output_dir, data_path=str(a.data_path),
                         sp_model_path=None if a.sp_model_path is None else str(a.sp_model_path),
                         world_size=world, dry_run=dry, limit=a.limit, skip_existing=a.skip_existing,
                         checkpoint_dir=ckpt_dir,
                         val_cache_dir=None if a.val_cache_dir is None else str(a.val_cache_dir))
    if a.full_val_score:
        cmds = full_val_commands(entries=selected, checkpoint_dir=ckpt_dir, results_dir=a.output_dir,
                                 world_size=world, cache_dir=a.val_cache_dir,
                                 budget_seconds=float(a.val_budget_seconds), dry_run=dry)
        if dry:
            summary["full_val_commands"] = cmds
    print(json.dumps(summary, indent=2, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
