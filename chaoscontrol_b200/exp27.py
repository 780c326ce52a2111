"""Test-time-training headline: calibrate the evaluation passes to the eval
budget, then evaluate the winning trunk with them
(experiments/27_ttt_headline/{calibrate,exp27,run_exp27}.py).

* `default_calc_type_hyperparams` / `write_manifest`: the default manifest.
* `probe_calc_types`: measures each registered pass on the first documents of
  a validation cache, extrapolates to the whole cache and shrinks the
  expensive knobs until the estimate fits the budget.  (The reference's
  calibrator only writes defaults.)
* `build_ttt_headline_matrix`: one entry per seed on top of the
  adaptive-residual-memory cell, carrying ``calc_types`` /
  ``calc_type_configs``; with a checkpoint the entry is eval-only.

``python -m chaoscontrol_b200.exp27 calibrate --manifest m.json [--checkpoint
ck.pt --val-cache-dir val/ --budget-seconds 600]`` and
``python -m chaoscontrol_b200.exp27 matrix --manifest m.json --config speed.yaml``.
"""
from __future__ import annotations

import argparse
import copy
import json
import time
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Optional, Sequence

from .exp26 import build_validation_matrix as _exp26_matrix

__all__ = ["CALC_TYPES_DEFAULT", "DEFAULT_HEADLINE_SEEDS", "EXP26_ARM_NAME", "default_calc_type_hyperparams",
           "build_manifest", "write_manifest", "load_manifest", "probe_calc_types", "build_ttt_headline_matrix",
           "main"]

CALC_TYPES_DEFAULT: tuple[str, ...] = ("score_only_reset", "adaptive_carry")
DEFAULT_HEADLINE_SEEDS: tuple[int, ...] = (1337, 2674, 4011)
EXP26_ARM_NAME = "validation_adaptive_residual_memory"
# per pass: the knob that buys time when the estimate is over budget, and its floor
_SHRINK = {"dreamworld_eval": ("K", 1), "adaptive_carry": ("online_episodic_write_tokens_per_chunk", 1)}


def default_calc_type_hyperparams() -> dict[str, dict[str, Any]]:
    """Defaults sized for a 600 s evaluation of the locked trunk (calibrate.py:32-56)."""
    return {
        "score_only_reset": {},
        "adaptive_carry": {"horizon_shifts": [-0.5, 0.0, 0.5], "online_eta": 1.0, "decay": 1.0,
                           "online_episodic_chunk_tokens": 256,
                           "online_episodic_write_tokens_per_chunk": 16, "online_episodic_gate": 1.0},
        "carry_state": {"decay": 1.0},
        "dreamworld_eval": {"K": 8, "L": 64, "lr": 0.001, "steps": 1, "per_doc_reset": True,
                            "dream_target_mode": "argmax", "dream_temperature": 1.0, "prefix_len": 16},
    }


def build_manifest(*, hyperparams: Optional[dict[str, dict[str, Any]]] = None, source: str = "defaults",
                   probe: Optional[dict[str, Any]] = None) -> dict[str, Any]:
    m = {"calibrated_at": datetime.now(timezone.utc).isoformat(), "source_trace": source,
         "calc_type_hyperparams": hyperparams or default_calc_type_hyperparams()}
    if probe is not None:
        m["probe"] = probe
    else:
        m["note"] = "default hyperparameters; no probe was run"
    return m


def write_manifest(path: Path | str, manifest: Optional[dict[str, Any]] = None) -> dict[str, Any]:
    manifest = manifest or build_manifest()
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(manifest, indent=2, sort_keys=True))
    return manifest


def load_manifest(path: Path | str) -> dict[str, Any]:
    """Reads and validates a calibration manifest (exp27.py:54-68)."""
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"calibration manifest missing: {p}")
    try:
        manifest = json.loads(p.read_text())
    except Exception as exc:  # noqa: BLE001
        raise ValueError(f"manifest at {p} is malformed: {exc!r}") from exc
    missing = {"calc_type_hyperparams", "calibrated_at"} - set(manifest)
    if missing:
        raise ValueError(f"manifest at {p} missing required keys: {sorted(missing)}")
    return manifest


def probe_calc_types(*, model, val_cache, device, luts: tuple, calc_types: Sequence[str],
                     budget_seconds: float = 600.0, probe_docs: int = 16, max_rounds: int = 4,
                     hyperparams: Optional[dict[str, dict[str, Any]]] = None,
                     time_fn=time.perf_counter) -> tuple[dict[str, dict[str, Any]], dict[str, Any]]:
    """Times each pass on the first ``probe_docs`` documents, scales by scored tokens to the whole
    cache, and halves the pass's shrink knob until the estimate fits ``budget_seconds`` (at most
    ``max_rounds`` times).  Returns ``(hyperparams, probe report)``."""
    from .eval.registry import evaluate_with_calc_types
    hp = copy.deepcopy(hyperparams or default_calc_type_hyperparams())
    total = int(val_cache.total_tokens)
    report: dict[str, Any] = {"budget_seconds": float(budget_seconds), "probe_docs": int(probe_docs),
                              "total_tokens": total, "calc_types": {}}
    for name in calc_types:
        cfg = hp.setdefault(name, {})
        rounds = []
        for _ in range(max_rounds + 1):
            t0 = time_fn()
            res = evaluate_with_calc_types(
                model=model, val_cache=val_cache, calc_types=[name],
                calc_type_configs={name: dict(cfg, max_docs=int(probe_docs))}, device=device,
                base_bytes_lut=luts[0], has_leading_space_lut=luts[1], is_boundary_token_lut=luts[2])[name]
            dt = time_fn() - t0
            scored = max(int(res["tokens_scored"]), 1)
            est = dt * total / scored
            knob, floor = _SHRINK.get(name, (None, None))
            rounds.append({"seconds": dt, "tokens_scored": scored, "estimated_full_seconds": est,
                           "bpb": res["bpb"], "knob": knob, "value": cfg.get(knob) if knob else None})
            if est <= budget_seconds or knob is None or int(cfg.get(knob, floor)) <= floor:
                break
            cfg[knob] = max(int(floor), int(cfg[knob]) // 2)
        report["calc_types"][name] = {"rounds": rounds, "fits_budget": rounds[-1]["estimated_full_seconds"]
                                      <= budget_seconds}
    return hp, report


def build_ttt_headline_matrix(*, speed_config: dict[str, Any], calibration_manifest_path: Path | str,
                              checkpoint_path: Optional[Path | str] = None, world_size: int = 4,
                              budget_seconds: float = 600.0, seed_values: Optional[Sequence[int]] = None,
                              calc_types: Optional[Sequence[str]] = None) -> list[dict[str, Any]]:
    """One entry per seed (exp27.py:71-180).  The headline pass is ``adaptive_carry`` when
    requested, else ``score_only_reset``, else the first one."""
    from .eval.ttt_eval import list_registered_calc_types
    seeds = list(seed_values) if seed_values is not None else list(DEFAULT_HEADLINE_SEEDS)
    requested = list(calc_types) if calc_types is not None else list(CALC_TYPES_DEFAULT)
    registered = set(list_registered_calc_types())
    for name in requested:
        if name not in registered:
            raise ValueError(f"unknown calc_type: {name!r}")
    by_type = dict(load_manifest(calibration_manifest_path).get("calc_type_hyperparams", {}))
    configs = {name: dict(by_type.get(name, {})) for name in requested}
    headline = next((n for n in ("adaptive_carry", "score_only_reset") if n in requested), requested[0])
    ckpt = str(checkpoint_path) if checkpoint_path is not None else None
    entries = []
    for seed in seeds:
        cells = [e for e in _exp26_matrix(speed_config=speed_config, world_size=int(world_size),
                                          budget_seconds=float(budget_seconds), seed=int(seed))
                 if e.get("arm") == EXP26_ARM_NAME]
        if len(cells) != 1:
            raise RuntimeError(f"expected one {EXP26_ARM_NAME!r} entry, got {len(cells)}")
        entry = copy.deepcopy(cells[0])
        entry.update({"name": f"exp27_ttt_headline_s{int(seed)}", "seed": int(seed),
                      "exp27_mechanism": "ttt_headline_v1", "calc_types": list(requested),
                      "calc_type_configs": copy.deepcopy(configs), "headline_calc_type": headline,
                      "checkpoint_path": ckpt})
        if ckpt is not None:
            entry.update({"eval_only": True, "warmup_steps": 0, "max_steps": 0, "restore_after_warmup": False})
        entries.append(entry)
    return entries


def _probe_from_checkpoint(checkpoint: Path, val_cache_dir: Path, sp_model_path: Path, calc_types: Sequence[str],
                           budget_seconds: float, probe_docs: int) -> tuple[dict, dict]:
    import sentencepiece as spm
    import torch
    from .eval_stream import load_val_cache
    from .fast_score import _load_model
    from .sp_eval import build_sentencepiece_luts
    dev = torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    model, _ = _load_model(str(checkpoint), dev)
    sp = spm.SentencePieceProcessor()
    sp.Load(str(sp_model_path))
    luts = build_sentencepiece_luts(sp, int(model.vocab_size), dev)
    return probe_calc_types(model=model, val_cache=load_val_cache(val_cache_dir), device=dev, luts=luts,
                            calc_types=calc_types, budget_seconds=budget_seconds, probe_docs=probe_docs)


def run_stages(a, say=print) -> int:
    """``run --stage calibrate|analyze|headline|all`` (run_exp27.py:96-340 of the reference).

    * calibrate: with a checkpoint, every requested evaluation pass is timed on the first documents and its
      shrink knob halved until the extrapolated pass fits the headline budget; the report goes to
      ``--trace-path`` (default: beside the manifest).  Without a checkpoint there is nothing to time.
    * analyze: writes the calibration manifest -- the probed hyper-parameters when a report exists, the
      defaults otherwise.
    * headline: one entry per seed (training a trunk, or evaluating ``--checkpoint-path``), each running the
      selected passes; launched through ``launch.run_matrix``.

    ``--dry-run`` writes and creates nothing: every stage prints what it would do."""
    from .fast_path import read_speed_config, write_matrix
    speed = read_speed_config(a.config) if a.config else {}
    trace = Path(a.trace_path) if a.trace_path else Path(a.manifest_path).with_name("probe_report.json")
    if a.stage in ("calibrate", "all"):
        probing = a.checkpoint_path is not None and a.sp_model_path is not None and Path(a.val_cache_dir).is_dir()
        say(f"[exp27] stage=calibrate probe={probing} dry_run={a.dry_run}")
        if a.dry_run:
            say(json.dumps(build_manifest(), indent=2, sort_keys=True, default=str))
        elif probing:
            hp, report = _probe_from_checkpoint(a.checkpoint_path, a.val_cache_dir, a.sp_model_path, a.calc_types,
                                                a.headline_budget, a.probe_docs)
            trace.parent.mkdir(parents=True, exist_ok=True)
            trace.write_text(json.dumps({"hyperparams": hp, "report": report, "source": str(a.checkpoint_path)}, indent=2))
    if a.stage in ("analyze", "all"):
        probed = json.loads(trace.read_text()) if trace.exists() else None
        manifest = (build_manifest(hyperparams=probed["hyperparams"], source=probed.get("source", str(trace)),
                                   probe=probed["report"]) if probed else build_manifest())
        say(f"[exp27] stage=analyze manifest={a.manifest_path} probed={probed is not None} dry_run={a.dry_run}")
        if a.dry_run:
            say(json.dumps(manifest, indent=2, sort_keys=True, default=str))
        else:
            write_manifest(a.manifest_path, manifest)
    if a.stage in ("headline", "all"):
        if a.dry_run and not Path(a.manifest_path).exists():
            say(f"[exp27] stage=headline dry_run=True manifest_absent=True: previewing default hyper-parameters")
            say(json.dumps(build_manifest(), indent=2, sort_keys=True, default=str))
            return 0
        entries = build_ttt_headline_matrix(speed_config=speed, calibration_manifest_path=a.manifest_path,
                                            checkpoint_path=a.checkpoint_path, world_size=a.world_size,
                                            budget_seconds=a.headline_budget, seed_values=a.seeds,
                                            calc_types=a.calc_types)
        say(f"[exp27] stage=headline entries={len(entries)} world_size={a.world_size} budget={a.headline_budget}s "
            f"dry_run={a.dry_run}")
        if a.dry_run:
            for e in entries:
                say(f"[exp27] {e['name']}")
                say(json.dumps(e, indent=2, sort_keys=True, default=str))
            return 0
        if entries and not Path(a.val_cache_dir).is_dir():
            raise FileNotFoundError("the evaluation passes need a validation cache: build it with "
                                    f"`python -m chaoscontrol_b200.cli build-val-cache` (missing: {a.val_cache_dir})")
        from .launch import run_matrix
        out = Path(a.headline_output_dir)
        out.mkdir(parents=True, exist_ok=True)
        write_matrix(out / "matrix.json", entries)
        run_matrix(entries, results_dir=out, data_path=str(a.data_path),
                   sp_model_path=None if a.sp_model_path is None else str(a.sp_model_path), world_size=int(a.world_size),
                   val_cache_dir=str(a.val_cache_dir), limit=a.limit, skip_existing=bool(a.skip_existing))
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("calibrate", help="write the calibration manifest (probe when a checkpoint is given)")
    c.add_argument("--manifest", type=Path, required=True)
    c.add_argument("--checkpoint", type=Path, default=None)
    c.add_argument("--val-cache-dir", type=Path, default=None)
    c.add_argument("--sp-model-path", type=Path, default=None)
    c.add_argument("--budget-seconds", type=float, default=600.0)
    c.add_argument("--probe-docs", type=int, default=16)
    c.add_argument("--calc-types", nargs="+", default=list(CALC_TYPES_DEFAULT))
    m = sub.add_parser("matrix", help="print / write the headline matrix")
    m.add_argument("--manifest", type=Path, required=True)
    m.add_argument("--config", type=Path, default=None)
    m.add_argument("--checkpoint", type=Path, default=None)
    m.add_argument("--world-size", type=int, default=4)
    m.add_argument("--budget", type=float, default=600.0)
    m.add_argument("--seeds", type=int, nargs="+", default=list(DEFAULT_HEADLINE_SEEDS))
    m.add_argument("--calc-types", nargs="+", default=None)
    m.add_argument("--out", type=Path, default=None)
    r = sub.add_parser("run", help="the staged orchestrator: calibrate -> analyze -> headline")
    r.add_argument("--stage", choices=["calibrate", "analyze", "headline", "all"], default="all")
    r.add_argument("--config", type=Path, default=None)
    r.add_argument("--data-path", type=Path, default=Path("data"))
    r.add_argument("--sp-model-path-16384", "--sp-model-path", dest="sp_model_path", type=Path, default=None)
    r.add_argument("--val-cache-dir", type=Path, default=Path("val_cache"))
    r.add_argument("--checkpoint-path", type=Path, default=None,
                   help="a trained trunk: the headline cells then only evaluate it")
    r.add_argument("--world-size", type=int, default=4)
    r.add_argument("--seeds", type=int, nargs="+", default=list(DEFAULT_HEADLINE_SEEDS))
    r.add_argument("--calc-types", nargs="+", default=list(CALC_TYPES_DEFAULT))
    r.add_argument("--manifest-path", type=Path, default=Path("calibration/manifest.json"))
    r.add_argument("--trace-path", type=Path, default=None, help="probe report of an earlier calibrate stage")
    r.add_argument("--headline-output-dir", type=Path, default=Path("results/exp27"))
    r.add_argument("--headline-budget", type=float, default=600.0)
    r.add_argument("--probe-docs", type=int, default=16)
    r.add_argument("--limit", type=int, default=None)
    r.add_argument("--skip-existing", action=argparse.BooleanOptionalAction, default=True)
    r.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "run":
        return run_stages(a)
    if a.cmd == "calibrate":
        if a.checkpoint is None:
            man = write_manifest(a.manifest)
            print(f"[calibrate] wrote {a.manifest} (defaults) with {len(man['calc_type_hyperparams'])} sets")
            return 0
        if a.val_cache_dir is None or a.sp_model_path is None:
            ap.error("probing needs --val-cache-dir and --sp-model-path")
        import sentencepiece as spm
        import torch
        from .eval_stream import load_val_cache
        from .fast_score import _load_model
        from .sp_eval import build_sentencepiece_luts
        dev = torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
        model, _ = _load_model(str(a.checkpoint), dev)
        sp = spm.SentencePieceProcessor()
        sp.Load(str(a.sp_model_path))
        luts = build_sentencepiece_luts(sp, int(model.vocab_size), dev)
        hp, report = probe_calc_types(model=model, val_cache=load_val_cache(a.val_cache_dir), device=dev,
                                      luts=luts, calc_types=a.calc_types, budget_seconds=a.budget_seconds,
                                      probe_docs=a.probe_docs)
        write_manifest(a.manifest, build_manifest(hyperparams=hp, source=str(a.checkpoint), probe=report))
        print(json.dumps({k: v["fits_budget"] for k, v in report["calc_types"].items()}))
        return 0
    import yaml
    speed = (yaml.safe_load(a.config.read_text()) or {}) if a.config else {}
    entries = build_ttt_headline_matrix(speed_config=speed, calibration_manifest_path=a.manifest,
                                        checkpoint_path=a.checkpoint, world_size=a.world_size,
                                        budget_seconds=a.budget, seed_values=a.seeds, calc_types=a.calc_types)
    if a.out:
        a.out.parent.mkdir(parents=True, exist_ok=True)
        a.out.write_text(json.dumps(entries, indent=2, default=str))
    for e in entries:
        print(e["name"])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
