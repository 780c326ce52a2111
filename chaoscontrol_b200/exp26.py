"""Adaptive-residual-memory validation matrix (experiments/26_arm/exp26.py:1-274).

Two cells at the artifact-size-locked model (dim 384, delta rank 32): the
fast/slow control, and the full stack -- CRCT teacher + controller, replay
eviction in active mode driven by the native maintenance scheduler and the
evidence engine, learned commit policy, refresh proposals, gradient-conflict
monitor.  The fast/slow interval is left to the learned action space, so the
entries carry no ``fast_slow_interval``.
"""
from __future__ import annotations

import copy
import json
from pathlib import Path
from typing import Any, Mapping, Optional, Sequence

from .exp24 import ARTIFACT_CHANGES_WEIGHTS_ONLY, _CRCT, _DW_OFF, _base_entry

__all__ = ["VALIDATION_ARMS", "EXP26_MODEL_DIM", "EXP26_DELTA_RANK", "DEFAULT_VALIDATION_TRACE_DIR",
           "build_validation_matrix", "run_validation", "main"]

VALIDATION_ARMS: tuple[str, ...] = ("validation_fastslow_control", "validation_adaptive_residual_memory")
EXP26_MODEL_DIM = 384
EXP26_DELTA_RANK = 32
DEFAULT_VALIDATION_DIR = Path("experiments/26_arm/validation")
DEFAULT_VALIDATION_TRACE_DIR = DEFAULT_VALIDATION_DIR / "traces"


def _size_lock() -> dict[str, Any]:
    return {"model_dim": EXP26_MODEL_DIM, "ssm_delta_rank": EXP26_DELTA_RANK, "lm_head_tile_size": 4096}


def _fast_slow_lock(trace_dir: Path) -> dict[str, Any]:
    """Fast/slow with the interval and EMA alpha handed to the controller's action heads."""
    return {
        "fast_slow_enabled": True, "fast_slow_alpha": 0.25, "fast_slow_eval_copy": "slow",
        "episodic_controller_action_space_enabled": True,
        "episodic_controller_shared_event_ssm_enabled": True,
        "episodic_controller_ssm_hidden_dim": 16,
        "episodic_controller_head_readiness": {"consolidation": 0.05, "ema_alpha": 1.0},
        "episodic_controller_head_max_delta": {"consolidation": 1.0, "ema_alpha": 0.5},
        "episodic_controller_action_learning_rate": 0.01,
        "episodic_controller_action_trace_path": str(trace_dir / "fast_slow_action_space.ndjson"),
        **_DW_OFF, "train_sampling_mode": "random",
    }


def _crct_lock(trace_dir: Path) -> dict[str, Any]:
    """The bundle's CRCT lock, re-tuned: teacher scores every step, 32 write tokens, plasticity
    budget, maintenance-selected compression, log_a / beta coupling in the optimizer."""
    lock = {k: v for k, v in _CRCT.items()
            if k not in ("crct_async_teacher_pending_batches", "crct_async_teacher_max_lag_steps",
                         "crct_teacher_param_sync_interval_steps")}
    lock.update({
        "crct_plasticity_budget_strength": 0.25, "crct_memory_write_tokens_per_step": 32,
        "crct_teacher_score_interval_steps": 1, "compression_selection": "maintenance",
        "optimizer_log_a_beta_coupling": True, "optimizer_log_a_beta_ema": 0.99,
        "optimizer_log_a_beta_min": 0.5,
        "crct_gradient_conflict_trace_path": str(trace_dir / "crct_conflict.ndjson"),
    })
    return lock


def _pipeline_lock() -> dict[str, Any]:
    return {
        "replay_eviction_enabled": True, "bucket_prototypes": True, "prototype_dim": 64,
        "replay_eviction_memory_streams": 8, "replay_eviction_arm_runtime_enabled": True,
        "replay_eviction_max_seconds": 0.0, "replay_eviction_scoring_mode": "oracle",
        "replay_eviction_oracle_confirm_top_k": 32, "replay_eviction_oracle_variant_chunk_size": 1,
        "replay_eviction_refresh_candidate_count": 16, "replay_eviction_refresh_proposal_rank": 8,
        "replay_eviction_refresh_proposal_noise_scale": 0.04,
        "replay_eviction_refresh_proposal_momentum": 0.9,
        "replay_eviction_refresh_candidate_variant_chunk_size": 16,
        "replay_eviction_refresh_proposal_seed": 1729,
        "replay_eviction_controller_state_dim": 32, "replay_eviction_controller_rank": 8,
        "replay_eviction_controller_dt": 1.0, "replay_eviction_controller_gamma": 0.08,
        "replay_eviction_controller_target_log_sv": -0.05,
        "replay_eviction_controller_max_state_norm": 8.0,
        "replay_eviction_controller_perturbation_scale": 0.25,
        "replay_eviction_controller_feedback_lr": 0.05,
        "replay_eviction_commit_policy": "learned", "replay_eviction_commit_online_lr": 0.05,
        "replay_eviction_commit_temperature": 0.75,
        "replay_eviction_evidence_engine_enabled": True,
        "replay_eviction_evidence_engine_d_model": EXP26_MODEL_DIM,
        "replay_eviction_probe_buffer_size": 32, "replay_eviction_frame_ttl_steps": 256,
        "replay_eviction_slot_work_chunk_size": 4, "replay_eviction_trace_max_rows": 200_000,
        "replay_eviction_trace_flush_rows": 256,
    }


def build_validation_matrix(*, speed_config: Mapping[str, Any], world_size: int = 4,
                            budget_seconds: float = 45.0, seed: int = 1337,
                            trace_dir: Path | str = DEFAULT_VALIDATION_TRACE_DIR) -> list[dict[str, Any]]:
    """Control + full-stack cell (exp26.py:213-274).  Runs that turn the native maintenance
    scheduler on get their own shared-memory namespace, the run name."""
    trace_dir = Path(trace_dir)
    seed = int(seed)
    full = {**_crct_lock(trace_dir), **_pipeline_lock(), "replay_eviction_mode": "active",
            "replay_eviction_action_agreement_count": 1,
            "replay_eviction_trace_path":
                str(trace_dir / f"arm_validation_adaptive_residual_memory_s{seed}.ndjson")}
    entries = []
    for arm, overrides in zip(VALIDATION_ARMS, ({}, full)):
        entry = _base_entry(speed_config=dict(speed_config), world_size=world_size,
                            budget_seconds=budget_seconds)
        entry.update({"arm": arm, "artifact_impact": ARTIFACT_CHANGES_WEIGHTS_ONLY, **_size_lock(),
                      **_fast_slow_lock(trace_dir), **overrides})
        entry.pop("fast_slow_interval", None)
        name = f"exp26_validation_{arm}_s{seed}"
        entry.update({"name": name, "seed": seed, "exp26_phase": "validation", "exp26_mechanism": "arm_v1"})
        if entry.get("replay_eviction_arm_runtime_enabled"):
            entry["replay_eviction_arm_runtime_namespace"] = name
        entries.append(copy.deepcopy(entry))
    return entries


def run_validation(*, speed_config: Mapping[str, Any], world_size: int = 4, seed: int = 1337, budget_seconds: float = 45.0,
                   data_path: Path | str = "data", sp_model_path: Optional[Path | str] = None,
                   output_dir: Path | str = DEFAULT_VALIDATION_DIR, trace_dir: Optional[Path | str] = None,
                   dry_run: bool = False, say=print) -> dict[str, Any]:
    """The fixed two-cell validation run (run_exp26.py:49-108 of the reference): build, print, and unless
    ``dry_run`` (which touches nothing on disk) write ``matrix.json`` and launch both cells."""
    output_dir = Path(output_dir)
    entries = build_validation_matrix(speed_config=speed_config, world_size=int(world_size), seed=int(seed),
                                      budget_seconds=float(budget_seconds),
                                      trace_dir=Path(trace_dir) if trace_dir is not None else output_dir / "traces")
    say(f"[exp26] validation entries={len(entries)} world_size={world_size} budget={budget_seconds}s dry_run={dry_run}")
    if dry_run:
        for e in entries:
            say(f"[exp26] {e['name']}")
            say(json.dumps(e, indent=2, sort_keys=True, default=str))
        return {"entries": entries, "commands": []}
    from .fast_path import write_matrix
    from .launch import run_matrix
    output_dir.mkdir(parents=True, exist_ok=True)
    write_matrix(output_dir / "matrix.json", entries)
    summary = run_matrix(entries, results_dir=output_dir, data_path=str(data_path),
                         sp_model_path=None if sp_model_path is None else str(sp_model_path), world_size=int(world_size))
    return {"entries": entries, **summary}


def main(argv: Optional[Sequence[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", type=Path, default=None, help="speed config (YAML / JSON); empty when omitted")
    ap.add_argument("--data-path", type=Path, default=Path("data"))
    ap.add_argument("--sp-model-path-16384", "--sp-model-path", dest="sp_model_path", type=Path, default=None)
    ap.add_argument("--world-size", type=int, default=4)
    ap.add_argument("--budget", type=float, default=45.0, help="wall budget per validation cell (seconds)")
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("--output-dir", type=Path, default=DEFAULT_VALIDATION_DIR)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    from .fast_path import read_speed_config
    run_validation(speed_config=read_speed_config(a.config) if a.config else {}, world_size=a.world_size, seed=a.seed,
                   budget_seconds=a.budget, data_path=a.data_path, sp_model_path=a.sp_model_path, output_dir=a.output_dir,
                   dry_run=a.dry_run)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
