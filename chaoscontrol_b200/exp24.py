"""Run-matrix builders for the training-time mechanism bundle.

Every builder returns a list of flat config dicts, one per (arm, seed), that
``runner_fast_path.run_condition`` / ``run_matrix`` consume.  The builder
names, arm names, run names and locked hyper-parameters follow the reference
(experiments/24_training_time_bundle/exp24.py:1-1727) so result files from
either framework line up; the construction here is table driven: an arm is a
``(label, overrides)`` pair, shared settings are frozen "lock" mappings
composed with ``|``, and one expander (`_expand`) does the base-entry
normalisation, the seed fan-out and the naming for all twenty builders.
"""
from __future__ import annotations

import copy
import os
import statistics
from types import MappingProxyType
from typing import Any, Callable, Iterable, Mapping, Sequence

DEFAULT_CONTROL_SEEDS = (1337, 2674, 4011)
ARTIFACT_CHANGES_WEIGHTS_ONLY = "artifact_changes_weights_only"
ARTIFACT_TRAINING_ONLY = "artifact_training_only"

# (dreamworld cache interval, dreamworld interval, dreamworld weight)
PHASE0_FASTSLOW_DW_CANDIDATES = ((16, 16, 0.10), (16, 16, 0.25), (8, 8, 0.10))
# (label, fast/slow interval, fast/slow alpha, dw cache interval, dw interval, dw weight)
PHASE0_CONFIRM_CONFIGS = (
    ("A", 32, 0.25, 16, 16, 0.10),
    ("B", 64, 0.25, 16, 16, 0.10),
)

EPISODIC_DW_CURATION_V1_ARMS: tuple[str, ...] = (
    "arm_a_uncurated", "arm_b_cosine_utility", "arm_bp_pressure_only", "arm_c_no_dw",
)
EPISODIC_DW_CURATION_V1_ESCALATION_ARMS: tuple[str, ...] = EPISODIC_DW_CURATION_V1_ARMS[:3]
EPISODIC_DW_CURATION_V1_ESCALATION_SEEDS: tuple[int, ...] = (5012, 7331, 9183)
EPISODIC_TTT_V1_ARMS: tuple[str, ...] = (
    "arm_a_no_cache_no_ttt", "arm_b_cache_train_ttt_with_cache",
    "arm_c_cache_train_no_ttt", "arm_d_no_cache_train_ttt_only",
)
EPISODIC_CONTROLLER_V1_ARMS: tuple[str, ...] = (
    "arm_a_control", "arm_b_heuristic", "arm_c_simplex_frozen",
    "arm_d_simplex_online", "arm_e_simplex_warm_online", "arm_f_simplex_sharp_online",
)
CRCT_V1_ARMS: tuple[str, ...] = (
    "arm_a_fastslow_control", "arm_b_crct_controller",
    "arm_c_crct_replay_shadow", "arm_d_crct_replay_active",
)
ARM_F_INITIAL_TEMPERATURE: float = 0.2
EPISODIC_CONTROLLER_V1_WEIGHTS_PATH = "TO_BE_FILLED/episodic_controller_v1_weights.pt"
EPISODIC_CONTROLLER_V1_WEIGHTS_PATH_ENV = "EPISODIC_CONTROLLER_V1_WEIGHTS_PATH"
EPISODIC_CONTROLLER_V1_TRACE_DIR = "experiments/24_training_time_bundle/results/traces"
EPISODIC_CONTROLLER_V1_TRACE_DIR_ENV = "EPISODIC_CONTROLLER_V1_TRACE_DIR"

_TRACE_ROOT = "experiments/24_training_time_bundle/results/traces"

# Keys every entry carries, with the type they are coerced to and the value
# used when the speed config does not set them (exp24.py:58-170).
_NORMALISED: tuple[tuple[str, Callable[[Any], Any], Any], ...] = (
    ("eval_batches", int, 0),
    ("train_sampling_mode", str, "random"),
    ("artifact_impact", str, ARTIFACT_CHANGES_WEIGHTS_ONLY),
    ("submit_valid", bool, True),
    ("fast_slow_enabled", bool, False),
    ("fast_slow_interval", int, 0),
    ("fast_slow_alpha", float, 0.0),
    ("fast_slow_eval_copy", str, "fast"),
    ("spectral_reg_lambda_dead", float, 0.0),
    ("spectral_reg_lambda_sticky", float, 0.0),
    ("spectral_reg_min_a", float, 0.05),
    ("spectral_reg_max_a", float, 0.98),
    ("predictive_aux_weight", float, 0.0),
    ("predictive_aux_horizon", int, 0),
    ("predictive_aux_dim", int, 0),
    ("dreamworld_enabled", bool, False),
    ("dreamworld_cache_interval", int, 0),
    ("dreamworld_interval", int, 0),
    ("dreamworld_weight", float, 0.0),
    ("dreamworld_prefix_tokens", int, 128),
    ("dreamworld_replay_tokens", int, 64),
    ("dreamworld_replay_batch_size", int, 0),
    ("dreamworld_buffer_size", int, 16),
    ("dreamworld_min_size", int, 2),
    ("dreamworld_max_age_steps", int, 256),
    ("event_sleep_enabled", bool, False),
    ("event_sleep_loss_ratio", float, 1.10),
    ("event_sleep_pressure_threshold", float, 0.05),
    ("event_sleep_ema_decay", float, 0.99),
    ("event_sleep_warmup_steps", int, 32),
    ("event_sleep_min_interval", int, 8),
    ("event_sleep_weight", float, 0.0),
    ("embed_freeze_steps", int, 0),
    ("semantic_layer_index", int, 0),
    ("semantic_momentum_min", float, 0.5),
    ("semantic_overhead_gate", float, 0.08),
    ("optimizer_param_grouping", str, "flat"),
    ("optimizer_dynamics_lr_mul", float, 0.1),
)


def _lock(**kv: Any) -> Mapping[str, Any]:
    return MappingProxyType(dict(kv))


_FS_SLOW = _lock(fast_slow_enabled=True, fast_slow_eval_copy="slow")
_FS_I32_A050 = _FS_SLOW | {"fast_slow_interval": 32, "fast_slow_alpha": 0.50}
_FS_I64_A025 = _FS_SLOW | {"fast_slow_interval": 64, "fast_slow_alpha": 0.25}
_DW_OFF = _lock(
    dreamworld_enabled=False, dreamworld_cache_interval=0, dreamworld_interval=0,
    dreamworld_weight=0.0, dreamworld_replay_batch_size=0,
)
_DW_BUFFER = _lock(
    dreamworld_enabled=True, dreamworld_prefix_tokens=128, dreamworld_replay_tokens=64,
    dreamworld_buffer_size=16, dreamworld_min_size=2, dreamworld_max_age_steps=256,
)
_EVENT_SLEEP = _lock(
    event_sleep_enabled=True, event_sleep_loss_ratio=1.10,
    event_sleep_pressure_threshold=0.05, event_sleep_ema_decay=0.99,
    event_sleep_warmup_steps=32, event_sleep_min_interval=8,
)
_SCOPT = _lock(
    scopt_warmup_steps=200, scopt_split_interval=4, scopt_trace_interval_steps=64,
    scopt_rare_ema_decay=0.9, scopt_rare_orthogonal_weight=1.0, scopt_rare_macro_c=0.5,
    scopt_pressure_upper_c=3.0, scopt_pressure_upper_floor=1.0,
    scopt_row_scarcity_power=0.5, scopt_tau_std_scale=0.5, scopt_layer_index=0,
    scopt_baseline_buckets=16, scopt_baseline_decay=0.99,
)
_EVAL_CACHE_SCHEMA = _lock(
    eval_episodic_cache_capacity=4096, eval_episodic_span_length=4,
    eval_episodic_key_rep_dim=-1, eval_episodic_grace_steps=1000,
    eval_episodic_fingerprint_window=8, eval_episodic_cache_reset_per_doc=False,
)
_CRITICALITY = _lock(
    lm_head_backward_mode="fused_streaming_cached", lm_head_emit_entropy=True,
    criticality_distill_enabled=True, criticality_distill_budget_frac=0.15,
    criticality_distill_critical_value=0.95,
    criticality_distill_trace_half_life_steps=256.0,
    criticality_distill_trace_ttl_steps=1024, criticality_distill_horizon_H=16,
    criticality_distill_event_frac=0.05, criticality_distill_seat_refresh_interval=64,
    criticality_distill_min_weighted_events_per_layer=256.0,
    criticality_distill_weight=1e-3, criticality_distill_uniform_pressure=False,
    criticality_distill_score_permute_before_topk=False,
    criticality_distill_fixed_random_seats=False,
    rare_bucket_ce_enabled=True, rare_bucket_ce_num_buckets=4,
)
_CRCT = _lock(
    crct_enabled=True, crct_lm_weight_alpha_max=0.15, crct_lm_weight_strength=0.10,
    crct_lm_weight_w_max=1.20, crct_lm_weight_tau=0.10, crct_target_read_rate=0.25,
    crct_target_write_rate=0.10, crct_dual_lr=0.01, crct_ema_beta=0.95,
    crct_max_price=0.50, crct_memory_write_tokens_per_step=128,
    crct_async_teacher_transport=True, crct_async_teacher_transport_backend="mailbox",
    crct_async_teacher_pending_batches=64, crct_async_teacher_max_lag_steps=128,
    crct_async_teacher_payload_dtype="auto", crct_teacher_score_interval_steps=64,
    crct_teacher_param_sync_interval_steps=0, outer_model_dim=64,
    outer_model_type="multislot", outer_max_slots=4096, outer_compress_ratio=2,
    buffer_mode="append_only", retrieval_mode="softmax_all", retrieval_k=16,
    train_sampling_mode="random", compile_full_path=False, cuda_graph_mode="none",
    crct_gradient_conflict_enabled=True, crct_gradient_conflict_soft_gate_strength=0.0,
    crct_gradient_conflict_trace_path=f"{_TRACE_ROOT}/crct_conflict.ndjson",
    crct_gradient_conflict_trace_max_rows=200_000,
)
_REPLAY_EVICTION = _lock(
    replay_eviction_enabled=True, bucket_prototypes=True, prototype_dim=64,
    replay_eviction_memory_streams=8, replay_eviction_oracle_confirm_top_k=32,
    replay_eviction_peak_preserve_utility_threshold=0.20,
    replay_eviction_peak_preserve_sharpness_threshold=0.20,
    replay_eviction_probe_buffer_size=32, replay_eviction_frame_ttl_steps=256,
    replay_eviction_slot_work_chunk_size=64, replay_eviction_action_agreement_count=2,
    replay_eviction_trace_path=f"{_TRACE_ROOT}/crct_replay_eviction.ndjson",
    replay_eviction_trace_max_rows=200_000,
)


def _dreamworld(cache_interval: int, interval: int, weight: float | None = None,
                *, sub: int | None = 128) -> dict[str, Any]:
    out = dict(_DW_BUFFER, dreamworld_cache_interval=cache_interval,
               dreamworld_interval=interval)
    if weight is not None:
        out["dreamworld_weight"] = weight
    if sub is not None:
        out["dreamworld_replay_batch_size"] = sub
    return out


def _pct(x: float) -> str:
    return f"{int(x * 100):03d}"


def _base_entry(*, speed_config: dict[str, Any], world_size: int,
                budget_seconds: float) -> dict[str, Any]:
    """Copy ``speed_config`` and pin the bundle's common keys to typed values
    (exp24.py:53-173): anything the speed config already sets is kept and
    coerced, anything missing gets the mechanism-off default."""
    entry = copy.deepcopy(speed_config)
    entry["mode"] = "exp24_training_time_bundle"
    entry["world_size"] = int(world_size)
    entry["budget_seconds"] = float(budget_seconds)
    for key, cast, default in _NORMALISED:
        entry[key] = cast(entry.get(key, default))
    return entry


def _named_entry(*, base: dict[str, Any], phase: str | None, mechanism: str,
                 arm: str, seed: int) -> dict[str, Any]:
    """Stamp name, seed, phase and mechanism onto a copy of ``base``
    (exp24.py:176-200).  A run without a phase belongs to the first wave and
    its name has no phase segment."""
    entry = copy.deepcopy(base)
    stem = f"exp24_{phase}_{arm}" if phase else f"exp24_{arm}"
    entry.update(name=f"{stem}_s{int(seed)}", seed=int(seed),
                 exp24_phase=phase if phase is not None else "first_wave",
                 exp24_mechanism=mechanism)
    return entry


def _select(arm_specs: list[tuple[str, dict[str, Any]]], arms: Sequence[str] | None,
            known: tuple[str, ...]) -> list[tuple[str, dict[str, Any]]]:
    if arms is None:
        return arm_specs
    wanted = set(arms)
    unknown = wanted - set(known)
    if unknown:
        raise ValueError(f"unknown arm(s) {sorted(unknown)}; allowed: {known}")
    return [(n, o) for n, o in arm_specs if n in wanted]


def _expand(speed_config: dict[str, Any], world_size: int, budget_seconds: float,
            arm_specs: Iterable[tuple[str, Mapping[str, Any]]], seeds: Iterable[int], *,
            phase: str | None, mechanism: str | None = None, common: Mapping[str, Any] | None = None,
            name_prefix: str = "",
            finish: Callable[[dict[str, Any], str, int], None] | None = None,
            ) -> list[dict[str, Any]]:
    """Arms × seeds → named entries.  ``common`` applies under each arm's own
    overrides; ``mechanism`` falls back to the arm's ``exp24_mechanism``;
    ``finish(entry, arm, seed)`` can patch per-run keys (trace paths)."""
    seeds = [int(s) for s in seeds]
    out: list[dict[str, Any]] = []
    for arm_name, overrides in arm_specs:
        for seed in seeds:
            entry = _base_entry(speed_config=speed_config, world_size=world_size,
                                budget_seconds=budget_seconds)
            entry.update(common or {})
            entry.update(overrides)
            named = _named_entry(
                base=entry, phase=phase,
                mechanism=mechanism or str(entry["exp24_mechanism"]),
                arm=f"{name_prefix}{arm_name}", seed=seed)
            if finish is not None:
                finish(named, arm_name, seed)
            out.append(named)
    return out


# ---------------------------------------------------------------------------
# controls, sampling and optimizer gates
# ---------------------------------------------------------------------------

def build_ring0_control_matrix(*, speed_config: dict[str, Any], world_size: int = 8,
                               budget_seconds: float = 600.0,
                               seeds: Sequence[int] = DEFAULT_CONTROL_SEEDS) -> list[dict[str, Any]]:
    """Seed-noise floor of the unmodified trainer (exp24.py:203-227)."""
    return _expand(speed_config, world_size, budget_seconds,
                   [("control", {"train_sampling_mode": "random"})], seeds,
                   phase="ring0", mechanism="control")


def build_phase_a_sampling_matrix(*, speed_config: dict[str, Any], world_size: int = 8,
                                  budget_seconds: float = 600.0,
                                  seeds: Sequence[int] = (1337,)) -> list[dict[str, Any]]:
    """Random vs sequential-epoch vs shuffled-epoch sampling (exp24.py:230-258)."""
    arms = [(p, {"train_sampling_mode": p})
            for p in ("random", "sequential_epoch", "shuffled_epoch")]
    return _expand(speed_config, world_size, budget_seconds, arms, seeds,
                   phase="phaseA", mechanism="sampling_policy")


def build_semantic_overhead_gate_matrix(*, speed_config: dict[str, Any], seed: int = 1337,
                                        world_size: int = 1,
                                        budget_seconds: float = 90.0) -> list[dict[str, Any]]:
    """Muon vs the semantic optimizer on one GPU: the throughput gate
    (exp24.py:261-293)."""
    arms = [(f"semantic_gate_{o}", {"optimizer": o}) for o in ("muon", "semantic")]
    return _expand(speed_config, world_size, budget_seconds, arms, [seed], phase="smoke",
                   mechanism="semantic_optimizer_gate",
                   common={"artifact_impact": ARTIFACT_CHANGES_WEIGHTS_ONLY})


def _scopt_common(batch_size: int) -> dict[str, Any]:
    return {"artifact_impact": ARTIFACT_CHANGES_WEIGHTS_ONLY, "batch_size": int(batch_size),
            "optimizer_param_grouping": "ssm_three_group", "optimizer_dynamics_lr_mul": 0.1}


def build_scopt_overhead_gate_matrix(*, speed_config: dict[str, Any], seed: int = 1337,
                                     world_size: int = 1, budget_seconds: float = 180.0,
                                     batch_size: int = 512) -> list[dict[str, Any]]:
    """Muon vs scarcity-aware optimizer with the three-group parameter split
    (exp24.py:296-356)."""
    arms = [("scopt_gate_muon", {"optimizer": "muon"}),
            ("scopt_gate_scopt", {"optimizer": "scopt", **_SCOPT})]
    return _expand(speed_config, world_size, budget_seconds, arms, [seed], phase="smoke",
                   mechanism="scopt_overhead_gate", common=_scopt_common(batch_size))


def build_scopt_calibration_sweep_matrix(*, speed_config: dict[str, Any], seed: int = 1337,
                                         world_size: int = 1, budget_seconds: float = 1200.0,
                                         batch_size: int = 512) -> list[dict[str, Any]]:
    """One-knob-at-a-time variants around the scarcity optimizer's defaults
    (exp24.py:359-426)."""
    variants = (("baseline_d95", {"scopt_baseline_decay": 0.95}),
                ("pressure_c15", {"scopt_pressure_upper_c": 1.5}),
                ("rare_ema_095", {"scopt_rare_ema_decay": 0.95}))
    arms = [(f"scopt_cal_{n}", o) for n, o in variants]
    return _expand(speed_config, world_size, budget_seconds, arms, [seed], phase="smoke",
                   mechanism="scopt_calibration_sweep",
                   common={**_scopt_common(batch_size), "optimizer": "scopt", **_SCOPT})


# ---------------------------------------------------------------------------
# first wave and phase 0
# ---------------------------------------------------------------------------

_FS_DW_ARM = ("fastslow_i32_a050_dreamworld_c8_i8_w025_sub128", {
    "exp24_mechanism": "fast_slow_dreamworld", "artifact_impact": ARTIFACT_TRAINING_ONLY,
    **_FS_I32_A050, **_dreamworld(8, 8, 0.25)})


def build_first_wave_mechanism_matrix(*, speed_config: dict[str, Any], world_size: int = 8,
                                      budget_seconds: float = 600.0,
                                      seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                                      ) -> list[dict[str, Any]]:
    """One arm per mechanism, each against the same control
    (exp24.py:429-560): fast/slow weights, spectral regulariser, predictive
    auxiliary loss, dream replay, and the two stacked variants."""
    train_only = {"artifact_impact": ARTIFACT_TRAINING_ONLY}
    arms = [
        ("fastslow_i32_a050", {"exp24_mechanism": "fast_slow", **train_only, **_FS_I32_A050}),
        ("spectral_dead1e-04_sticky1e-04", {
            "exp24_mechanism": "spectral", "artifact_impact": ARTIFACT_CHANGES_WEIGHTS_ONLY,
            "spectral_reg_lambda_dead": 1e-4, "spectral_reg_lambda_sticky": 1e-4}),
        ("predictive_h4_w010", {"exp24_mechanism": "predictive_aux", **train_only,
                                "predictive_aux_weight": 0.10, "predictive_aux_horizon": 4}),
        ("dreamworld_c4_i4_w025", {"exp24_mechanism": "dreamworld", **train_only,
                                   **_dreamworld(4, 4, 0.25, sub=None)}),
        _FS_DW_ARM,
        ("fastslow_i32_a050_dreamworld_eventsleep_r110_p005_sub128", {
            **_FS_DW_ARM[1], "exp24_mechanism": "fast_slow_dreamworld_event_sleep",
            **_EVENT_SLEEP}),
    ]
    return _expand(speed_config, world_size, budget_seconds, arms, seed_values, phase=None)


def build_first_wave_matrix(*, speed_config: dict[str, Any], world_size: int = 8,
                            budget_seconds: float = 600.0,
                            seeds: Sequence[int] = DEFAULT_CONTROL_SEEDS) -> list[dict[str, Any]]:
    """Alias of `build_first_wave_mechanism_matrix` with the older keyword
    (exp24.py:1689-1701)."""
    return build_first_wave_mechanism_matrix(
        speed_config=speed_config, world_size=world_size,
        budget_seconds=budget_seconds, seed_values=seeds)


def build_fastslow_dreamworld_matrix(*, speed_config: dict[str, Any], world_size: int = 8,
                                     budget_seconds: float = 600.0,
                                     seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                                     ) -> list[dict[str, Any]]:
    """Only the stacked fast/slow + dream-replay arm (exp24.py:563-607)."""
    return _expand(speed_config, world_size, budget_seconds, [_FS_DW_ARM], seed_values,
                   phase=None)


def _fs_dw_arm(prefix: str, fs_i: int, fs_a: float, c: int, i: int, w: float):
    return (f"{prefix}fs_i{fs_i}a{_pct(fs_a)}_dw_c{c}i{i}_w{_pct(w)}", {
        "exp24_mechanism": "fast_slow_dreamworld", "artifact_impact": ARTIFACT_TRAINING_ONLY,
        **_FS_SLOW, "fast_slow_interval": fs_i, "fast_slow_alpha": fs_a,
        **_dreamworld(c, i, w)})


def build_phase0_dreamworld_sweep(*, speed_config: dict[str, Any], world_size: int = 4,
                                  budget_seconds: float = 600.0,
                                  seed_values: Sequence[int] = (1337,)) -> list[dict[str, Any]]:
    """Dream interval × weight grid under fixed fast/slow i32 α0.5
    (exp24.py:610-668)."""
    arms = [_fs_dw_arm("", 32, 0.50, n, n, w) for n in (4, 8, 16) for w in (0.10, 0.25, 0.50)]
    return _expand(speed_config, world_size, budget_seconds, arms, seed_values, phase="phase0")


def build_phase0_fastslow_sweep(*, speed_config: dict[str, Any], world_size: int = 4,
                                budget_seconds: float = 600.0,
                                seed_values: Sequence[int] = (1337,)) -> list[dict[str, Any]]:
    """Fast/slow interval × alpha grid for each surviving dream setting
    (exp24.py:671-738)."""
    arms = [_fs_dw_arm("", fi, fa, c, i, w)
            for c, i, w in PHASE0_FASTSLOW_DW_CANDIDATES
            for fi in (16, 32, 64) for fa in (0.25, 0.50)]
    return _expand(speed_config, world_size, budget_seconds, arms, seed_values, phase="phase0")


def build_phase0_confirm(*, speed_config: dict[str, Any], world_size: int = 4,
                         budget_seconds: float = 600.0,
                         seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS) -> list[dict[str, Any]]:
    """Three-seed confirmation of the two phase-0 winners (exp24.py:741-800)."""
    arms = [_fs_dw_arm(f"confirm_{lab}_", fi, fa, c, i, w)
            for lab, fi, fa, c, i, w in PHASE0_CONFIRM_CONFIGS]
    return _expand(speed_config, world_size, budget_seconds, arms, seed_values, phase="phase0")


def build_phase0_fastslow_only_control(*, speed_config: dict[str, Any], world_size: int = 4,
                                       budget_seconds: float = 600.0,
                                       seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                                       ) -> list[dict[str, Any]]:
    """Fast/slow i64 α0.25 with dream replay off: the control the phase-3
    matrices are judged against (exp24.py:803-850)."""
    arm = ("control_fastslow_only_i64a025", {
        "exp24_mechanism": "fast_slow", "artifact_impact": ARTIFACT_TRAINING_ONLY,
        **_FS_I64_A025, **_DW_OFF})
    return _expand(speed_config, world_size, budget_seconds, [arm], seed_values, phase="phase0")


# ---------------------------------------------------------------------------
# phase 3: episodic memory, controller, test-time training, CRCT
# ---------------------------------------------------------------------------

def build_episodic_dw_curation_v1_matrix(*, speed_config: dict[str, Any], world_size: int = 4,
                                         budget_seconds: float = 600.0,
                                         seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                                         arms: Sequence[str] | None = None) -> list[dict[str, Any]]:
    """Does curating dream replay from the episodic cache beat uncurated
    replay?  Uncurated / cosine-utility query / pressure-only query / cache
    with replay weight 0 (exp24.py:874-1010)."""
    specs = _select([
        ("arm_a_uncurated", {"episodic_enabled": False, "dreamworld_weight": 0.10}),
        ("arm_b_cosine_utility", {"episodic_enabled": True, "controller_query_enabled": True,
                                  "dreamworld_weight": 0.10,
                                  "controller_query_mode": "cosine_utility_weighted"}),
        ("arm_bp_pressure_only", {"episodic_enabled": True, "controller_query_enabled": True,
                                  "dreamworld_weight": 0.10,
                                  "controller_query_mode": "pressure_only"}),
        ("arm_c_no_dw", {"episodic_enabled": True, "dreamworld_weight": 0.0}),
    ], arms, EPISODIC_DW_CURATION_V1_ARMS)
    common = {"exp24_mechanism": "episodic_dw_curation_v1",
              "artifact_impact": ARTIFACT_TRAINING_ONLY, **_FS_I64_A025, **_dreamworld(16, 16)}
    return _expand(speed_config, world_size, budget_seconds, specs, seed_values, phase="phase3",
                   mechanism="episodic_dw_curation_v1", common=common,
                   name_prefix="episodic_dw_curation_v1_")


def _resolve_episodic_controller_v1_weights_path() -> str:
    return os.environ.get(EPISODIC_CONTROLLER_V1_WEIGHTS_PATH_ENV,
                          EPISODIC_CONTROLLER_V1_WEIGHTS_PATH)


def _resolve_episodic_controller_v1_trace_dir() -> str:
    return os.environ.get(EPISODIC_CONTROLLER_V1_TRACE_DIR_ENV, EPISODIC_CONTROLLER_V1_TRACE_DIR)


def build_episodic_controller_v1_matrix(*, speed_config: dict[str, Any], world_size: int = 4,
                                        budget_seconds: float = 600.0,
                                        seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                                        ) -> list[dict[str, Any]]:
    """Heuristic vs learned simplex controller, frozen and online, cold and
    warm eval cache, plus a sharp-temperature variant (exp24.py:1050-1240).
    Weights path and trace directory come from the environment at call time."""
    no_cache = {**_EVAL_CACHE_SCHEMA, "eval_episodic_cache_enabled": False,
                "eval_steps_per_chunk": 0, "eval_adapt_set": "none",
                "eval_episodic_cache_mode": "none"}
    cold = {**no_cache, "eval_episodic_cache_enabled": True, "eval_episodic_cache_mode": "cold"}
    warm = {**cold, "eval_episodic_cache_mode": "warm", "eval_episodic_cache_source": "checkpoint"}
    heuristic = {"episodic_controller_runtime": "heuristic", "controller_train_online": False}
    frozen = {"episodic_controller_runtime": "simplex_v1",
              "episodic_controller_weights_path": _resolve_episodic_controller_v1_weights_path(),
              "episodic_controller_selection_mode": "sample",
              "controller_train_online": False, "episodic_compute_replay_ce_pair": True}
    online = {**frozen, "controller_train_online": True, "episodic_controller_entropy_beta": 0.05}

    def on(event_log: bool) -> dict[str, Any]:
        return {"episodic_enabled": True, "controller_query_enabled": True,
                "episodic_event_log_enabled": event_log}

    specs = [
        ("arm_a_control", {"episodic_enabled": False, "controller_query_enabled": False,
                           "episodic_event_log_enabled": False, **heuristic, **no_cache}),
        ("arm_b_heuristic", {**on(False),
                             "episodic_controller_score_mode": "cosine_utility_weighted",
                             **heuristic, **cold}),
        ("arm_c_simplex_frozen", {**on(True), **frozen, **cold}),
        ("arm_d_simplex_online", {**on(True), **online, **cold}),
        ("arm_e_simplex_warm_online", {**on(True), **online, **warm}),
        ("arm_f_simplex_sharp_online", {
            **on(True), **online,
            "episodic_controller_initial_temperature": ARM_F_INITIAL_TEMPERATURE, **cold}),
    ]
    specs = [(n, {"arm": n, **o}) for n, o in specs]
    trace_dir = _resolve_episodic_controller_v1_trace_dir()

    def finish(entry: dict[str, Any], arm: str, seed: int) -> None:
        if entry.get("episodic_enabled"):
            # the memory rank takes no shard: epoch sharding would drop one
            entry["train_sampling_mode"] = "random"
        if "simplex" in arm:
            entry["episodic_controller_simplex_trace_path"] = (
                f"{trace_dir}/episodic_controller_v1_{arm}_s{seed}.ndjson")

    common = {"exp24_mechanism": "episodic_controller_v1",
              "artifact_impact": ARTIFACT_TRAINING_ONLY, **_FS_I64_A025, **_DW_OFF}
    return _expand(speed_config, world_size, budget_seconds, specs, seed_values, phase="phase3",
                   mechanism="episodic_controller_v1", common=common,
                   name_prefix="episodic_controller_v1_", finish=finish)


def build_episodic_ttt_v1_matrix(*, speed_config: dict[str, Any], world_size: int = 4,
                                 budget_seconds: float = 600.0,
                                 seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                                 arms: Sequence[str] | None = None) -> list[dict[str, Any]]:
    """2×2 of {cache-curated training, none} × {LM-head test-time training
    with the eval cache, none} (exp24.py:1243-1379)."""
    cache_train = {**_dreamworld(16, 16, 0.10), "episodic_enabled": True,
                   "controller_query_enabled": True,
                   "controller_query_mode": "cosine_utility_weighted"}
    no_cache_train = dict(_DW_OFF)
    no_ttt = {**_EVAL_CACHE_SCHEMA, "eval_episodic_cache_enabled": False,
              "eval_steps_per_chunk": 0, "eval_adapt_set": "none"}
    ttt = {**_EVAL_CACHE_SCHEMA, "eval_episodic_cache_enabled": True,
           "eval_steps_per_chunk": 1, "eval_adapt_set": "lm_head"}
    specs = _select([
        ("arm_a_no_cache_no_ttt", {**no_cache_train, **no_ttt}),
        ("arm_b_cache_train_ttt_with_cache", {**cache_train, **ttt}),
        ("arm_c_cache_train_no_ttt", {**cache_train, **no_ttt}),
        ("arm_d_no_cache_train_ttt_only", {**no_cache_train, **ttt}),
    ], arms, EPISODIC_TTT_V1_ARMS)
    common = {"exp24_mechanism": "episodic_ttt_v1", "artifact_impact": ARTIFACT_TRAINING_ONLY,
              **_FS_I64_A025}
    return _expand(speed_config, world_size, budget_seconds, specs, seed_values, phase="phase3",
                   mechanism="episodic_ttt_v1", common=common, name_prefix="episodic_ttt_v1_")


def build_crct_v1_matrix(*, speed_config: dict[str, Any], world_size: int = 4,
                         budget_seconds: float = 600.0,
                         seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS,
                         arms: Sequence[str] | None = None) -> list[dict[str, Any]]:
    """Cache-reweighted continuation training on top of fixed fast/slow:
    control, teacher + controller, and replay eviction in shadow and active
    mode (exp24.py:1382-1527).  Every arm samples randomly because the last
    rank is the memory coprocessor and holds no data shard."""
    specs = _select([
        ("arm_a_fastslow_control", {}),
        ("arm_b_crct_controller", dict(_CRCT)),
        ("arm_c_crct_replay_shadow", {**_CRCT, **_REPLAY_EVICTION,
                                      "replay_eviction_mode": "shadow"}),
        ("arm_d_crct_replay_active", {**_CRCT, **_REPLAY_EVICTION,
                                      "replay_eviction_mode": "active"}),
    ], arms, CRCT_V1_ARMS)
    specs = [(n, {"arm": n, **o}) for n, o in specs]

    def finish(entry: dict[str, Any], arm: str, seed: int) -> None:
        if entry.get("replay_eviction_enabled"):
            entry["replay_eviction_trace_path"] = (
                f"{_TRACE_ROOT}/crct_replay_eviction_{arm}_s{seed}.ndjson")

    common = {"exp24_mechanism": "crct_v1", "artifact_impact": ARTIFACT_CHANGES_WEIGHTS_ONLY,
              **_FS_I64_A025, **_DW_OFF, "train_sampling_mode": "random"}
    return _expand(speed_config, world_size, budget_seconds, specs, seed_values, phase="phase3",
                   mechanism="crct_v1", common=common, name_prefix="crct_v1_", finish=finish)


# ---------------------------------------------------------------------------
# criticality distillation
# ---------------------------------------------------------------------------

_CD_CELLS = (
    ("treatment", {}),
    ("telemetry", {"criticality_distill_weight": 0.0}),
    ("shuffled", {"criticality_distill_score_permute_before_topk": True}),
    ("budget_only", {"criticality_distill_fixed_random_seats": True}),
    ("hl_short", {"criticality_distill_trace_half_life_steps": 128.0}),
    ("hl_long", {"criticality_distill_trace_half_life_steps": 512.0}),
    ("H_short", {"criticality_distill_horizon_H": 8}),
    ("H_long", {"criticality_distill_horizon_H": 32}),
)


def _criticality_matrix(speed_config, world_size, budget_seconds, seeds, phase, cells):
    common = {"exp24_mechanism": "fast_slow", "artifact_impact": ARTIFACT_TRAINING_ONLY,
              **_FS_I64_A025, **_DW_OFF, **_CRITICALITY}
    wanted = [(n, o) for n, o in _CD_CELLS if n in cells]
    return _expand(speed_config, world_size, budget_seconds, wanted, seeds, phase=phase,
                   mechanism="fast_slow", common=common)


def build_criticality_distillation_first_smoke_matrix(
        *, speed_config: dict[str, Any], world_size: int = 1, budget_seconds: float = 600.0,
        seed_values: Sequence[int] = DEFAULT_CONTROL_SEEDS) -> list[dict[str, Any]]:
    """Treatment, three falsifier controls (telemetry-only, shuffled scores,
    fixed random seats) and four half-life / horizon variants
    (exp24.py:1530-1609)."""
    return _criticality_matrix(speed_config, world_size, budget_seconds, seed_values,
                               "cd_first_smoke", {n for n, _ in _CD_CELLS})


def build_criticality_distillation_multiseed_matrix(
        *, speed_config: dict[str, Any], world_size: int = 1, budget_seconds: float = 600.0,
        seed_values: Sequence[int] = (1337, 17, 42, 1234, 2024)) -> list[dict[str, Any]]:
    """Five-seed rerun of the cells that mattered in the first smoke
    (exp24.py:1612-1686)."""
    return _criticality_matrix(
        speed_config, world_size, budget_seconds, seed_values, "cd_multiseed",
        {"treatment", "telemetry", "shuffled", "budget_only", "H_short"})


# ---------------------------------------------------------------------------
# result summaries
# ---------------------------------------------------------------------------

def summarize_control_noise(results: list[dict[str, Any]]) -> dict[str, Any]:
    """Seed-to-seed spread of the control runs: the yardstick a mechanism's
    bpb delta is compared with (exp24.py:1704-1727)."""
    seeds, bpb, elapsed, tps = [], [], [], []
    for row in results:
        seeds.append(int(row.get("config", {}).get("seed")))
        bpb.append(float(row.get("eval", {}).get("bpb")))
        elapsed.append(float(row.get("train", {}).get("elapsed_s")))
        tps.append(float(row.get("train", {}).get("aggregate_tokens_per_sec")))
    return {
        "count": len(seeds),
        "seeds": seeds,
        "bpb_mean": float(statistics.fmean(bpb)),
        "bpb_sample_std": float(statistics.stdev(bpb)) if len(bpb) > 1 else 0.0,
        "bpb_min": float(min(bpb)),
        "bpb_max": float(max(bpb)),
        "elapsed_s_mean": float(statistics.fmean(elapsed)),
        "tokens_per_sec_mean": float(statistics.fmean(tps)),
    }


MATRIX_BUILDERS: dict[str, Callable[..., list[dict[str, Any]]]] = {
    name[len("build_"):]: fn for name, fn in list(globals().items())
    if name.startswith("build_") and callable(fn)
}


def main(argv: Sequence[str] | None = None) -> int:
    """``python -m chaoscontrol_b200.exp24 <matrix> --speed-config cfg.yaml
    [--out matrix.json]``: write (or print the names of) one matrix."""
    import argparse
    import json

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("matrix", choices=sorted(MATRIX_BUILDERS))
    ap.add_argument("--speed-config", default=None)
    ap.add_argument("--world-size", type=int, default=None)
    ap.add_argument("--budget-seconds", type=float, default=None)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    speed: dict[str, Any] = {}
    if args.speed_config:
        import yaml
        with open(args.speed_config) as fh:
            speed = yaml.safe_load(fh) or {}
    kw: dict[str, Any] = {"speed_config": speed}
    if args.world_size is not None:
        kw["world_size"] = args.world_size
    if args.budget_seconds is not None:
        kw["budget_seconds"] = args.budget_seconds
    entries = MATRIX_BUILDERS[args.matrix](**kw)
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(entries, fh, indent=1)
    for e in entries:
        print(e["name"])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
