"""Append-only NDJSON writers for the episodic-memory research path: one row per
replay event and one row per action-space intervention (behaviour of
src/chaoscontrol/episodic/diagnostics.py:99-359).

Rows are validated against a pinned column list (a missing or unknown column is a
``KeyError``: schema drift is a bug, not a runtime condition), written in that
order, one JSON object per line, with NaN / inf mapped to ``null`` so a columnar
reader types the column as numeric.  Files are opened in append mode so a
relaunch keeps earlier rows.
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Any

__all__ = ["REPLAY_LOG_SCHEMA", "ACTION_SPACE_TRACE_SCHEMA", "DiagnosticsLogger", "ActionSpaceTraceLogger"]

REPLAY_LOG_SCHEMA: tuple[str, ...] = (
    # replay event
    "step", "slot", "key_fp", "write_step", "write_pressure", "write_bucket", "query_cosine", "utility_pre",
    "replay_id", "query_event_id", "source_write_id", "selection_step", "policy_version", "selected_rank",
    "teacher_score", "controller_logit", "replay_loss", "ce_before_replay", "ce_after_replay", "ce_delta_raw",
    "bucket_baseline", "reward_shaped", "replay_grad_norm", "replay_grad_cos_common", "replay_grad_cos_rare",
    "replay_grad_cos_total", "utility_signal_raw", "utility_signal_transformed", "utility_post",
    "outcome_status", "flags",
    # simplex-policy telemetry (full 16-vertex distributions for off-policy analysis)
    "arm", "chosen_idx", "p_chosen", "p_behavior", "entropy", "gerber_weight", "advantage_raw",
    "advantage_corrected", "lambda_hxh", "feature_manifest_hash", "candidate_slot_ids", "candidate_scores",
    "logits")

ACTION_SPACE_TRACE_SCHEMA: tuple[str, ...] = (
    "gpu_step", "event_type", "head_name", "raw_action_json", "bounded_action_json", "invariant_name",
    "clamp_amount", "readiness", "reward_context_json", "accepted")

_ACTION_INPUT = ("gpu_step", "event_type", "head_name", "raw_action", "bounded_action", "invariant_name",
                 "clamp_amount", "readiness", "reward_context", "accepted")


def _plain(value: Any) -> Any:
    """JSON-ready form of a logged value: tensors / numpy scalars through ``.item()``,
    non-finite floats to ``None``, containers element-wise."""
    if value is None or isinstance(value, (bool, int, str)):
        return value
    if isinstance(value, float):
        return value if math.isfinite(value) else None
    if isinstance(value, dict):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    tolist = getattr(value, "tolist", None)
    if callable(tolist):
        try:
            return _plain(tolist())
        except Exception:
            return value
    item = getattr(value, "item", None)
    if callable(item):
        try:
            return _plain(item())
        except Exception:
            return value
    return value


def _check(row: dict, expected: tuple[str, ...], who: str) -> None:
    keys = set(row)
    missing = sorted(set(expected) - keys)
    if missing:
        raise KeyError(f"{who} row missing columns: {missing}")
    extra = sorted(keys - set(expected))
    if extra:
        raise KeyError(f"{who} row has unknown columns: {extra}; the schema is pinned to {expected}")


class _NdjsonWriter:
    __slots__ = ("path", "_fh")

    def __init__(self, path: Path | str) -> None:
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self._fh = self.path.open("a", encoding="utf-8")

    def _emit(self, ordered: dict[str, Any]) -> None:
        self._fh.write(json.dumps(ordered) + "\n")

    def flush(self) -> None:
        self._fh.flush()

    def close(self) -> None:
        if not self._fh.closed:
            self._fh.flush()
            self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()

    def __del__(self) -> None:  # pragma: no cover - interpreter shutdown order varies
        try:
            self.close()
        except Exception:
            pass


class DiagnosticsLogger(_NdjsonWriter):
    """Per-rank replay log (``run_dir/episodic_replay_log_rank{R}.ndjson``)."""
    __slots__ = ()

    def write_row(self, row: dict[str, Any]) -> None:
        _check(row, REPLAY_LOG_SCHEMA, "DiagnosticsLogger")
        self._emit({c: _plain(row[c]) for c in REPLAY_LOG_SCHEMA})


class ActionSpaceTraceLogger(_NdjsonWriter):
    """Sink for ``ConstrainedActionSpace`` interventions; nested actions are stored
    as compact JSON strings so every column is a scalar."""
    __slots__ = ()

    def append(self, row: dict[str, Any]) -> None:
        _check(row, _ACTION_INPUT, "ActionSpaceTraceLogger")
        blob = lambda v: json.dumps(_plain(v), separators=(",", ":"))
        self._emit({
            "gpu_step": int(row["gpu_step"]), "event_type": str(row["event_type"]),
            "head_name": str(row["head_name"]), "raw_action_json": blob(row["raw_action"]),
            "bounded_action_json": blob(row["bounded_action"]), "invariant_name": str(row["invariant_name"]),
            "clamp_amount": _plain(float(row["clamp_amount"])), "readiness": _plain(float(row["readiness"])),
            "reward_context_json": blob(row["reward_context"]), "accepted": bool(row["accepted"])})
